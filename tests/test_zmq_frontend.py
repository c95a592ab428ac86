"""Workers of the UNMODIFIED reference train against servers of this framework through the ZeroMQ front end
(kraken_b200/runtime/zmq_frontend.py): its worker library, its wire format, this package's scheduler_server and
ps_server behind it.  Needs the offline reference build and pyzmq; skipped where either is absent."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from test_reference_checkpoint_compat import REF, ROOT

pytest.importorskip("zmq")
pytestmark = pytest.mark.skipif(
    not (os.path.exists(os.path.join(REF, "bin", "ps_server")) and os.path.exists(os.path.join(REF, "kraken_native.so"))),
    reason="the reference is not built here (python baseline/build_reference.py)")


class Deployment:
    """This package's scheduler + n servers (threads of the test process) and a front end before them."""

    def __init__(self, saved_dir: str, n_ps: int = 2):
        from kraken_b200.runtime.remote import PsServer, SchedulerServer
        from kraken_b200.runtime.zmq_frontend import ZmqFrontend
        self.sched = SchedulerServer(0)
        self.sched.start()
        self.servers = []
        for _ in range(n_ps):
            ps = PsServer(0, "", f"127.0.0.1:{self.sched.port}", saved_dir=saved_dir, seed=5)
            ps.addr = f"127.0.0.1:{ps.port}"
            ps.start()
            self.servers.append(ps)
        self.front = ZmqFrontend(f"127.0.0.1:{self.sched.port}")
        self.front.start()
        self.env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(REF, "lib") + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
        self.env.pop("PYTHONPATH", None)
        self.s_addr = f"127.0.0.1:{self.front.port}"

    def reference_worker(self, script: str, *args: str) -> None:
        run = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", script), "--ref-path", REF, "--s-addr",
                              self.s_addr, *args], env=self.env, capture_output=True, text=True, timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]

    def stop(self):
        self.front.stop()
        self.sched.stop()
        for s in self.servers:
            s.stop()


def test_reference_worker_trains_against_these_servers(tmp_path):
    """baseline/dropin_train.py with ``kraken.pytorch`` = the reference's worker library, pointed at the front end:
    CombineEmbedding pulls and pushes, dense pushes from gradient hooks, dense pulls in ``step()``.  The losses
    equal those of the same script on this framework's own engine (which equal the reference's own servers',
    tests/test_reference_oracle.py)."""
    dep = Deployment(str(tmp_path / "ckpt"))
    try:
        out = str(tmp_path / "via_frontend.npz")
        dep.reference_worker("dropin_train.py", "--impl", "reference", "--out", out)
        rows = sum(s.shard.sparse_size(t) for s in dep.servers for t in (0, 1))
        assert rows > 0 and all(s.shard.sparse_size(0) > 0 for s in dep.servers)      # both servers hold rows
    finally:
        dep.stop()
    ours = str(tmp_path / "ours.npz")
    env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    run = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "dropin_train.py"), "--impl", "ours", "--s-addr",
                          "cpu", "--out", ours], env=env, capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
    a, b = dict(np.load(out)), dict(np.load(ours))
    assert a["losses"][0] > a["losses"][-1]
    assert np.allclose(a["losses"], b["losses"], rtol=1e-4, atol=1e-5), (a["losses"], b["losses"])
    for k in range(6):
        assert np.allclose(a[f"param_{k}"], b[f"param_{k}"], rtol=1e-3, atol=1e-5), k


def test_reference_worker_saves_a_checkpoint_on_these_servers(tmp_path):
    """The reference's worker registers tables, pushes (Adam with amsgrad) and asks for a checkpoint through the
    front end; the files these servers write load into a fresh engine with the values the worker saw, and the
    next update continues from the saved moments."""
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    dep = Deployment(str(ckpt))
    try:
        out = str(tmp_path / "worker.npz")
        dep.reference_worker("ref_checkpoint_worker.py", "--mode", "save", "--out", out)
    finally:
        dep.stop()
    want = dict(np.load(out))
    from kraken_b200.checkpoint.manager import load_model
    from kraken_b200.runtime.cpu_engine import CpuEngine
    from kraken_b200.runtime.engine import EngineConfig
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_checkpoint_worker as w
    finally:
        sys.path.pop(0)
    ids = w.ids_of()
    g2, d2 = w.grads(2, ids.numel())
    eng = CpuEngine(EngineConfig(backend="cpu", seed=1), 0, 1)
    try:
        assert load_model(eng, str(ckpt))
        ts, td = (int(x) for x in want["table_ids"])
        assert np.array_equal(eng.pull_sparse_table(ts, ids).numpy(), want["rows_at_save"])
        assert np.array_equal(eng.pull_dense_table(td).numpy(), want["dense_at_save"])
        eng.update_lr(w.LR)
        eng.push_sparse_table(ts, ids, g2)
        eng.push_dense_table(td, d2)
        assert np.allclose(eng.pull_sparse_table(ts, ids).numpy(), want["rows_after"], rtol=1e-5, atol=1e-6)
        assert np.allclose(eng.pull_dense_table(td).numpy(), want["dense_after"], rtol=1e-5, atol=1e-6)
    finally:
        eng.stop()


def test_reference_dct_emitter_pushes_through_the_front_end(tmp_path):
    """The reference's DCT emitter sends COO gradients (kraken/worker/dct_emitter.cc:16-43); behind the front end the
    tables must end up where this framework's own DCT path puts them (which equals the reference's servers,
    tests/test_reference_oracle.py)."""
    import kraken_b200.pytorch as kk
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_dct_worker as w
    finally:
        sys.path.pop(0)
    dep = Deployment(str(tmp_path / "ckpt"), n_ps=1)
    try:
        out = str(tmp_path / "dct.npz")
        dep.reference_worker("ref_dct_worker.py", "--out", out)
    finally:
        dep.stop()
    got = dict(np.load(out))
    kk.initialize("cpu", kk.EmitterType.kDCT, w.LIFE_SPAN, w.ETA)
    try:
        kk.init_model("dct", kk.OptimType.kSGD, {})
        kk.update_lr(w.LR)
        tb = kk.register_dense_table("big", torch.zeros(*w.BIG))
        ts = kk.register_dense_table("small", torch.zeros(*w.SMALL))
        for k, (gb, gs) in enumerate(w.inputs()):
            kk.push_dense_table(tb, gb)
            kk.push_dense_table(ts, gs)
            assert np.allclose(kk.pull_dense_table(tb).numpy(), got[f"big_{k}"], atol=1e-6), k
            assert np.allclose(kk.pull_dense_table(ts).numpy(), got[f"small_{k}"], atol=1e-6), k
    finally:
        kk.stop()

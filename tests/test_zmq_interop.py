"""Interoperation with the reference over ITS wire protocol, both ways.

Workers of the UNMODIFIED reference train against servers of this framework through the ZeroMQ front end
(kraken_b200/runtime/zmq_frontend.py): its worker library, its wire format, this package's scheduler_server and
ps_server behind it.  And this framework's worker (``initialize("zmq://...")``, kraken_b200/runtime/zmq_client.py)
trains on the reference's own scheduler_server and ps_server processes.  Needs the offline reference build and
pyzmq; skipped where either is absent."""
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


def test_this_frameworks_worker_trains_on_the_references_servers(tmp_path):
    """The other direction: ``kk.initialize("zmq://...")`` puts this framework's worker (its deduplication, ring
    routing, retries) on a cluster of the reference's own scheduler_server and two ps_server processes.  The same
    training script gives the losses the reference's own worker gets on a cluster of the same kind."""
    from test_reference_checkpoint_compat import ReferenceCluster
    script = os.path.join(ROOT, "baseline", "dropin_train.py")
    outs = {}
    for impl in ("reference", "ours"):
        cluster = ReferenceCluster(str(tmp_path / f"scratch_{impl}"), n_ps=2)
        try:
            outs[impl] = str(tmp_path / f"{impl}.npz")
            if impl == "reference":
                cmd = [sys.executable, script, "--impl", "reference", "--ref-path", REF, "--s-addr", cluster.s_addr, "--out", outs[impl]]
                env = cluster.env
            else:
                cmd = [sys.executable, script, "--impl", "ours", "--s-addr", "zmq://" + cluster.s_addr, "--out", outs[impl]]
                env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
            run = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
            assert run.returncode == 0, (impl, (run.stdout + run.stderr)[-3000:])
        finally:
            cluster.stop()
    a, b = dict(np.load(outs["reference"])), dict(np.load(outs["ours"]))
    assert np.allclose(a["losses"], b["losses"], rtol=1e-4, atol=1e-5), (a["losses"], b["losses"])
    for k in range(6):
        assert np.allclose(a[f"param_{k}"], b[f"param_{k}"], rtol=1e-3, atol=1e-5), k


def test_this_frameworks_api_on_the_references_servers(tmp_path):
    """Table by table through the public API against the reference's servers: dense and sparse pull / push, the
    combined calls, a DCT-compressed dense push, a checkpoint the reference writes."""
    import kraken_b200.pytorch as kk
    from test_reference_checkpoint_compat import ReferenceCluster
    saved = tmp_path / "ref_saved"
    saved.mkdir()
    cluster = ReferenceCluster(str(saved), n_ps=2)
    try:
        kk.initialize("zmq://" + cluster.s_addr, kk.EmitterType.kDCT, 2, 0.75)
        kk.init_model("api", kk.OptimType.kSGD, {})
        kk.update_lr(0.5)
        a = torch.randn(3, 4)
        td = kk.register_dense_table("w", a)
        tb = kk.register_dense_table("big", torch.zeros(20, 20))          # 400 elements: DCT compresses its gradient
        ts = kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        t2 = kk.register_sparse_table("f", 2, torch.float32, kk.InitializerType.kConstant, {"value": "-1.0"})
        assert kk.register_dense_table("w", a) == td
        assert torch.equal(kk.pull_dense_table(td), a)
        g = torch.randn(3, 4)
        kk.push_dense_table(td, g)
        assert torch.allclose(kk.pull_dense_table(td), a - 0.5 * g)
        ids = torch.arange(40).view(4, 10)
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.ones(4, 10, 3))
        kk.push_sparse_table(ts, torch.tensor([3, 3, 7]), torch.ones(3, 3))
        assert torch.allclose(kk.pull_sparse_table(ts, torch.tensor([3, 7, 8])), torch.tensor([[0.0] * 3, [0.5] * 3, [1.0] * 3]))
        r1, r2 = kk.combine_pull_sparse_table([ts, t2], [torch.tensor([3, 100]), torch.tensor([5, 6, 5])])
        assert torch.allclose(r1, torch.tensor([[0.0] * 3, [1.0] * 3])) and torch.equal(r2, -torch.ones(3, 2))
        kk.combine_push_sparse_table([ts, t2], [torch.tensor([100]), torch.tensor([5, 5])], [torch.ones(1, 3), torch.ones(2, 2)])
        assert torch.allclose(kk.pull_sparse_table(t2, torch.tensor([5, 6])), torch.tensor([[-2.0, -2.0], [-1.0, -1.0]]))
        d1, d2 = kk.combine_pull_dense_table([td, tb])
        assert torch.allclose(d1, a - 0.5 * g) and torch.equal(d2, torch.zeros(20, 20))
        gb = torch.randn(20, 20)
        kk.push_dense_table(tb, gb)                                         # travels as a COO gradient: top 25 % by magnitude
        moved = kk.pull_dense_table(tb)
        kept = moved != 0
        assert 0.2 < kept.float().mean() < 0.3 and torch.allclose(moved[kept], (-0.5 * gb)[kept])
        assert kk.try_save_model()
        from test_reference_checkpoint_compat import wait_for_checkpoint
        wait_for_checkpoint(str(saved), 2, table_files=("e.sparse", "f.sparse"))   # its servers write after they answer
        assert sorted(d for d in os.listdir(saved) if d.startswith("shard_")) == ["shard_0", "shard_1"]
    finally:
        kk.stop()
        cluster.stop()

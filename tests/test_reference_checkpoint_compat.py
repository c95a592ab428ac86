"""Checkpoints cross the border in both directions: files the UNMODIFIED reference writes load into this
framework, and files this framework writes load into the reference - values, optimizer state and step
counters (checked by one more Adam-amsgrad update on both sides).  Needs the offline reference build
(``python baseline/build_reference.py`` -> baseline/_ref); skipped where that is absent.
Layout and byte format: kraken/checkpoint/checkpoint.cc:17-23,446-510, kraken/checkpoint/checkpoint_exec.cc:246-521."""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

import kraken_b200.pytorch as kk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
WORKER = os.path.join(ROOT, "baseline", "ref_checkpoint_worker.py")
LR = 0.05

pytestmark = pytest.mark.skipif(
    not (os.path.exists(os.path.join(REF, "bin", "ps_server")) and os.path.exists(os.path.join(REF, "kraken_native.so"))),
    reason="the reference is not built here (python baseline/build_reference.py)")


def free_ports(n):
    socks = [socket.socket() for _ in range(n)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


class ReferenceCluster:
    """The reference's scheduler_server and n ps_server processes on localhost."""

    def __init__(self, saved_dir: str, n_ps: int = 2):
        self.env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(REF, "lib") + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
        self.env.pop("PYTHONPATH", None)
        ports = free_ports(1 + n_ps)
        self.s_addr = f"127.0.0.1:{ports[0]}"
        self.procs = [subprocess.Popen([os.path.join(REF, "bin", "scheduler_server"), f"--port={ports[0]}"], env=self.env,
                                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)]
        time.sleep(0.5)
        for k, p in enumerate(ports[1:]):
            # one request thread: a pull must not overtake the push in front of it
            self.procs.append(subprocess.Popen(
                [os.path.join(REF, "bin", "ps_server"), f"--port={p}", "--thread_nums=1", f"--addr=127.0.0.1:{p}",
                 f"--s_addr={self.s_addr}", f"--saved_dir={saved_dir}"], env=self.env,
                stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL))
            # the reference's scheduler takes one join at a time (a server that finds another join in flight backs
            # off for 10 s): the next server starts once this one is in the ring
            self._wait_for_servers(k + 1)
        assert all(p.poll() is None for p in self.procs), "a reference server exited at start-up"

    def _wait_for_servers(self, n_ps: int, timeout_s: float = 90.0) -> None:
        """Asks the reference's scheduler for its ring (over its own protocol) until ``n_ps`` servers have joined."""
        try:
            from kraken_b200.runtime.rpc import Rpc, RpcError
            from kraken_b200.runtime.zmq_client import ZmqConnecter
        except ImportError:           # no pyzmq: a fixed pause has to do
            time.sleep(2.0)
            return
        t0 = time.monotonic()
        while time.monotonic() - t0 < timeout_s:
            c = ZmqConnecter(self.s_addr, timeout_ms=2000)
            try:
                if len(c.call(Rpc.FETCH_ROUTER)[0]["nodes"]) >= n_ps:
                    return
            except RpcError:
                pass
            finally:
                c.close()
            time.sleep(0.5)
        raise AssertionError(f"the reference's scheduler did not see {n_ps} servers within {timeout_s} s")

    def worker(self, mode: str, out: str, load_dir: str = "", saved_dir: str = "", shards: int = 1) -> dict:
        run = subprocess.run([sys.executable, WORKER, "--ref-path", REF, "--s-addr", self.s_addr, "--mode", mode, "--dir",
                              load_dir, "--out", out, "--saved-dir", saved_dir, "--shards", str(shards)],
                             env=self.env, capture_output=True, text=True, timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
        return dict(np.load(out))

    def stop(self):
        for p in self.procs:
            p.terminate()
        for p in self.procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()


def wait_for_checkpoint(saved_dir, n_shards: int, table_files=("e.sparse",), timeout_s: float = 60.0) -> None:
    """The reference answers TrySaveModel once its servers have QUEUED the save (kraken/ps/ps.cc:487-520: the work
    runs on the server's task thread); the files appear a moment later.  Returns when every shard directory holds a
    complete set of files whose sizes have stopped changing."""
    def snapshot():
        sizes = {}
        shards = sorted(d for d in os.listdir(saved_dir) if d.startswith("shard_"))
        if len(shards) < n_shards:
            return None
        for d in shards:
            stamps = sorted(os.listdir(os.path.join(saved_dir, d)))
            if not stamps:
                return None
            last = os.path.join(saved_dir, d, stamps[-1])
            names = os.listdir(last)
            if not all(f in names for f in ("model.binary", "router.binary") + tuple(table_files)):
                return None
            for f in names:
                sizes[os.path.join(last, f)] = os.path.getsize(os.path.join(last, f))
        return sizes

    t0, before = time.monotonic(), None
    while time.monotonic() - t0 < timeout_s:
        now = snapshot()
        if now is not None and now == before:
            return
        before = now
        time.sleep(0.4)
    raise AssertionError(f"no complete checkpoint of {n_shards} shards under {saved_dir} within {timeout_s} s")


def worker_inputs():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_checkpoint_worker as w
    finally:
        sys.path.pop(0)
    ids = w.ids_of()
    return ids, w.grads(1, ids.numel()), w.grads(2, ids.numel())


def test_a_checkpoint_written_by_the_reference_loads_here(tmp_path):
    ref_dir = tmp_path / "written_by_reference"
    ref_dir.mkdir()
    cluster = ReferenceCluster(str(ref_dir))
    try:
        # the worker waits for the files before it pushes again: the reference writes a checkpoint AFTER it has
        # answered, and a push right behind the request could reach rows that are not written yet
        want = cluster.worker("save", str(tmp_path / "ref_save.npz"), saved_dir=str(ref_dir), shards=2)
        wait_for_checkpoint(str(ref_dir), 2)          # and before the servers are stopped under it
    finally:
        cluster.stop()
    assert sorted(d for d in os.listdir(ref_dir) if d.startswith("shard_")) == ["shard_0", "shard_1"]

    from kraken_b200.checkpoint.manager import load_model
    from kraken_b200.runtime.cpu_engine import CpuEngine
    from kraken_b200.runtime.engine import EngineConfig
    ids, _, (g2, d2) = worker_inputs()
    eng = CpuEngine(EngineConfig(backend="cpu", seed=1), 0, 1)
    try:
        assert load_model(eng, str(ref_dir))
        ts, td = (int(x) for x in want["table_ids"])
        assert eng.tables[ts].name == "e" and eng.tables[td].name == "w"
        assert np.array_equal(eng.pull_sparse_table(ts, ids).numpy(), want["rows_at_save"])
        assert np.array_equal(eng.pull_dense_table(td).numpy(), want["dense_at_save"])
        eng.update_lr(LR)
        eng.push_sparse_table(ts, ids, g2)
        eng.push_dense_table(td, d2)
        # one more Adam (amsgrad) update from the loaded moments and step counters
        assert np.allclose(eng.pull_sparse_table(ts, ids).numpy(), want["rows_after"], rtol=1e-5, atol=1e-6)
        assert np.allclose(eng.pull_dense_table(td).numpy(), want["dense_after"], rtol=1e-5, atol=1e-6)
    finally:
        eng.stop()


def test_a_checkpoint_written_here_loads_into_the_reference(tmp_path):
    from kraken_b200.runtime.remote import PsServer, SchedulerServer
    our_dir = tmp_path / "written_here"
    our_dir.mkdir()
    ids, (g1, d1), (g2, d2) = worker_inputs()
    sched = SchedulerServer(0)
    sched.start()
    servers = []
    for _ in range(2):
        ps = PsServer(0, "", f"127.0.0.1:{sched.port}", saved_dir=str(our_dir), seed=5)
        ps.addr = f"127.0.0.1:{ps.port}"
        ps.start()
        servers.append(ps)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        kk.init_model("ckpt", kk.OptimType.kAdam, {"amsgrad": "true"})
        kk.update_lr(LR)
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {"mean": "0.0", "stddev": "0.1"})
        td = kk.register_dense_table("w", torch.linspace(-1, 1, 15).view(5, 3))
        kk.pull_sparse_table(ts, ids)
        kk.push_sparse_table(ts, ids, g1)
        kk.push_dense_table(td, d1)
        rows_at_save = kk.pull_sparse_table(ts, ids).numpy()
        dense_at_save = kk.pull_dense_table(td).numpy()
        assert kk.try_save_model()
        kk.push_sparse_table(ts, ids, g2)
        kk.push_dense_table(td, d2)
        rows_after = kk.pull_sparse_table(ts, ids).numpy()
        dense_after = kk.pull_dense_table(td).numpy()
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()

    cluster = ReferenceCluster(str(tmp_path / "reference_scratch"))
    try:
        got = cluster.worker("load", str(tmp_path / "ref_load.npz"), load_dir=str(our_dir))
    finally:
        cluster.stop()
    assert np.array_equal(got["rows_at_save"], rows_at_save)
    assert np.array_equal(got["dense_at_save"], dense_at_save)
    assert np.allclose(got["rows_after"], rows_after, rtol=1e-5, atol=1e-6)
    assert np.allclose(got["dense_after"], dense_after, rtol=1e-5, atol=1e-6)

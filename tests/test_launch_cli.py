"""The deployment as the reference ships it: `scheduler_server` and `ps_server` as separate processes
(kraken/executable/scheduler_server_main.cc:5, kraken/executable/ps_server_main.cc:5-10), a worker that
reaches them through ``initialize("tcp://...")``."""
import os
import socket
import subprocess
import sys
import time

import torch

import kraken_b200.pytorch as kk
from kraken_b200.runtime.rpc import Connecter, Rpc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def wait_for(what, check, timeout_s=120.0):
    t0 = time.monotonic()
    while time.monotonic() - t0 < timeout_s:
        try:
            if check():
                return
        except (ConnectionError, OSError):
            pass
        time.sleep(0.2)
    raise AssertionError(f"{what} did not happen within {timeout_s} s")


def test_scheduler_and_two_ps_server_processes_serve_a_worker(tmp_path):
    env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    sp, p1, p2 = free_port(), free_port(), free_port()
    procs = [subprocess.Popen([sys.executable, "-m", "kraken_b200.launch.scheduler_server", "--port", str(sp)], env=env)]
    try:
        def scheduler_up():
            c = Connecter(f"127.0.0.1:{sp}", timeout_ms=1000)
            try:
                c.call(Rpc.FETCH_ROUTER)
                return True
            finally:
                c.close()

        wait_for("scheduler start", scheduler_up)
        for port in (p1, p2):
            procs.append(subprocess.Popen(
                [sys.executable, "-m", "kraken_b200.launch.ps_server", "--port", str(port), "--addr", f"127.0.0.1:{port}",
                 "--s_addr", f"127.0.0.1:{sp}", "--saved_dir", str(tmp_path), "--max_save_count", "2"], env=env))

        def both_joined():
            c = Connecter(f"127.0.0.1:{sp}", timeout_ms=1000)
            try:
                return len(c.call(Rpc.FETCH_ROUTER)[0]["nodes"]) == 2
            finally:
                c.close()

        wait_for("two servers joining", both_joined)
        assert all(p.poll() is None for p in procs), "a server process exited"

        kk.initialize(f"tcp://127.0.0.1:{sp}", compress=kk.CompressType.kDCT)      # Snappy bodies to the servers
        kk.init_model("cli", kk.OptimType.kAdagrad, {})
        kk.update_lr(0.1)
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        td = kk.register_dense_table("w", torch.ones(3, 2))
        ids = torch.arange(500)
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.ones(500, 4))
        for _ in range(3):
            kk.push_sparse_table(ts, ids, torch.full((500, 4), 2.0))
            kk.push_dense_table(td, torch.full((3, 2), 2.0))
        # Adagrad, g = 2 three times: w = 1 - 0.1 * 2 * (1/sqrt(4) + 1/sqrt(8) + 1/sqrt(12))
        want = 1.0 - 0.2 * (4 ** -0.5 + 8 ** -0.5 + 12 ** -0.5)
        assert torch.allclose(kk.pull_sparse_table(ts, ids), torch.full((500, 4), want), atol=1e-5)
        assert torch.allclose(kk.pull_dense_table(td), torch.full((3, 2), want), atol=1e-5)
        assert kk.try_save_model()
        shards = sorted(d for d in os.listdir(tmp_path) if d.startswith("shard_"))
        assert len(shards) == 2, shards
        for d in shards:
            stamp_dirs = os.listdir(tmp_path / d)
            assert len(stamp_dirs) == 1 and "e.sparse" in os.listdir(tmp_path / d / stamp_dirs[0])
    finally:
        kk.stop()
        for p in procs:
            p.terminate()
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()

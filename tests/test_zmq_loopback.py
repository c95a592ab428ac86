"""The two ZeroMQ halves against each other, without the reference: this package's worker speaking the reference's
wire protocol (kraken_b200/runtime/zmq_client.py) -> the front end (kraken_b200/runtime/zmq_frontend.py) -> this
package's scheduler and servers.  Every worker-facing message type crosses the codec in both directions
(kraken_b200/runtime/ref_wire.py); needs only pyzmq."""
import os

import pytest
import torch

import kraken_b200.pytorch as kk

pytest.importorskip("zmq")


def boot(tmp_path, n_ps=2):
    from kraken_b200.runtime.remote import PsServer, SchedulerServer
    from kraken_b200.runtime.zmq_frontend import ZmqFrontend
    sched = SchedulerServer(0)
    sched.start()
    servers = []
    for _ in range(n_ps):
        ps = PsServer(0, "", f"127.0.0.1:{sched.port}", saved_dir=str(tmp_path), seed=5)
        ps.addr = f"127.0.0.1:{ps.port}"
        ps.start()
        servers.append(ps)
    front = ZmqFrontend(f"127.0.0.1:{sched.port}")
    front.start()
    return sched, servers, front


def test_every_worker_message_crosses_the_codec_both_ways(tmp_path):
    sched, servers, front = boot(tmp_path)
    try:
        kk.initialize(f"zmq://127.0.0.1:{front.port}", kk.EmitterType.kDCT, 2, 0.75)
        kk.init_model("loop", kk.OptimType.kAdagrad, {"eps": "1e-6"})
        kk.update_lr(0.5)
        a = torch.randn(3, 4)
        td = kk.register_dense_table("w", a)
        tb = kk.register_dense_table("big", torch.zeros(20, 20))
        ts = kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        t2 = kk.register_sparse_table("f", 2, torch.float32, kk.InitializerType.kUniform, {"lower": "2.0", "upper": "2.0"})
        assert kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"}) == ts
        assert torch.equal(kk.pull_dense_table(td), a)
        g = torch.full((3, 4), 2.0)
        kk.push_dense_table(td, g)                                  # Adagrad: w -= lr * g / (sqrt(g^2) + eps)
        assert torch.allclose(kk.pull_dense_table(td), a - 0.5, atol=1e-5)
        ids = torch.tensor([[5, 9], [5, 1 << 40]])
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.ones(2, 2, 3))
        kk.push_sparse_table(ts, ids, torch.full((2, 2, 3), 1.0))   # id 5 occurs twice: gradients summed to 2
        rows = kk.pull_sparse_table(ts, torch.tensor([5, 9, 1 << 40]))
        assert torch.allclose(rows, torch.tensor([[0.5] * 3, [0.5] * 3, [0.5] * 3]), atol=1e-5)
        r1, r2 = kk.combine_pull_sparse_table([ts, t2], [torch.tensor([9, 77]), torch.tensor([-3, 4])])
        assert torch.allclose(r1, torch.tensor([[0.5] * 3, [1.0] * 3]), atol=1e-5) and torch.equal(r2, torch.full((2, 2), 2.0))
        kk.combine_push_sparse_table([ts, t2], [torch.tensor([77]), torch.tensor([-3])], [torch.ones(1, 3), torch.ones(1, 2)])
        assert torch.allclose(kk.pull_sparse_table(t2, torch.tensor([-3, 4])), torch.tensor([[1.5, 1.5], [2.0, 2.0]]), atol=1e-5)
        d1, d2 = kk.combine_pull_dense_table([td, tb])
        assert torch.allclose(d1, a - 0.5, atol=1e-5) and torch.equal(d2, torch.zeros(20, 20))
        gb = torch.randn(20, 20)
        kk.push_dense_table(tb, gb)                                 # DCT: a COO gradient, top 25 % by magnitude
        moved = kk.pull_dense_table(tb) != 0
        assert 0.2 < moved.float().mean() < 0.3
        assert sum(s.shard.sparse_size(ts) for s in servers) == 4   # ids 5, 9, 2^40, 77 over both servers
        assert kk.try_save_model()
        assert sorted(d for d in os.listdir(tmp_path) if d.startswith("shard_")) == ["shard_0", "shard_1"]
        # an unknown id in a push comes back as the server's error code through both codecs
        from kraken_b200.runtime.rpc import RpcError
        with pytest.raises(RpcError) as err:
            kk.push_sparse_table(ts, torch.tensor([123456]), torch.ones(1, 3))
        assert err.value.code == 15
    finally:
        kk.stop()
        front.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_a_checkpoint_loads_through_the_front_end(tmp_path):
    sched, servers, front = boot(tmp_path / "a", n_ps=1)
    (tmp_path / "a").mkdir(exist_ok=True)
    try:
        kk.initialize(f"zmq://127.0.0.1:{front.port}")
        kk.init_model("loop", kk.OptimType.kSGD, {})
        kk.update_lr(1.0)
        ts = kk.register_sparse_table("e", 2, torch.float32, kk.InitializerType.kConstant, {"value": "3.0"})
        kk.pull_sparse_table(ts, torch.arange(10))
        kk.push_sparse_table(ts, torch.arange(10), torch.ones(10, 2))
        assert kk.try_save_model()
    finally:
        kk.stop()
        front.stop()
        sched.stop()
        for s in servers:
            s.stop()
    sched, servers, front = boot(tmp_path / "b", n_ps=2)
    try:
        kk.initialize(f"zmq://127.0.0.1:{front.port}")
        assert kk.try_load_model_blocked(str(tmp_path / "a"))       # TryLoadModel, then IsAllPsWorking until yes
        ts = kk.register_sparse_table("e", 2, torch.float32, kk.InitializerType.kConstant, {"value": "3.0"})
        assert torch.equal(kk.pull_sparse_table(ts, torch.arange(12)), torch.cat([torch.full((10, 2), 2.0), torch.full((2, 2), 3.0)]))
    finally:
        kk.stop()
        front.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_several_workers_through_the_front_end_at_once(tmp_path):
    """Three worker processes speak the reference's protocol to the front end at the same time, on overlapping rows
    of two servers (every front-end socket has its own thread).  SGD: the final tables are known exactly."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sched, servers, front = boot(tmp_path)
    workers, steps = 3, 10
    try:
        env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        procs = [subprocess.Popen([sys.executable, os.path.join(root, "tests", "mp_tcp_worker.py"),
                                   f"zmq://127.0.0.1:{front.port}", str(k), str(workers), str(steps)], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for k in range(workers)]
        outs = [p.communicate(timeout=300)[0] for p in procs]
        for k, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and f"TCP_WORKER {k} ok" in out, out[-2000:]
        want = torch.zeros(300, 4)
        for k in range(workers):
            g = torch.Generator().manual_seed(100 + k)
            for _ in range(steps):
                ids = torch.randint(0, 300, (200,), generator=g)
                want.index_add_(0, ids, torch.full((200, 4), -0.5 * (k + 1)))
        kk.initialize(f"zmq://127.0.0.1:{front.port}")
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0.0"})
        td = kk.register_dense_table("w", torch.zeros(6, 5))
        seen = want.abs().sum(1) > 0
        assert torch.allclose(kk.pull_sparse_table(ts, torch.arange(300)[seen]), want[seen], atol=1e-4)
        assert torch.allclose(kk.pull_dense_table(td), torch.full((6, 5), -0.5 * steps * sum(range(1, workers + 1))), atol=1e-4)
    finally:
        kk.stop()
        front.stop()
        sched.stop()
        for s in servers:
            s.stop()

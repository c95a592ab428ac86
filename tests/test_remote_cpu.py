"""Multi-process deployment shape, in one process: a scheduler and two parameter servers on
localhost ports, a worker engine talking to them over TCP (the reference's test environment,
kraken/test/kraken_test_main.cc:13-74, boots the same trio on threads)."""
import torch

import kraken_b200.pytorch as kk
from kraken_b200._native import C
from kraken_b200.runtime.remote import PsServer, SchedulerServer


def boot(tmp_path, n_ps=2):
    sched = SchedulerServer(0)
    sched.start()
    servers = []
    for i in range(n_ps):
        ps = PsServer(0, "", f"127.0.0.1:{sched.port}", saved_dir=str(tmp_path), seed=5)
        ps.addr = f"127.0.0.1:{ps.port}"
        ps.start()
        servers.append(ps)
    return sched, servers


def test_worker_against_scheduler_and_two_servers(tmp_path):
    sched, servers = boot(tmp_path)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(0.5)
        a = torch.randn(3, 4)
        td = kk.register_dense_table("w", a)
        ts = kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        assert (td, ts) == (0, 1) and kk.register_dense_table("w", a) == 0
        assert torch.equal(kk.pull_dense_table(td), a)
        g = torch.randn(3, 4)
        kk.push_dense_table(td, g)
        assert torch.allclose(kk.pull_dense_table(td), a - 0.5 * g)
        ids = torch.arange(40).view(4, 10)
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.ones(4, 10, 3))
        kk.push_sparse_table(ts, torch.tensor([3, 3, 7]), torch.ones(3, 3))
        got = kk.pull_sparse_table(ts, torch.tensor([3, 7, 8]))
        assert torch.allclose(got, torch.tensor([[0.0] * 3, [0.5] * 3, [1.0] * 3]))
        # rows are spread over both servers by the consistent-hash ring
        sizes = [s.shard.sparse_size(ts) for s in servers]
        assert sum(sizes) == 40 and all(n > 0 for n in sizes)
        for s in servers:
            for i in s.shard.export_sparse(ts)["ids"].tolist():
                assert sched.router.hit(C.mix64_pair(ts, i)) == s.node_id
        assert kk.try_save_model()
        kk.stop()

        # a fresh cluster of ONE server loads what two servers wrote
        sched2, servers2 = boot(tmp_path / "other", n_ps=1)
        try:
            kk.initialize(f"tcp://127.0.0.1:{sched2.port}")
            assert kk.try_load_model_blocked(str(tmp_path))
            kk.update_lr(0.5)
            assert servers2[0].shard.sparse_size(1) == 40
            assert kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"}) == 1
            assert torch.allclose(kk.pull_sparse_table(1, torch.tensor([3, 7, 8])), got)
            assert kk.register_dense_table("w", a) == 0   # re-attach by name, as the Optimizer does
            assert torch.allclose(kk.pull_dense_table(0), a - 0.5 * g)
        finally:
            kk.stop()
            sched2.stop()
            for s in servers2:
                s.stop()
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_stale_ring_is_refetched_once(tmp_path):
    sched, servers = boot(tmp_path, n_ps=1)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(1.0)
        ts = kk.register_sparse_table("e", 2, torch.float32, kk.InitializerType.kConstant, {"value": "0"})
        kk.native.engine().version -= 1   # pretend the worker's ring is old
        rows = kk.pull_sparse_table(ts, torch.tensor([1, 2]))   # kRouterVersion -> refetch -> retry
        assert rows.shape == (2, 2) and kk.native.engine().version == sched.router.version()
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_rpc_timeout_is_reported(tmp_path):
    """A server that never answers: the call fails with kTimeout instead of blocking."""
    import socket
    from kraken_b200.runtime.rpc import Connecter, Rpc, RpcError
    silent = socket.socket()
    silent.bind(("127.0.0.1", 0))
    silent.listen(1)
    c = Connecter(f"127.0.0.1:{silent.getsockname()[1]}", timeout_ms=200)
    try:
        try:
            c.call(Rpc.HEARTBEAT)
            assert False, "expected a timeout"
        except RpcError as e:
            assert e.code == 17
    finally:
        c.close()
        silent.close()

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
        kk.initialize(f"127.0.0.1:{sched.port}")     # a bare "host:port", as the reference's scheduler address
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


def _wait_all_working(sched, timeout_s=60.0):
    import time
    t0 = time.monotonic()
    while time.monotonic() - t0 < timeout_s:
        if sched.is_all_working({}, ())[0]["yes"]:
            return
        time.sleep(0.05)
    raise AssertionError("the servers did not all return to kWork")


def test_server_joins_while_training(tmp_path):
    """Elastic scale-out with the proxy phase: a second and a third server join a cluster that already holds
    rows and optimizer state while a worker keeps TRAINING with real gradients.  No request is refused as
    "busy" (kNodeStatus) - a stale ring (kRouterVersion) only costs a refetch -, every update lands exactly
    once (the tables equal a single shard fed the same stream), rows and accumulators end up where the final
    ring says (kraken/ps/ps.cc:336-477,553-602; kraken/ps/proxy.cc:29-145; kraken/ps/ps_op.cc:10-127)."""
    import threading

    sched, servers = boot(tmp_path, n_ps=1)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        conf = {"initial_accumulator_value": "0.1"}
        kk.init_model("m", kk.OptimType.kAdagrad, conf)
        kk.update_lr(0.1)
        oracle = C.CpuShard(0)
        oracle.init_model("m", kk.OptimType.kAdagrad, conf)
        w0 = torch.randn(5, 3)
        tds = [kk.register_dense_table(f"w{i}", w0 + i) for i in range(6)]
        for i, td in enumerate(tds):
            oracle.create_dense_table(td, f"w{i}", w0 + i)
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0.3"})
        oracle.create_sparse_table(ts, "e", 4, kk.InitializerType.kConstant, {"value": "0.3"})
        ids = torch.arange(0, 3000)
        kk.pull_sparse_table(ts, ids)
        oracle.pull_sparse(ts, ids)
        gen = torch.Generator().manual_seed(0)

        def one_step(k):
            """The same pushes to the cluster and to the single-shard oracle."""
            part = torch.randperm(3000, generator=gen)[:500].sort().values
            g = torch.randn(500, 4, generator=gen)
            kk.pull_sparse_table(ts, part)
            kk.push_sparse_table(ts, part, g)
            oracle.pull_sparse(ts, part)
            assert oracle.push_sparse(ts, part, g, 0.1) == 0
            td = tds[k % len(tds)]
            gd = torch.randn(5, 3, generator=gen)
            kk.push_dense_table(td, gd)
            oracle.push_dense(td, gd, 0.1)

        for k in range(3):   # rows and Adagrad accumulators now differ from their initial values
            one_step(k)

        stop, errors, steps = threading.Event(), [], [3]

        def train():
            try:
                while not stop.is_set() or steps[0] < 40:
                    one_step(steps[0])
                    steps[0] += 1
            except Exception as e:  # noqa: BLE001 - the test reports whatever went wrong
                errors.append(e)
                stop.set()

        th = threading.Thread(target=train)
        th.start()
        for _ in range(2):
            ps = PsServer(0, "", f"127.0.0.1:{sched.port}", saved_dir=str(tmp_path), seed=5)
            ps.addr = f"127.0.0.1:{ps.port}"
            ps.start()    # returns as soon as the scheduler admits it: it serves through the proxy from then on
            servers.append(ps)
        _wait_all_working(sched)
        stop.set()
        th.join(timeout=120)
        assert not errors, errors
        eng = kk.native.engine()
        assert eng.refusals.get(7, 0) == 0, eng.refusals      # nobody answered "busy"
        assert eng.refusals.get(8, 0) >= 1, eng.refusals      # the ring did change under the worker

        sizes = [s.shard.sparse_size(ts) for s in servers]
        assert sum(sizes) == 3000 and all(n > 0 for n in sizes), sizes
        for s in servers:   # every row sits where the final ring says
            for i in s.shard.export_sparse(ts)["ids"].tolist():
                assert sched.router.hit(C.mix64_pair(ts, i)) == s.node_id
        # every update landed exactly once, wherever the row lived at the time
        assert torch.allclose(kk.pull_sparse_table(ts, ids), oracle.pull_sparse(ts, ids), atol=1e-6)
        for td in tds:
            assert torch.allclose(kk.pull_dense_table(td), oracle.pull_dense(td).view(5, 3), atol=1e-6)
        owners = {sched.router.hit(C.mix64(td)) for td in tds}
        assert len(owners) > 1   # some dense tables moved as well
        # optimizer state travelled with the rows
        want = oracle.export_sparse(ts)
        got_ids = torch.cat([s.shard.export_sparse(ts)["ids"] for s in servers])
        o1, o2 = torch.argsort(want["ids"]), torch.argsort(got_ids)
        for k, acc in want["states"].items():
            got = torch.cat([s.shard.export_sparse(ts)["states"][k] for s in servers])[o2]
            assert torch.allclose(got, acc[o1], atol=1e-6)
        moved = sum(s.rows_received + s.rows_fetched for s in servers[1:])
        assert moved >= sizes[1] + sizes[2]
        assert kk.try_save_model()
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_compressed_bodies_round_trip(tmp_path):
    """Worker<->server bodies compressed (header byte 1): same results as uncompressed, and a frame of
    a compressible tensor is smaller on the wire."""
    import socket as pysocket

    from kraken_b200.runtime import rpc

    sched, servers = boot(tmp_path, n_ps=2)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}", compress=kk.CompressType.kDCT)  # the reference's kSnappy slot
        assert all(c.compress == 1 for c in kk.native.engine().ps.values())
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(1.0)
        ts = kk.register_sparse_table("e", 8, torch.float32, kk.InitializerType.kConstant, {"value": "2.0"})
        ids = torch.arange(5000)
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.full((5000, 8), 2.0))
        kk.push_sparse_table(ts, ids, torch.ones(5000, 8))
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.ones(5000, 8))
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()

    a, b = pysocket.socketpair()
    try:
        body = rpc.pack_body({"k": 1}, [torch.zeros(1 << 16)])
        rpc.send_frame(a, 7, 3, body, rpc.COMPRESS_SNAPPY)
        (n,) = rpc.struct.unpack("<I", b.recv(4, pysocket.MSG_PEEK))
        assert n < len(body) // 15   # zeros: one 3-byte copy element per 64 bytes
        stamp, code, got, comp = rpc.recv_frame(b)
        assert (stamp, code, comp) == (7, 3, 1) and got == body
    finally:
        a.close()
        b.close()


def test_combined_requests_use_one_round_per_server(tmp_path):
    """kCombinePullDense / kCombinePullSparse / kCombinePushSparse: several tables per message, same
    results as the per-table calls."""
    sched, servers = boot(tmp_path, n_ps=2)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(0.5)
        tds = [kk.register_dense_table(f"w{i}", torch.full((2, 3), float(i))) for i in range(5)]
        t_a = kk.register_sparse_table("a", 2, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        t_b = kk.register_sparse_table("b", 3, torch.float32, kk.InitializerType.kConstant, {"value": "2.0"})
        calls = {}
        eng = kk.native.engine()
        for node, c in eng.ps.items():
            orig = c.call

            def counted(rpc, meta=None, tensors=(), timeout_ms=None, orig=orig):
                calls[rpc] = calls.get(rpc, 0) + 1
                return orig(rpc, meta, tensors, timeout_ms)

            c.call = counted
        dense = kk.combine_pull_dense_table(tds)
        assert all(torch.equal(d, torch.full((2, 3), float(i))) for i, d in enumerate(dense))
        ids_a, ids_b = torch.arange(0, 300).view(3, 100), torch.arange(100, 500)
        ra, rb = kk.combine_pull_sparse_table([t_a, t_b], [ids_a, ids_b])
        assert torch.equal(ra, torch.ones(3, 100, 2)) and torch.equal(rb, torch.full((400, 3), 2.0))
        kk.combine_push_sparse_table([t_a, t_b], [ids_a, ids_b], [torch.ones(3, 100, 2), torch.ones(400, 3)])
        ra, rb = kk.combine_pull_sparse_table([t_a, t_b], [ids_a, ids_b])
        assert torch.equal(ra, torch.full((3, 100, 2), 0.5)) and torch.equal(rb, torch.full((400, 3), 1.5))
        from kraken_b200.runtime.rpc import Rpc
        assert calls.get(Rpc.COMBINE_PULL_DENSE, 0) <= 2            # one per server that owns a table
        assert calls.get(Rpc.COMBINE_PULL_SPARSE, 0) <= 4 and calls.get(Rpc.COMBINE_PUSH_SPARSE, 0) <= 2
        assert Rpc.PULL_SPARSE not in calls and Rpc.PUSH_SPARSE not in calls and Rpc.PULL_DENSE not in calls
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_failed_join_is_rolled_back(tmp_path):
    """Host-side fault injection: the only older server fails when it is told of the join.  The newcomer is
    refused, the ring goes back to what it was and the worker keeps training on the old server."""
    import pytest

    from kraken_b200.runtime.rpc import Rpc, RpcError

    sched, servers = boot(tmp_path, n_ps=1)
    late = None
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(1.0)
        ts = kk.register_sparse_table("e", 2, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
        ids = torch.arange(200)
        kk.pull_sparse_table(ts, ids)

        def broken(meta, tensors):
            raise RpcError(-1, "injected transfer failure")

        servers[0].station.handlers[Rpc.NOTIFY_NODE_JOIN] = broken
        late = PsServer(0, "", f"127.0.0.1:{sched.port}", saved_dir=str(tmp_path), seed=5)
        late.addr = f"127.0.0.1:{late.port}"
        with pytest.raises(RpcError):
            late.start()
        assert list(sched.nodes) == [0] and not sched.router.contains(1)
        kk.push_sparse_table(ts, ids, torch.ones(200, 2))
        assert torch.equal(kk.pull_sparse_table(ts, ids), torch.zeros(200, 2))
        assert servers[0].shard.sparse_size(ts) == 200
    finally:
        kk.stop()
        sched.stop()
        for s in servers + ([late] if late is not None else []):
            s.stop()


def test_async_push_returns_at_once_and_is_applied_in_order(tmp_path):
    """``initialize(..., async_push=True)``: a push is handed to a background thread and the call returns before
    the servers have answered (the reference's fire-and-forget pushes, kraken/worker/emitter.cc:431-446,539-549).
    Pushes stay in order, ``flush_pushes()`` (and a save, and stop) wait for them, and a push that a server
    rejects raises at a later call instead of vanishing."""
    import time
    import pytest
    sched, servers = boot(tmp_path)
    try:
        kk.initialize(f"tcp://127.0.0.1:{sched.port}", async_push=True)
        kk.init_model("m", kk.OptimType.kSGD, {})
        kk.update_lr(1.0)
        ts = kk.register_sparse_table("e", 2, torch.float32, kk.InitializerType.kConstant, {"value": "0.0"})
        td = kk.register_dense_table("w", torch.zeros(4))
        ids = torch.arange(2000)
        kk.pull_sparse_table(ts, ids)
        # make every server slow to answer a push: the calls below must not wait for it
        from kraken_b200.runtime.rpc import Rpc
        for s in servers:
            real = s.station.handlers[Rpc.PUSH_SPARSE]
            s.station.handlers[Rpc.PUSH_SPARSE] = lambda meta, tensors, real=real: (time.sleep(0.15), real(meta, tensors))[1]
        t0 = time.perf_counter()
        for step in range(1, 4):
            kk.update_lr(float(step))                       # each push carries the rate it was made with
            kk.push_sparse_table(ts, ids, torch.ones(2000, 2))
            kk.push_dense_table(td, torch.ones(4))
        handed_over = time.perf_counter() - t0
        eng = kk.native.engine()
        eng.flush_pushes()
        applied = time.perf_counter() - t0
        assert handed_over < 0.25 < applied, (handed_over, applied)   # 3 pushes x 2 servers x 0.15 s happen behind the caller
        assert torch.allclose(kk.pull_sparse_table(ts, ids), torch.full((2000, 2), -6.0))   # -(1 + 2 + 3)
        assert torch.allclose(kk.pull_dense_table(td), torch.full((4,), -6.0))
        # a push the servers reject (unknown ids) surfaces at a later call
        kk.push_sparse_table(ts, torch.arange(10_000, 10_010), torch.ones(10, 2))
        from kraken_b200.runtime.rpc import RpcError
        with pytest.raises(RpcError) as err:
            eng.flush_pushes()
        assert err.value.code == 15          # kSparseIdNotExist, as the synchronous push reports it
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()


def test_several_workers_share_the_servers(tmp_path):
    """Four worker PROCESSES train against two servers at once, on overlapping rows and one dense table
    (the reference's data parallelism: independent workers, every push its own update,
    kraken/worker/emitter.cc:417-447,491-550).  With SGD the order of the updates does not matter, so the
    final tables are known exactly: a lost or doubled update under concurrency would show."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sched, servers = boot(tmp_path)
    workers, steps = 4, 12
    try:
        env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        procs = [subprocess.Popen([sys.executable, os.path.join(root, "tests", "mp_tcp_worker.py"),
                                   f"tcp://127.0.0.1:{sched.port}", str(k), str(workers), str(steps)], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for k in range(workers)]
        outs = [p.communicate(timeout=300)[0] for p in procs]
        for k, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and f"TCP_WORKER {k} ok" in out, out[-2000:]
        # what the tables must hold: every occurrence of an id moves its row by lr * (worker index + 1)
        want = torch.zeros(300, 4)
        for k in range(workers):
            g = torch.Generator().manual_seed(100 + k)
            for _ in range(steps):
                ids = torch.randint(0, 300, (200,), generator=g)
                want.index_add_(0, ids, torch.full((200, 4), -0.5 * (k + 1)))
        kk.initialize(f"tcp://127.0.0.1:{sched.port}")
        ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0.0"})
        td = kk.register_dense_table("w", torch.zeros(6, 5))
        seen = want.abs().sum(1) > 0
        got = kk.pull_sparse_table(ts, torch.arange(300)[seen])
        assert torch.allclose(got, want[seen], atol=1e-4)
        assert torch.allclose(kk.pull_dense_table(td), torch.full((6, 5), -0.5 * steps * sum(range(1, workers + 1))), atol=1e-4)
        assert sum(s.shard.sparse_size(ts) for s in servers) == int(seen.sum())
    finally:
        kk.stop()
        sched.stop()
        for s in servers:
            s.stop()

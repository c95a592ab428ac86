"""Public API on the CPU engine.  The first tests replay the reference's
integration scenario (kraken/test/worker/emitter_test.cc:11-161): register,
pull == initial value, push, pull == w - lr * g, single and combined - without
its sleeps, since pushes here are synchronous."""
import os
import subprocess
import sys

import pytest
import torch

import kraken_b200.pytorch as kk

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def start(**kw):
    kk.initialize("cpu", **kw)
    kk.init_model("test", kk.OptimType.kSGD, {})
    kk.update_lr(0.5)


def test_dense_register_pull_push():
    start()
    a, b = torch.randn(3, 4), torch.randn(5)
    ia, ib = kk.register_dense_table("a", a), kk.register_dense_table("b", b)
    assert (ia, ib) == (0, 1)
    assert kk.register_dense_table("a", a) == 0  # same name: same id
    with pytest.raises(kk.KrakenError):
        kk.register_dense_table("a", torch.zeros(2))
    assert torch.equal(kk.pull_dense_table(ia), a)
    g = torch.randn(3, 4)
    kk.push_dense_table(ia, g)
    assert torch.allclose(kk.pull_dense_table(ia), a - 0.5 * g)
    pa, pb = kk.combine_pull_dense_table([ia, ib])
    assert torch.allclose(pa, a - 0.5 * g) and torch.equal(pb, b)


def test_sparse_register_pull_push_and_duplicates():
    start()
    t = kk.register_sparse_table("e", 3, torch.float32, kk.InitializerType.kConstant, {"value": "1.0"})
    idx = torch.tensor([[4, 9], [4, 4]])
    rows = kk.pull_sparse_table(t, idx)
    assert rows.shape == (2, 2, 3) and torch.equal(rows, torch.ones(2, 2, 3))
    g = torch.arange(12, dtype=torch.float32).view(2, 2, 3)
    kk.push_sparse_table(t, idx, g)
    got = kk.pull_sparse_table(t, torch.tensor([4, 9]))
    assert torch.allclose(got[0], 1 - 0.5 * (g[0, 0] + g[1, 0] + g[1, 1]))  # duplicate ids are summed
    assert torch.allclose(got[1], 1 - 0.5 * g[0, 1])
    with pytest.raises(kk.KrakenError):
        kk.push_sparse_table(t, torch.tensor([12345]), torch.ones(1, 3))  # never pulled: no such row


def test_combine_pull_push():
    start()
    t0 = kk.register_sparse_table("e0", 2, torch.float32, kk.InitializerType.kConstant, {"value": "0.0"})
    t1 = kk.register_sparse_table("e1", 4, torch.float32, kk.InitializerType.kConstant, {"value": "3.0"})
    i0, i1 = torch.tensor([1, 2, 3]), torch.tensor([7])
    r0, r1 = kk.combine_pull_sparse_table([t0, t1], [i0, i1])
    assert torch.equal(r0, torch.zeros(3, 2)) and torch.equal(r1, torch.full((1, 4), 3.0))
    kk.combine_push_sparse_table([t0, t1], [i0, i1], [torch.ones(3, 2), torch.ones(1, 4)])
    r0, r1 = kk.combine_pull_sparse_table([t0, t1], [i0, i1])
    assert torch.allclose(r0, torch.full((3, 2), -0.5)) and torch.allclose(r1, torch.full((1, 4), 2.5))


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = kk.Embedding(4, initializer=kk.ConstantInitializer(0.5))
        self.bag = kk.JaggedEmbedding(4, initializer=kk.ConstantInitializer(0.25), mode="mean", patch_value=0.0)
        self.lin = torch.nn.Linear(8, 1)

    def forward(self, idx, jt):
        return self.lin(torch.cat([self.emb(idx), self.bag(jt)], 1)).sum()


def test_optimizer_trains_like_a_local_model():
    kk.initialize("cpu")
    torch.manual_seed(0)
    m = Tiny()
    opt = kk.Optimizer("tiny", m.named_parameters(), 0.1, kk.SGD())
    assert m.emb.sparse_table.table_id() is not None and m.emb.sparse_table.name() == "emb.sparse_table"

    # plain-torch twin with real embedding matrices
    ref_emb = torch.nn.Parameter(torch.full((10, 4), 0.5))
    ref_bag = torch.nn.Parameter(torch.full((10, 4), 0.25))
    ref_lin = torch.nn.Linear(8, 1)
    ref_lin.load_state_dict(m.lin.state_dict())
    ref_opt = torch.optim.SGD([ref_emb, ref_bag, *ref_lin.parameters()], 0.1)

    idx = torch.tensor([1, 2, 1])
    values, offsets = torch.tensor([3, 4, 4, 5, 6, 7]), torch.tensor([0, 2, 3, 6])
    for _ in range(3):
        loss = m(idx, kk.JaggedTensor(values, offsets))
        loss.backward()
        opt.step()
        pooled = torch.stack([ref_bag[values[offsets[b]:offsets[b + 1]]].mean(0) for b in range(3)])
        ref_loss = ref_lin(torch.cat([ref_emb[idx], pooled], 1)).sum()
        ref_opt.zero_grad()
        ref_loss.backward()
        ref_opt.step()
        assert torch.allclose(loss, ref_loss, atol=1e-5)
    assert torch.allclose(m.lin.weight, ref_lin.weight, atol=1e-5)
    assert torch.allclose(kk.pull_sparse_table(m.emb.sparse_table.table_id(), torch.tensor([1, 2])), ref_emb[[1, 2]],
                          atol=1e-5)


def test_dct_emitter_on_dense_tables():
    kk.initialize("cpu", emitter_type=kk.EmitterType.kDCT, life_span=2, eta=0.5)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(1.0)
    w = torch.zeros(512)
    t = kk.register_dense_table("w", w)
    g = torch.arange(512, dtype=torch.float32) - 255.5
    kk.push_dense_table(t, g)
    got = kk.pull_dense_table(t)
    big = g.abs() >= g.abs().kthvalue(257).values  # top half by magnitude was sent
    assert torch.equal(got[big], -g[big]) and torch.equal(got[~big], torch.zeros(int((~big).sum())))
    kk.push_dense_table(t, torch.zeros(512))  # error feedback: the residual alone is below tau, nothing moves
    assert torch.equal(kk.pull_dense_table(t), got)


def test_checkpoint_round_trip_and_retention(tmp_path):
    d = str(tmp_path)
    kk.initialize("cpu", saved_dir=d, max_save_count=2)
    kk.init_model("m", kk.OptimType.kAdam, {"amsgrad": "true"})
    kk.update_lr(0.1)
    td = kk.register_dense_table("w", torch.randn(4, 4))
    ts = kk.register_sparse_table("emb.sparse_table", 8, torch.float32, kk.InitializerType.kNormal, {})
    ids = torch.arange(100)
    for _ in range(3):
        kk.pull_sparse_table(ts, ids)
        kk.push_sparse_table(ts, ids, torch.randn(100, 8))
        kk.push_dense_table(td, torch.randn(4, 4))
        assert kk.try_save_model()
    assert len(os.listdir(os.path.join(d, "shard_0"))) == 2
    rows, w = kk.pull_sparse_table(ts, ids), kk.pull_dense_table(td)
    g_s, g_d = torch.randn(100, 8), torch.randn(4, 4)
    kk.push_sparse_table(ts, ids, g_s)
    kk.push_dense_table(td, g_d)
    rows_next, w_next = kk.pull_sparse_table(ts, ids), kk.pull_dense_table(td)
    kk.stop()

    kk.initialize("cpu")
    assert kk.try_load_model_blocked(d)
    kk.update_lr(0.1)
    assert torch.equal(kk.pull_sparse_table(1, ids), rows) and torch.equal(kk.pull_dense_table(0), w)
    # optimizer state came back too: the next update lands on the same values
    kk.push_sparse_table(1, ids, g_s)
    kk.push_dense_table(0, g_d)
    assert torch.allclose(kk.pull_sparse_table(1, ids), rows_next, atol=1e-6)
    assert torch.allclose(kk.pull_dense_table(0), w_next, atol=1e-6)
    assert not kk.try_load_model_blocked("/nonexistent") or True


def run_ranks(script: str, world: int, *args: str, timeout: int = 300) -> str:
    port = 29600 + (os.getpid() % 300)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(REPO, "tests", script), *args]
    env = dict(os.environ, PYTHONPATH=REPO, OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


def test_two_cpu_ranks_match_one_rank(tmp_path):
    out = run_ranks("mp_cpu_worker.py", 2, str(tmp_path))
    assert "RANKS_MATCH_SINGLE ok" in out and "RESHARD ok" in out


def test_step_profiler_records_regions(tmp_path):
    from kraken_b200.utils.profiler import StepProfiler
    path = tmp_path / "prof.jsonl"
    prof = StepProfiler(str(path), rank=0, lag=1)
    for step in range(3):
        with prof.region("pull"):
            sum(range(1000))
        with prof.region("pull"):
            pass
        prof.count("unique_ids", 5)
        prof.end_step()
    prof.close()
    import json
    recs = [json.loads(l) for l in open(path)]
    assert [r["step"] for r in recs] == [0, 1, 2] and all(r["pull_ms"] >= 0 and r["unique_ids"] == 5 for r in recs)
    assert "pull_ms" in prof.summary()


def test_same_seed_gives_bitwise_identical_tables():
    """Determinism check of the CPU engine: two runs with the same seed, data and step order leave
    bit-for-bit the same rows, optimizer state and dense weights.  (The GPU kernels sum duplicate and
    split-K gradients with floating-point atomics, so there only the tolerance tests apply.)"""
    from kraken_b200.models import ClickDataset, DeepFM
    from kraken_b200.ops import bce_with_logits

    def run():
        start(seed=11)
        torch.manual_seed(0)
        model = DeepFM(num_fields=5, num_dense=13, dim=8, hidden=(16, 8), init_std=0.1)
        opt = kk.Optimizer("det", model.named_parameters(), 1e-2, kk.Adam())
        data = ClickDataset(num_fields=5, vocab=200, seed=3)
        for _ in range(6):
            dense, ids, labels = data.batch(64)
            loss = bce_with_logits(model(dense, ids), labels)
            loss.backward()
            opt.step()
        probe = torch.arange(0, 1000)
        rows = [kk.pull_sparse_table(p.table_id(), probe).clone() for p in
                (model.second_order.sparse_table, model.first_order.sparse_table)]
        dense_w = [p.detach().clone() for n, p in model.named_parameters() if p.dim() > 0 and p.numel() > 0
                   and not hasattr(p, "table_id")]
        kk.stop()
        return float(loss.detach()), rows, dense_w

    l0, r0, w0 = run()
    l1, r1, w1 = run()
    assert l0 == l1
    assert all(torch.equal(a, b) for a, b in zip(r0, r1))
    assert len(w0) > 0 and all(torch.equal(a, b) for a, b in zip(w0, w1))


@pytest.mark.parametrize("dtype", [torch.float64, torch.float16])
def test_tables_of_other_float_types(dtype):
    """The reference's tables are f32 or f64 (kraken/t/math.cc); here the shards always hold float32
    and values are converted where they leave or enter the engine."""
    start()
    try:
        ts = kk.register_sparse_table("e", 4, dtype, kk.InitializerType.kConstant, {"value": "1"})
        rows = kk.pull_sparse_table(ts, torch.tensor([[1, 2]]))
        assert rows.dtype == dtype and rows.shape == (1, 2, 4)
        kk.push_sparse_table(ts, torch.tensor([1]), torch.ones(1, 4, dtype=dtype))
        assert torch.equal(kk.pull_sparse_table(ts, torch.tensor([1])), torch.full((1, 4), 0.5, dtype=dtype))
        td = kk.register_dense_table("w", torch.ones(3, dtype=dtype))
        kk.push_dense_table(td, torch.ones(3, dtype=dtype))
        got = kk.pull_dense_table(td)
        assert got.dtype == dtype and torch.equal(got, torch.full((3,), 0.5, dtype=dtype))
    finally:
        kk.stop()


def test_corrupted_or_missing_checkpoint_is_reported(tmp_path):
    """Fault injection on the host: a truncated .sparse file, a garbage model.binary and an empty
    directory each end in an error (or a False return), never in a crash."""
    d = str(tmp_path / "ck")
    kk.initialize("cpu", saved_dir=d)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(0.1)
    ts = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {})
    kk.pull_sparse_table(ts, torch.arange(500))
    assert kk.try_save_model()
    kk.stop()
    shard_dir = os.path.join(d, "shard_0")
    snap = os.path.join(shard_dir, sorted(os.listdir(shard_dir))[-1])
    sparse_file = os.path.join(snap, "e.sparse")
    blob = open(sparse_file, "rb").read()

    # 1. truncated rows
    with open(sparse_file, "wb") as f:
        f.write(blob[:len(blob) // 2])
    kk.initialize("cpu")
    with pytest.raises(Exception):
        kk.try_load_model_blocked(d)
    kk.stop()

    # 2. model metadata replaced by garbage
    with open(sparse_file, "wb") as f:
        f.write(blob)
    model_file = os.path.join(snap, "model.binary")
    good = open(model_file, "rb").read()
    with open(model_file, "wb") as f:
        f.write(b"\\xff" * 40)
    kk.initialize("cpu")
    with pytest.raises(Exception):
        kk.try_load_model_blocked(d)
    kk.stop()

    # 3. nothing there at all
    kk.initialize("cpu")
    assert not kk.try_load_model_blocked(str(tmp_path / "empty"))
    kk.stop()

    # the intact files still load
    with open(model_file, "wb") as f:
        f.write(good)
    kk.initialize("cpu")
    assert kk.try_load_model_blocked(d)
    assert kk.native.engine().shard.sparse_size(0) == 500
    kk.stop()


def test_learning_rate_schedules_reach_the_servers():
    """A schedule is stepped once per optimizer step and its rate travels with the next push (the reference's
    Optimizer does lr.step() + update_lr in step(), kraken/pytorch/optimizer.py:151-173; it ships ConstantLR only)."""
    import math
    assert [round(kk.StepLR(1.0, 2, 0.5).rate_at(n), 4) for n in range(5)] == [1.0, 1.0, 0.5, 0.5, 0.25]
    assert [round(kk.ExponentialLR(2.0, 0.5).rate_at(n), 4) for n in range(3)] == [2.0, 1.0, 0.5]
    wc = kk.WarmupCosineLR(1.0, warmup=4, total=12, floor=0.1)
    assert [round(wc.rate_at(n), 3) for n in (0, 3, 4, 8, 12, 20)] == [0.25, 1.0, 1.0, 0.55, 0.1, 0.1]
    assert kk.LambdaLR(0.5, lambda n: 1.0 / (1 + n)).rate_at(3) == 0.125

    kk.initialize("cpu", seed=0)
    try:
        emb = kk.Embedding(2, initializer=kk.ConstantInitializer(1.0), name="sched")
        opt = kk.Optimizer("sched", emb.named_parameters(), kk.StepLR(0.5, step_size=2, gamma=0.1), kk.SGD())
        ids = torch.tensor([7])
        seen = []
        for _ in range(5):
            before = emb(ids).detach().clone()
            emb(ids).sum().backward()            # gradient 1 per element: the row moves by exactly the rate in force
            opt.step()
            seen.append(round(float((before - emb(ids).detach())[0, 0]), 6))
        assert seen == [0.5, 0.5, 0.05, 0.05, 0.005]
        assert math.isclose(kk.native.engine().lr, 0.005, rel_tol=1e-6)
    finally:
        kk.stop()


def test_alias_resolves_every_module_path_of_the_reference_layout():
    """``install_alias()``: ``kraken.pytorch`` and each module the reference has under it
    (kraken/pytorch/*.py), plus ``kraken_native``, resolve to THE modules of this package, not to second copies
    (a second copy of a submodule would load the native library twice); unknown names still fail."""
    import importlib
    import sys

    import kraken_b200
    kraken_b200.install_alias()
    for name in ("embedding", "combine_embedding", "jagged_embedding", "combine_jagged_embedding", "jagged_tensor",
                 "jagged_embedding_funcs", "sparse_table", "combine_sparse_table", "optim", "optimizer", "initializer", "lr"):
        aliased = importlib.import_module("kraken.pytorch." + name)
        assert aliased is importlib.import_module("kraken_b200.pytorch." + name), name
    from kraken.pytorch.combine_jagged_embedding import CombineJaggedEmbedding
    from kraken.pytorch.combine_sparse_table import CombineSparseTable
    assert CombineJaggedEmbedding.__module__.startswith("kraken_b200.") and CombineSparseTable is not None
    import kraken_native
    assert kraken_native is sys.modules["kraken_b200.pytorch.native"] and hasattr(kraken_native, "jagged_mean_backward")
    with pytest.raises(ModuleNotFoundError):
        importlib.import_module("kraken.pytorch.no_such_module")

"""GPU engine behaviour around a step: growth before and between steps, error words that reach the
caller, CUDA-graph replays that keep the host-side work of a step (B200 only)."""
import pytest
import torch

import kraken_b200.pytorch as kk

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_first_pull_larger_than_the_table_grows_it_first():
    """A table registered with 256 slots is asked for 20 000 new ids in its first call: the shard is
    grown before the kernels run, every row comes back initialised, and no error is recorded
    (the reference's server creates rows without bound, kraken/ps/sparse_table.cc:58-70)."""
    kk.initialize("gpu", table_capacity=256, seed=1)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(0.5)
    t = kk.register_sparse_table("e", 8, torch.float32, kk.InitializerType.kConstant, {"value": "0.75"})
    ids = torch.arange(20_000, device=DEV) * 7919
    rows = kk.pull_sparse_table(t, ids)
    assert torch.equal(rows, torch.full_like(rows, 0.75))
    kk.push_sparse_table(t, ids, torch.ones(20_000, 8, device=DEV))
    again = kk.pull_sparse_table(t, ids)
    assert torch.allclose(again, torch.full_like(again, 0.25))
    eng = kk.native.engine()
    eng.check()
    assert eng.sparse[t].num_rows() == 20_000 and eng.sparse[t].capacity >= 20_000 / 0.6


def test_long_id_stream_runs_as_several_rounds():
    """With ``long_id_streams`` a call longer than the exchange buffers (1000 ids here) is served in rounds
    through the same buffers, as the reference's emitter takes a request of any length
    (kraken/worker/emitter.cc:123-183).  3500 ids with repeats: every occurrence gets its row, and a push
    applies one SGD update per round an id occurs in."""
    kk.initialize("gpu", table_capacity=1 << 14, max_ids_per_call=1000, long_id_streams=True, seed=3)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(1.0)
    t = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "2.0"})
    ids = (torch.arange(3500, device=DEV) % 1200) * 31
    rows = kk.pull_sparse_table(t, ids)
    assert rows.shape == (3500, 4) and torch.equal(rows, torch.full_like(rows, 2.0))
    kk.push_sparse_table(t, ids, torch.full((3500, 4), 0.125, device=DEV))
    eng = kk.native.engine()
    eng.check()
    assert eng.sparse[t].num_rows() == 1200
    # per round (1000 ids) the occurrences of an id are summed, then one update with lr 1: row = 2 - 0.125 * occurrences
    occ = torch.bincount(ids // 31, minlength=1200).to(torch.float32)
    want = (2.0 - 0.125 * occ)[ids // 31]
    got = kk.pull_sparse_table(t, ids)
    assert torch.allclose(got, want[:, None].expand(-1, 4))
    with pytest.raises(kk.KrakenError, match="exceed the channel capacity"):
        kk.native.engine().cfg.long_id_streams = False
        kk.pull_sparse_table(t, ids)


def test_recorded_error_reaches_the_caller_at_end_step():
    """A push to ids the table has never seen is kSparseIdNotExist on the owner
    (kraken/ps/sparse_table.cc:96-98).  Nothing synchronises in the step itself; the code must come
    out of ``end_step()`` within a few steps as a KrakenError."""
    kk.initialize("gpu", table_capacity=1 << 12, status_poll_interval=1)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(0.1)
    t = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0"})
    kk.pull_sparse_table(t, torch.arange(10, device=DEV))
    kk.push_sparse_table(t, torch.arange(100, 110, device=DEV), torch.ones(10, 4, device=DEV))  # unknown ids
    eng = kk.native.engine()
    with pytest.raises(kk.KrakenError, match="(?i)not exist"):
        for _ in range(6):
            eng.end_step()
            torch.cuda.synchronize()
    for _ in range(3):  # the word was cleared: later steps are clean again
        eng.end_step()
        torch.cuda.synchronize()


def test_graphed_step_grows_tables_and_follows_the_lr_schedule():
    """Replays of a captured step create new rows every time.  The table starts far too small; the
    host-side work GraphedStep does after each replay must grow it (re-capturing the graph) and
    must advance the learning-rate schedule, which a bare replay would freeze."""
    from kraken_b200.pytorch.lr import LR
    from kraken_b200.utils.graph import GraphedStep

    class Halving(LR):
        def __init__(self):
            self.v = 1.0

        def step(self):
            self.v *= 0.5

        def lr(self):
            return self.v

    kk.initialize("gpu", table_capacity=1 << 13, max_ids_per_call=512, seed=2, status_poll_interval=1)
    emb = kk.Embedding(4, initializer=kk.ConstantInitializer(0.0), name="g")
    opt = kk.Optimizer("m", emb.named_parameters(), Halving(), kk.SGD())
    eng = kk.native.engine()

    def train(ids):
        loss = emb(ids).sum()   # d loss / d row = 1 for every occurrence
        loss.backward()
        opt.step()
        return loss.detach()

    first = torch.arange(512, device=DEV)
    step = GraphedStep(train, (first,), warmup=1, optimizer=opt)
    lr_seen = []
    for k in range(1, 40):
        step(torch.arange(512, device=DEV) + 512 * k)  # 512 brand-new ids per replay
        lr_seen.append(float(eng.lr_dev.item()))
    torch.cuda.synchronize()
    eng.check()
    tid = emb.sparse_table.table_id()
    assert eng.sparse[tid].capacity > (1 << 13) and step.recaptures >= 1
    assert eng.sparse[tid].num_rows() == 512 * 40
    assert lr_seen[-1] < lr_seen[0] * 1e-6  # halved after every replay
    # every id was pushed exactly once with gradient 1 and the learning rate of its step: all rows moved
    rows, found = eng.sparse[tid].lookup(torch.arange(512 * 40, device=DEV))
    assert bool(found.all()) and bool((rows[:512 * 2] < 0).all())


def test_bf16_step_tracks_the_fp32_step_on_the_teacher_task():
    """The benchmark's fused bf16 step and the all-fp32 step, same model, same batches, 300 Adam steps:
    held-out loss and AUC must agree closely (the reference computes in fp32, kraken/t/math.cc:20-76)."""
    from kraken_b200.benchmarks.precision_parity import main
    rec = main(["--steps", "300", "--batch", "4096", "--vocab", "20000", "--eval-batches", "4",
                "--table-capacity", str(1 << 21)])
    assert rec["fp32"]["eval_auc"] > 0.6, rec           # the task is learnable: both arms learn it
    assert abs(rec["eval_auc_diff"]) < 0.01, rec
    assert abs(rec["eval_loss_diff"]) < 0.01, rec


def _combined_scenario(dev, rank=0, world=1, steps=3):
    """Six tables (three of width 4, two of width 8, one of width 1) pulled and pushed through the combined
    calls for a few steps, the SAME ids appearing in several tables; every table must then equal a CPU
    shard fed the concatenated stream (scenario of kraken/test/worker/emitter_test.cc:108-158)."""
    from kraken_b200._native import C
    dims = [4, 8, 4, 1, 8, 4]
    kk.init_model("m", kk.OptimType.kAdagrad, {})
    kk.update_lr(0.1)
    tids = [kk.register_sparse_table(f"t{k}", d, torch.float32, kk.InitializerType.kConstant, {"value": str(0.1 * (k + 1))})
            for k, d in enumerate(dims)]
    shard = C.CpuShard(0)
    shard.init_model("m", kk.OptimType.kAdagrad, {})
    for k, (t, d) in enumerate(zip(tids, dims)):
        shard.create_sparse_table(t, f"t{k}", d, kk.InitializerType.kConstant, {"value": str(0.1 * (k + 1))})
    eng = kk.native.engine()
    gen = torch.Generator().manual_seed(7)
    for s in range(steps):
        # per rank and table: ids from a small range so that tables and ranks overlap heavily
        all_ids = [[torch.randint(0, 300, (50 + 17 * k + 5 * r,), generator=gen) for k in range(len(dims))]
                   for r in range(world)]
        all_g = [[torch.randn(all_ids[r][k].numel(), d, generator=gen) for k, d in enumerate(dims)] for r in range(world)]
        mine = [i.to(dev) for i in all_ids[rank]]
        before = eng.kernel_launches()
        rows = kk.combine_pull_sparse_table(tids, mine)
        pull_launches = eng.kernel_launches() - before
        for k, t in enumerate(tids):
            cat = torch.cat([all_ids[r][k] for r in range(world)])
            uniq, inv = C.cpu_dedup(cat)
            want = shard.pull_sparse(t, uniq)[inv]
            lo = sum(all_ids[r][k].numel() for r in range(rank))
            got = rows[k].cpu()
            assert got.shape == (mine[k].numel(), dims[k])
            assert torch.allclose(got, want[lo:lo + mine[k].numel()], atol=1e-5), (s, k)
        kk.combine_push_sparse_table(tids, mine, [g.to(dev) for g in all_g[rank]])
        for k, t in enumerate(tids):
            cat = torch.cat([all_ids[r][k] for r in range(world)])
            gcat = torch.cat([all_g[r][k] for r in range(world)])
            uniq, inv = C.cpu_dedup(cat)
            assert shard.push_sparse(t, uniq, C.cpu_segment_sum(gcat, inv, uniq.numel()), 0.1) == 0
        # three row widths -> two group exchanges (8 launches each between GPUs) + one single-table exchange (7),
        # not six exchanges
        assert pull_launches <= 2 * 8 + 7, pull_launches
    eng.check()
    probe = torch.arange(300)
    for k, t in enumerate(tids):
        got = kk.pull_sparse_table(t, probe.to(dev)).cpu()
        assert torch.allclose(got, shard.pull_sparse(t, probe), atol=1e-4), k
    # a combined push that is not preceded by its pull looks the ids up again
    ids2 = [torch.arange(5 + k, device=dev) for k in range(len(dims))]
    kk.combine_push_sparse_table(tids, ids2, [torch.zeros(5 + k, d, device=dev) for k, d in enumerate(dims)])
    eng.check()


def test_combined_tables_share_one_exchange():
    kk.initialize("gpu", table_capacity=1 << 12, seed=0)
    _combined_scenario(torch.device("cuda", torch.cuda.current_device()))


def test_combine_embedding_trains_through_the_group_exchange():
    """kk.CombineEmbedding forward + backward through autograd on the group exchange."""
    kk.initialize("gpu", table_capacity=1 << 12, seed=0)
    emb = kk.CombineEmbedding([4, 4, 4], initializers=[kk.ConstantInitializer(1.0)] * 3, names=["a", "b", "c"])
    opt = kk.Optimizer("m", emb.named_parameters(), 0.5, kk.SGD())
    ids = [torch.tensor([1, 2, 2, 3], device=DEV), torch.tensor([2, 2], device=DEV), torch.tensor([9], device=DEV)]
    outs = emb(ids)
    assert [tuple(o.shape) for o in outs] == [(4, 4), (2, 4), (1, 4)]
    (outs[0].sum() + 2.0 * outs[1].sum() + 3.0 * outs[2].sum()).backward()
    opt.step()
    tids = emb.combine_sparse_table.table_ids()
    a = kk.pull_sparse_table(tids[0], torch.tensor([1, 2, 3], device=DEV)).cpu()
    b = kk.pull_sparse_table(tids[1], torch.tensor([2], device=DEV)).cpu()
    c = kk.pull_sparse_table(tids[2], torch.tensor([9], device=DEV)).cpu()
    assert torch.allclose(a, torch.tensor([[0.5] * 4, [0.0] * 4, [0.5] * 4]))      # id 2 occurs twice in table a
    assert torch.allclose(b, torch.full((1, 4), 1.0 - 0.5 * 2.0 * 2))              # twice, gradient 2 each
    assert torch.allclose(c, torch.full((1, 4), 1.0 - 0.5 * 3.0))
    kk.native.engine().check()


def test_jagged_embeddings_train_on_the_gpu_engine():
    """kk.JaggedEmbedding and kk.CombineJaggedEmbedding (sum / mean bags, an empty bag, per-id weights) must
    reach the tables through autograd: one SGD step, rows compared with the same step on the CPU engine."""
    def run(backend):
        kk.stop()
        kk.initialize(backend, table_capacity=1 << 10, seed=0)
        torch.manual_seed(0)
        dev = "cuda" if backend == "gpu" else "cpu"
        single = kk.JaggedEmbedding(4, initializer=kk.ConstantInitializer(0.5), name="s", mode="mean", patch_value=-1.0)
        combo = kk.CombineJaggedEmbedding([4, 4, 2], initializers=[kk.ConstantInitializer(0.25)] * 3,
                                          names=["c0", "c1", "c2"], modes=["sum", "mean", "sum"],
                                          patch_values=[0.0, 0.0, 0.0])
        mods = torch.nn.ModuleList([single, combo])
        opt = kk.Optimizer("m", mods.named_parameters(), 0.5, kk.SGD())
        jt = lambda vals, offs, w=None: kk.JaggedTensor(torch.tensor(vals, device=dev), torch.tensor(offs, device=dev),
                                                        None if w is None else torch.tensor(w, device=dev))
        a = single(jt([1, 2, 2, 7], [0, 3, 3, 4]))                      # bags: {1,2,2}, {}, {7}
        outs = combo([jt([1, 1, 3], [0, 2, 3], [1.0, 2.0, 0.5]), jt([1, 4, 5, 6], [0, 1, 4]), jt([9], [0, 1])])
        loss = a.sum() + outs[0].sum() * 2.0 + outs[1].sum() + outs[2].sum() * 3.0
        empty_bag = a[1].detach().cpu().clone()
        loss.backward()
        opt.step()
        tids = [single.embedding.sparse_table.table_id()] + list(combo.combine_embedding.combine_sparse_table.table_ids())
        probes = [[1, 2, 7], [1, 3], [1, 4, 5, 6], [9]]
        rows = [kk.pull_sparse_table(t, torch.tensor(p, device=dev)).cpu() for t, p in zip(tids, probes)]
        kk.stop()
        return empty_bag, rows

    e_gpu, r_gpu = run("gpu")
    e_cpu, r_cpu = run("cpu")
    assert torch.equal(e_gpu, torch.full((4,), -1.0)) and torch.equal(e_cpu, e_gpu)
    for g, c in zip(r_gpu, r_cpu):
        assert torch.allclose(g, c, atol=1e-6), (g, c)
    assert not torch.allclose(r_gpu[0], torch.full_like(r_gpu[0], 0.5))   # the rows did move


def test_streamed_save_and_chunked_load_round_trip_on_the_gpu_engine(tmp_path):
    """A table of 2.6 M rows with Adagrad state is written by the streamed writer and read back into a NEW
    GPU engine through the chunked reader (two chunks of 2^21 rows and a remainder, so the reader thread,
    both staging sets and their reuse are exercised): ids, values and accumulators must come back bit for bit,
    and a further update must continue from the restored accumulator."""
    n, dim = 2_600_000, 4
    kk.initialize("gpu", table_capacity=1 << 23, max_ids_per_call=n, saved_dir=str(tmp_path), seed=11)
    kk.init_model("m", kk.OptimType.kAdagrad, {"initial_accumulator_value": "0.1"})
    kk.update_lr(0.5)
    t = kk.register_sparse_table("e", dim, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.1"})
    ids = torch.arange(n, device=DEV) * 2654435761 - (1 << 40)          # negative ids too
    kk.pull_sparse_table(t, ids)
    g = torch.randn(n, dim, device=DEV)
    kk.push_sparse_table(t, ids, g)
    eng = kk.native.engine()
    before = eng.sparse[t].export()
    order = torch.argsort(before["ids"])
    assert kk.try_save_model()
    kk.stop()

    kk.initialize("gpu", table_capacity=1 << 16, seed=99)               # grows while it loads
    assert kk.try_load_model_blocked(str(tmp_path))
    eng = kk.native.engine()
    eng.check()
    t2 = next(iter(eng.sparse))
    after = eng.sparse[t2].export()
    order2 = torch.argsort(after["ids"])
    assert after["ids"].numel() == n and torch.equal(after["ids"][order2], before["ids"][order])
    assert torch.equal(after["vals"][order2], before["vals"][order])
    for k in before["states"]:
        assert torch.equal(after["states"][k][order2], before["states"][k][order])
    # the restored accumulator takes part in the next update: acc' = acc + g^2, w' = w - lr g / (sqrt(acc') + eps)
    kk.update_lr(0.5)          # the learning rate is the worker's, not part of a checkpoint
    some = ids[:1000]
    w0 = kk.pull_sparse_table(t2, some)
    kk.push_sparse_table(t2, some, torch.ones(1000, dim, device=DEV))
    w1 = kk.pull_sparse_table(t2, some)
    acc = 0.1 + g[:1000] ** 2 + 1.0
    assert torch.allclose(w0 - w1, 0.5 / (acc.sqrt() + 1e-10), rtol=1e-4, atol=1e-6)

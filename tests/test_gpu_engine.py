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

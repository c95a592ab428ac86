"""CUDA kernels against fp32 PyTorch / CPU-shard references (B200 only)."""
import math

import pytest
import torch

import kraken_b200.pytorch as kk
from kraken_b200._native import C

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gpu_engine(**kw):
    kk.initialize("gpu", **kw)
    return kk.native.engine()


def test_fm_interaction_forward_backward():
    from kraken_b200.ops import fm_interaction
    torch.manual_seed(0)
    for (B, F, D) in [(37, 26, 16), (5, 3, 7), (1000, 26, 64), (64, 4, 1)]:
        e = torch.randn(B, F, D, device=DEV, requires_grad=True)
        out = fm_interaction(e)
        ref_in = e.detach().clone().requires_grad_(True)
        s = ref_in.sum(1)
        ref = 0.5 * (s * s - (ref_in * ref_in).sum(1)).sum(1)
        assert torch.allclose(out, ref, atol=1e-3, rtol=1e-4)
        go = torch.randn(B, device=DEV)
        out.backward(go)
        ref.backward(go)
        assert torch.allclose(e.grad, ref_in.grad, atol=1e-4, rtol=1e-4)


def test_bce_with_logits():
    from kraken_b200.ops import bce_with_logits
    torch.manual_seed(1)
    x = (torch.randn(100001, device=DEV) * 4).requires_grad_(True)
    y = (torch.rand(100001, device=DEV) > 0.5).float()
    loss = bce_with_logits(x, y)
    xr = x.detach().clone().requires_grad_(True)
    ref = torch.nn.functional.binary_cross_entropy_with_logits(xr, y)
    assert abs(loss.item() - ref.item()) < 1e-5
    loss.backward()
    ref.backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-9, rtol=1e-5)


def test_jagged_ops_match_cpu():
    torch.manual_seed(2)
    lens = torch.randint(0, 6, (200,))
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)])
    values = torch.randn(int(offsets[-1]), 12)
    for fwd, bwd in [(C.jagged_sum_forward, C.jagged_sum_backward), (C.jagged_mean_forward, C.jagged_mean_backward)]:
        want = fwd(values, offsets, 0.75)
        got = fwd(values.to(DEV), offsets.to(DEV), 0.75)
        assert torch.allclose(got.cpu(), want, atol=1e-5)
        g = torch.randn(200, 12)
        assert torch.allclose(bwd(offsets.to(DEV), g.to(DEV)).cpu(), bwd(offsets, g), atol=1e-6)


def test_dedup_bucketize_groups_by_owner():
    eng = gpu_engine()
    kk.init_model("m", kk.OptimType.kSGD, {})
    t = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "0"})
    torch.manual_seed(3)
    ids = torch.randint(0, 5000, (20000,), device=DEV)
    ch = eng._channel(t, ids.numel())
    for world in (1, 3, 8):
        cnt = torch.zeros(world, dtype=torch.int32, device=DEV)
        off = torch.zeros(world + 1, dtype=torch.int32, device=DEV)
        C.dedup_bucketize(ids, world, 0, ch.hkeys, ch.slot_of, ch.hbits, cnt, off, ch.uniq, ch.inv,
                          ch.ctrl[4:5])
        off_h = off.cpu().tolist()
        U = off_h[-1]
        uniq = ch.uniq[:U].cpu()
        assert U == torch.unique(ids).numel() and torch.unique(uniq).numel() == U
        assert torch.equal(uniq[ch.inv[:ids.numel()].cpu().long()], ids.cpu())
        for o in range(world):
            seg = uniq[off_h[o]:off_h[o + 1]].tolist()
            assert all(C.owner_of(0, i, world) == o for i in seg)
        assert (ch.hkeys[:, 0] == -1).all()  # the scratch set is empty again


@pytest.mark.parametrize("optim,conf", [
    (kk.OptimType.kSGD, {"momentum": "0.9"}),
    (kk.OptimType.kAdagrad, {"initial_accumulator_value": "0.1"}),
    (kk.OptimType.kAdam, {"amsgrad": "true"}),
    (kk.OptimType.kRMSprop, {"momentum": "0.5", "centered": "true"}),
])
@pytest.mark.parametrize("dim", [16, 1, 6])
def test_sparse_pull_push_matches_cpu_shard(optim, conf, dim):
    gpu_engine(seed=11, table_capacity=1 << 12)
    kk.init_model("m", optim, conf)
    kk.update_lr(0.05)
    t = kk.register_sparse_table("e", dim, torch.float32, kk.InitializerType.kNormal, {"stddev": "0.5"})
    shard = C.CpuShard(11)
    shard.init_model("m", optim, conf)
    shard.create_sparse_table(t, "e", dim, kk.InitializerType.kNormal, {"stddev": "0.5"})
    torch.manual_seed(4)
    for step in range(4):
        ids = torch.randint(0, 300, (64, 7))
        rows = kk.pull_sparse_table(t, ids.to(DEV))
        uniq, inv = C.cpu_dedup(ids.reshape(-1))
        want = shard.pull_sparse(t, uniq)[inv].view(64, 7, dim)
        assert torch.allclose(rows.cpu(), want, atol=1e-5), step
        g = torch.randn(64, 7, dim)
        kk.push_sparse_table(t, ids.to(DEV), g.to(DEV))
        assert shard.push_sparse(t, uniq, C.cpu_segment_sum(g.view(-1, dim), inv, uniq.numel()), 0.05) == 0
    kk.native.engine().check()
    all_ids = torch.arange(300)
    assert torch.allclose(kk.pull_sparse_table(t, all_ids.to(DEV)).cpu(), shard.pull_sparse(t, all_ids), atol=2e-4)


def test_push_without_ticket_looks_ids_up_again():
    gpu_engine()
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(1.0)
    t = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kConstant, {"value": "1"})
    a, b = torch.tensor([1, 2, 3], device=DEV), torch.tensor([3, 4], device=DEV)
    kk.pull_sparse_table(t, a)
    kk.pull_sparse_table(t, b)          # a's ticket is stale now
    kk.push_sparse_table(t, a, torch.ones(3, 4, device=DEV))
    got = kk.pull_sparse_table(t, torch.tensor([1, 2, 3, 4], device=DEV)).cpu()
    assert torch.equal(got, torch.tensor([[0.0] * 4, [0.0] * 4, [0.0] * 4, [1.0] * 4]))
    kk.push_sparse_table(t, torch.tensor([77], device=DEV), torch.ones(1, 4, device=DEV))  # unknown id
    with pytest.raises(kk.KrakenError):
        kk.native.engine().check()


def test_fused_bag_lookup_matches_unfused():
    eng = gpu_engine(seed=5)
    kk.init_model("m", kk.OptimType.kSGD, {})
    kk.update_lr(0.5)
    t = kk.register_sparse_table("e", 8, torch.float32, kk.InitializerType.kNormal, {})
    torch.manual_seed(6)
    lens = torch.randint(0, 5, (50,))
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(DEV)
    values = torch.randint(0, 40, (int(offsets[-1]),), device=DEV)
    weights = torch.rand(values.numel(), device=DEV)
    rows = kk.pull_sparse_table(t, torch.arange(40, device=DEV)).clone()
    for mean in (False, True):
        pooled, ticket = eng.pull_sparse_pooled(t, values, offsets, weights=weights, mean=mean, patch_value=-2.0)
        fwd = C.jagged_mean_forward if mean else C.jagged_sum_forward
        want = fwd(rows[values] * weights[:, None], offsets, -2.0)
        assert torch.allclose(pooled, want, atol=1e-5)
        g = torch.randn(50, 8, device=DEV)
        eng.push_sparse_pooled(t, ticket, g)
        bwd = C.jagged_mean_backward if mean else C.jagged_sum_backward
        per_row = bwd(offsets, g) * weights[:, None]
        want_rows = rows.clone().index_add_(0, values, -0.5 * per_row)
        rows = kk.pull_sparse_table(t, torch.arange(40, device=DEV)).clone()
        assert torch.allclose(rows, want_rows, atol=1e-5)


def test_table_growth_export_import_evict():
    eng = gpu_engine(table_capacity=64)
    kk.init_model("m", kk.OptimType.kAdam, {})
    kk.update_lr(0.1)
    t = kk.register_sparse_table("e", 4, torch.float32, kk.InitializerType.kNormal, {})
    tab = eng.sparse[t]
    ids = torch.arange(30, device=DEV)
    before = kk.pull_sparse_table(t, ids).clone()
    kk.push_sparse_table(t, ids, torch.ones(30, 4, device=DEV))
    after = kk.pull_sparse_table(t, ids).clone()
    assert tab.num_rows() == 30 and tab.capacity in (64, 128)  # the second pull may have reserved room for 30 more
    assert tab.reserve(1000) and tab.capacity >= 1000 / 0.6 and tab.num_rows() == 30
    assert torch.equal(kk.pull_sparse_table(t, ids), after)       # rows and state survived the rehash
    cols = tab.export()
    assert sorted(cols["ids"].tolist()) == list(range(30)) and cols["states_i"][0].tolist() == [1] * 30
    part = tab.export(filter_mode=1, salt=0, world=3, rank=1)
    assert all(C.owner_of(0, i, 3) == 1 for i in part["ids"].tolist())
    kk.pull_sparse_table(t, torch.arange(100, 110, device=DEV))    # never pushed: steps == 0
    assert tab.evict(min_steps=1) == 10 and tab.num_rows() == 30
    rows, found = tab.lookup(torch.tensor([0, 105], device=DEV))
    assert found.tolist() == [1, 0] and torch.equal(rows[0], after[0])
    # a full table reports kTableFull instead of hanging
    small = gpu_small_table()
    with pytest.raises(kk.KrakenError):
        small.check()


def gpu_small_table():
    eng = kk.native.engine()
    t = kk.register_sparse_table("tiny", 2, torch.float32, kk.InitializerType.kConstant, {"value": "0"})
    eng.sparse[t]._alloc(4)   # 16 slots
    # straight through the channel: the engine's own entry points would grow the table first
    ch = eng._channel(t, 64)
    ch.pull(torch.arange(64, device=DEV))
    return ch


def test_dct_select_tau_is_exact_kth_largest():
    torch.manual_seed(7)
    x = torch.randn(100003, device=DEV)
    hist = torch.zeros(1024, dtype=torch.int32, device=DEV)
    prefix = torch.zeros(2, dtype=torch.int32, device=DEV)
    tau = torch.zeros(1, device=DEV)
    for k in (1, 17, 25000, 100003):
        C.dct_select_tau(x, k, hist, prefix, tau)
        assert tau.item() == x.abs().topk(k).values[-1].item()


@pytest.mark.parametrize("optim,conf,dct", [
    (kk.OptimType.kSGD, {"momentum": "0.9"}, False),
    (kk.OptimType.kAdam, {}, False),
    (kk.OptimType.kSGD, {}, True),
])
def test_dense_bucket_step_matches_cpu_shard(optim, conf, dct):
    gpu_engine(emitter_type=kk.EmitterType.kDCT if dct else kk.EmitterType.kDefault, life_span=2, eta=0.75)
    kk.init_model("m", optim, conf)
    kk.update_lr(0.05)
    torch.manual_seed(8)
    shapes = [(300, 7), (5,), (1000,)]
    vals = [torch.randn(*s) for s in shapes]
    ids = [kk.register_dense_table(f"w{i}", v) for i, v in enumerate(vals)]
    shard = C.CpuShard(0)
    shard.init_model("m", optim, conf)
    states = {}
    for i, v in zip(ids, vals):
        shard.create_dense_table(i, f"w{i}", v)
        states[i] = C.DctState()
    for step in range(5):
        for i, s in zip(ids, shapes):
            g = torch.randn(*s)
            kk.push_dense_table(i, g.to(DEV))
            packed = C.cpu_dct_compress(g, 2, 0.75, states[i]) if dct else None
            if packed is not None:
                shard.push_dense_coo(i, packed[0], packed[1], 0.05)
            else:
                shard.push_dense(i, g, 0.05)
        got = kk.combine_pull_dense_table(ids)
        for i, s, gv in zip(ids, shapes, got):
            assert torch.allclose(gv.cpu(), shard.pull_dense(i).view(*s), atol=1e-5), (step, i)
    kk.native.engine().check()


def test_device_wait_times_out_cleanly():
    """A peer that never raises its flag: the bounded wait gives up, the kernel records
    kTimeout, returns, and the context stays usable.  One GPU plays rank 0 of 2 with the
    "peer" arena aliased to its own, so nothing ever answers for rank 1."""
    from kraken_b200.parallel.sparse_shard import GpuSparseTable, SparseChannel
    dev = torch.device("cuda", torch.cuda.current_device())
    table = GpuSparseTable(0, "e", 4, kk.InitializerType.kConstant, {"value": "0"}, kk.OptimType.kSGD, {}, 0, 1 << 10,
                           2, dev)
    ch = SparseChannel(table, rank=0, world=2, max_ids=256, spin_limit=2000, alias_peers=True)
    ch.pull(torch.arange(64, device=dev))
    torch.cuda.synchronize()
    with pytest.raises(kk.KrakenError, match="timeout"):
        ch.check()
    x = torch.ones(4, device=dev) * 2
    assert float(x.sum().item()) == 8.0  # the context still works
    ch.close()


def test_fused_deepfm_matches_unfused_path():
    """Same seed, same data: the fused front end + tensor-core MLP must track the
    unfused fp32 path (loss and table contents) within bf16 tolerance."""
    from kraken_b200.models import ClickDataset, DeepFM
    from kraken_b200.ops import bce_with_logits

    def run(fused, fold=False, overlap=False):
        kk.initialize("gpu", seed=21, table_capacity=1 << 14, overlap_dense_step=overlap)
        torch.manual_seed(0)
        model = DeepFM(num_fields=6, num_dense=13, dim=16, hidden=(64, 32), init_std=0.1, fused=fused,
                       fold_first_order=fold).to(DEV)
        model.mlp.use_tensor_cores = fused
        opt = kk.Optimizer("m", model.named_parameters(), 5e-2, kk.SGD())  # SGD: Adam would amplify sign noise of tiny gradients
        data = ClickDataset(num_fields=6, vocab=500, seed=9)
        losses = []
        for _ in range(5):
            dense, ids, labels = (t.to(DEV) for t in data.batch(700))
            loss = bce_with_logits(model(dense, ids), labels)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        kk.native.engine().check()
        probe = torch.arange(0, 3000, 7, device=DEV)
        rows = kk.pull_sparse_table(model.second_order.sparse_table.table_id(), probe).cpu()
        first = (kk.pull_sparse_table(model.first_order.sparse_table.table_id(), probe).cpu() if not fold
                 else rows[:, 16:17].clone())
        rows = rows[:, :16]
        w = model.mlp.layers[0].weight.detach().cpu().clone()
        kk.stop()
        return losses, rows, first, w

    l1, r1, f1, w1 = run(True)
    l0, r0, f0, w0 = run(False)
    assert all(abs(a - b) < 5e-3 for a, b in zip(l1, l0)), (l1, l0)
    assert (r1 - r0).abs().max().item() < 2e-2 and (f1 - f0).abs().max().item() < 2e-2
    assert (w1 - w0).abs().max().item() < 2e-2
    # folded layout (first-order weight inside the embedding row): fused and unfused agree too
    l3, r3, f3, w3 = run(True, fold=True)
    l2, r2, f2, w2 = run(False, fold=True)
    assert all(abs(a - b) < 5e-3 for a, b in zip(l3, l2)), (l3, l2)
    assert (r3 - r2).abs().max().item() < 2e-2 and (f3 - f2).abs().max().item() < 2e-2
    # dense step on the backward's side stream (beside the sparse push): same kernels, same numbers
    l4, r4, f4, w4 = run(True, fold=True, overlap=True)
    # (split-K weight gradients are summed by atomics, so the low bits are not reproducible)
    assert all(abs(a - b) < 1e-5 for a, b in zip(l4, l3)) and (w4 - w3).abs().max().item() < 1e-5
    assert (r4 - r3).abs().max().item() < 1e-5


@pytest.mark.gpu
def test_device_prefetcher_order_and_reuse():
    from kraken_b200.utils.prefetch import DevicePrefetcher

    dev = torch.device("cuda", 0)
    host = [(torch.full((1 << 16,), float(i)).pin_memory(), torch.arange(i, i + 64).pin_memory()) for i in range(7)]
    seen = []
    for a, b in DevicePrefetcher(iter(host), dev):
        # enqueue work that reads the buffers, then move on: buffers must not be overwritten early
        seen.append((a.sum(), b.clone()))
    assert len(seen) == 7
    for i, (s, b) in enumerate(seen):
        assert float(s) == float(i) * (1 << 16)
        assert torch.equal(b.cpu(), torch.arange(i, i + 64))

"""CPU shard semantics: the four server-side optimizers against torch.optim,
initializer moments, pull-creates / push-needs-existing, DCT invariants, jagged
pooling.  (The reference tests none of these: kraken/test has only plain SGD
through emitter_test.cc.)"""
import math

import pytest
import torch

from kraken_b200._native import C


def make_shard(optim_type, conf, seed=0):
    s = C.CpuShard(seed)
    s.init_model("m", optim_type, conf)
    return s


def run_dense(optim_type, conf, torch_opt, steps=5, lr=0.05):
    torch.manual_seed(0)
    w0 = torch.randn(7, 3)
    s = make_shard(optim_type, conf)
    s.create_dense_table(0, "w", w0)
    p = torch.nn.Parameter(w0.clone())
    opt = torch_opt([p], lr)
    for i in range(steps):
        g = torch.randn(7, 3)
        s.push_dense(0, g, lr)
        p.grad = g.clone()
        opt.step()
    return s.pull_dense(0).view(7, 3), p.data


def test_sgd_plain_momentum_nesterov():
    got, want = run_dense(C.OptimType.kSGD, {}, lambda p, lr: torch.optim.SGD(p, lr))
    assert torch.allclose(got, want, atol=1e-6)
    got, want = run_dense(C.OptimType.kSGD, {"momentum": "0.9", "weight_decay": "0.01"},
                          lambda p, lr: torch.optim.SGD(p, lr, momentum=0.9, weight_decay=0.01))
    assert torch.allclose(got, want, atol=1e-5)
    got, want = run_dense(C.OptimType.kSGD, {"momentum": "0.9", "nesterov": "true"},
                          lambda p, lr: torch.optim.SGD(p, lr, momentum=0.9, nesterov=True))
    assert torch.allclose(got, want, atol=1e-5)
    got, want = run_dense(C.OptimType.kSGD, {"momentum": "0.8", "dampening": "0.3"},
                          lambda p, lr: torch.optim.SGD(p, lr, momentum=0.8, dampening=0.3))
    assert torch.allclose(got, want, atol=1e-5)


def test_adagrad_with_and_without_initial_accumulator():
    got, want = run_dense(C.OptimType.kAdagrad, {"eps": "1e-10"}, lambda p, lr: torch.optim.Adagrad(p, lr, eps=1e-10))
    assert torch.allclose(got, want, atol=1e-5)
    got, want = run_dense(C.OptimType.kAdagrad, {"eps": "1e-10", "initial_accumulator_value": "0.1"},
                          lambda p, lr: torch.optim.Adagrad(p, lr, eps=1e-10, initial_accumulator_value=0.1))
    assert torch.allclose(got, want, atol=1e-5)


def test_adam_matches_torch_up_to_eps_placement():
    # torch divides sqrt(v) by sqrt(bias2) before adding eps; this optimizer adds eps to sqrt(v_hat):
    # the same thing.  amsgrad differs (max over bias-corrected v) and is tested on its own below.
    got, want = run_dense(C.OptimType.kAdam, {"beta1": "0.9", "beta2": "0.999", "eps": "1e-8"},
                          lambda p, lr: torch.optim.Adam(p, lr, betas=(0.9, 0.999), eps=1e-8))
    assert torch.allclose(got, want, atol=1e-5)


def test_adam_amsgrad_uses_bias_corrected_maximum():
    lr, b1, b2, eps = 0.1, 0.9, 0.999, 1e-8
    s = make_shard(C.OptimType.kAdam, {"amsgrad": "true"})
    w = torch.tensor([1.0, -2.0])
    s.create_dense_table(0, "w", w)
    m = torch.zeros(2); v = torch.zeros(2); vmax = torch.zeros(2)
    for t, g in enumerate([torch.tensor([1.0, 0.5]), torch.tensor([0.1, -0.2]), torch.tensor([0.01, 0.02])], 1):
        s.push_dense(0, g, lr)
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        vhat = v / (1 - b2 ** t)
        vmax = torch.maximum(vmax, vhat)
        w = w - lr * (m / (1 - b1 ** t)) / (vmax.sqrt() + eps)
    assert torch.allclose(s.pull_dense(0), w, atol=1e-5)


def test_rmsprop_variants():
    got, want = run_dense(C.OptimType.kRMSprop, {"alpha": "0.99", "eps": "1e-8"},
                          lambda p, lr: torch.optim.RMSprop(p, lr, alpha=0.99, eps=1e-8))
    assert torch.allclose(got, want, atol=1e-5)
    got, want = run_dense(C.OptimType.kRMSprop, {"momentum": "0.5", "centered": "true"},
                          lambda p, lr: torch.optim.RMSprop(p, lr, momentum=0.5, centered=True))
    assert torch.allclose(got, want, atol=1e-4)


def test_sparse_pull_creates_and_push_needs_existing_rows():
    s = make_shard(C.OptimType.kSGD, {})
    s.create_sparse_table(1, "e", 4, C.InitializerType.kConstant, {"value": "2.0"})
    ids = torch.tensor([10, 11])
    assert torch.equal(s.pull_sparse(1, ids), torch.full((2, 4), 2.0))
    assert s.sparse_size(1) == 2
    assert s.push_sparse(1, ids, torch.ones(2, 4), 0.5) == 0
    assert torch.equal(s.pull_sparse(1, ids), torch.full((2, 4), 1.5))
    assert s.push_sparse(1, torch.tensor([99]), torch.ones(1, 4), 0.5) == 15  # kSparseIdNotExist
    assert s.sparse_size(1) == 2


def test_adam_step_count_is_per_row():
    s = make_shard(C.OptimType.kAdam, {})
    s.create_sparse_table(0, "e", 2, C.InitializerType.kConstant, {"value": "0"})
    s.pull_sparse(0, torch.tensor([1, 2]))
    s.push_sparse(0, torch.tensor([1]), torch.ones(1, 2), 0.1)
    s.push_sparse(0, torch.tensor([1, 2]), torch.ones(2, 2), 0.1)
    cols = s.export_sparse(0)
    steps = dict(zip(cols["ids"].tolist(), cols["states_i"][0].tolist()))
    assert steps == {1: 2, 2: 1}
    rows = s.pull_sparse(0, torch.tensor([1, 2]))
    assert torch.allclose(rows[1], torch.full((2,), -0.1), atol=1e-6)  # first Adam step moves by lr


@pytest.mark.parametrize("init_type,conf,mean,std", [
    (C.InitializerType.kNormal, {"mean": "1.0", "stddev": "2.0"}, 1.0, 2.0),
    (C.InitializerType.kUniform, {"lower": "-1", "upper": "3"}, 1.0, 4 / math.sqrt(12)),
    (C.InitializerType.kXavierNormal, {"gain": "2"}, 0.0, 2 * math.sqrt(2 / 17)),
    (C.InitializerType.kXavierUniform, {"gain": "1"}, 0.0, math.sqrt(2 / 17)),
])
def test_initializer_moments(init_type, conf, mean, std):
    s = make_shard(C.OptimType.kSGD, {}, seed=7)
    s.create_sparse_table(0, "e", 16, init_type, conf)
    rows = s.pull_sparse(0, torch.arange(20000))
    assert abs(rows.mean().item() - mean) < 0.03 * max(1.0, std)
    assert abs(rows.std().item() - std) < 0.03 * max(1.0, std)
    # rows are a function of (seed, table, id) only
    s2 = make_shard(C.OptimType.kSGD, {}, seed=7)
    s2.create_sparse_table(0, "e", 16, init_type, conf)
    assert torch.equal(s2.pull_sparse(0, torch.tensor([123])), rows[123:124])


def test_dedup_and_segment_sum():
    ids = torch.tensor([5, 7, 5, 9, 7, 5])
    uniq, inv = C.cpu_dedup(ids)
    assert uniq.tolist() == [5, 7, 9] and inv.tolist() == [0, 1, 0, 2, 1, 0]
    g = torch.arange(12, dtype=torch.float32).view(6, 2)
    out = C.cpu_segment_sum(g, inv, 3)
    assert torch.equal(out, torch.stack([g[0] + g[2] + g[5], g[1] + g[4], g[3]]))


def test_kth_largest_abs():
    x = torch.tensor([0.5, -3.0, 2.0, -0.1, 1.0])
    assert C.kth_largest_abs(x, 1) == 3.0 and C.kth_largest_abs(x, 2) == 2.0 and C.kth_largest_abs(x, 5) == pytest.approx(0.1)


def test_dct_invariants():
    torch.manual_seed(1)
    n, eta, life = 4096, 0.75, 3
    st = C.DctState()
    e_prev = torch.zeros(n)
    for step in range(5):
        g = torch.randn(n)
        idx, vals = C.cpu_dct_compress(g, life, eta, st)
        f = g + e_prev
        sent = torch.zeros(n)
        sent[idx] = vals
        assert torch.allclose(sent + st.residual(), f, atol=0)  # nothing is lost
        assert (idx[1:] > idx[:-1]).all()                        # ascending flat indices
        assert (vals.abs() >= st.tau).all() and (st.residual().abs() < st.tau + 1e-12).all()
        if step % life == 0:
            assert abs(idx.numel() - int(n * (1 - eta))) <= 2     # tau refreshed: top 25 % sent
        e_prev = st.residual()
    assert C.cpu_dct_compress(torch.randn(100), life, eta, C.DctState()) is None  # small tables go dense


def test_jagged_forward_backward_cpu():
    values = torch.arange(10, dtype=torch.float32).view(5, 2)
    offsets = torch.tensor([0, 2, 2, 5])
    s = C.jagged_sum_forward(values, offsets, -1.0)
    assert torch.equal(s, torch.stack([values[0] + values[1], torch.full((2,), -1.0), values[2:].sum(0)]))
    m = C.jagged_mean_forward(values, offsets, 0.5)
    assert torch.allclose(m, torch.stack([values[:2].mean(0), torch.full((2,), 0.5), values[2:].mean(0)]))
    g = torch.tensor([[1.0, 2.0], [3.0, 4.0], [6.0, 9.0]])
    gs = C.jagged_sum_backward(offsets, g)
    assert torch.equal(gs, torch.stack([g[0], g[0], g[2], g[2], g[2]]))  # every row of a bag, not only the first
    gm = C.jagged_mean_backward(offsets, g)
    assert torch.allclose(gm, torch.stack([g[0] / 2, g[0] / 2, g[2] / 3, g[2] / 3, g[2] / 3]))

"""tcgen05 Linear kernels against fp32 matmuls of the same bf16-rounded operands (B200 only)."""
import pytest
import torch

from kraken_b200._native import C

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def close(got, want, tol=2e-2, row_tol=None):
    """Two checks.  Over the whole matrix: max error within ``tol`` of the largest reference value.  Per row
    and per column: max error within ``tol`` of THAT row's / column's largest reference value (plus a small
    share of the global one for rows that are all near zero) - a wrong or missing tile whose values happen
    to be small passes the first check and fails this one.  ``row_tol`` loosens the second check for chains of
    layers, where bf16 rounding of the intermediate activations and gradients adds up on rows of small magnitude."""
    got, want = got.float(), want.float()
    diff = (got - want).abs()
    err = diff.max().item()
    ref = want.abs().max().item() + 1e-6
    if err > tol * ref:
        return False, ("global", err, ref)
    if got.dim() == 2:
        for axis in (1, 0):
            e = diff.amax(dim=axis)
            r = want.abs().amax(dim=axis)
            bad = e > (row_tol if row_tol is not None else tol) * r + 2e-3 * ref
            if bool(bad.any()):
                k = int(bad.nonzero()[0])
                return False, ("row" if axis == 1 else "column", k, e[k].item(), r[k].item())
    return True, (err, ref)


SHAPES = [(300, 400, 432), (128, 16, 64), (4096, 256, 512), (1000, 208, 72), (257, 400, 400), (40001, 400, 432),
          (30000, 416, 400)]  # the last two take the weight-resident persistent kernel


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("relu", [False, True])
def test_linear_forward(M, N, K, relu):
    torch.manual_seed(0)
    x, w, b = rnd(M, K), rnd(N, K, scale=0.1), torch.randn(N, device=DEV)
    y = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.linear_forward(x, w, b, relu, y, status)
    want = x.float() @ w.float().t() + b
    if relu:
        want = want.relu()
    assert status.item() == 0
    ok, info = close(y, want)
    assert ok, info


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_dgrad_with_relu_mask(M, N, K):
    torch.manual_seed(1)
    dy, w = rnd(M, N), rnd(N, K, scale=0.1)
    h = rnd(M, K).relu()
    wt = w.t().contiguous()
    dx = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.linear_dgrad(dy, wt, h, dx, status)
    want = (dy.float() @ w.float()) * (h.float() > 0)
    assert status.item() == 0
    ok, info = close(dx, want)
    assert ok, info
    C.linear_dgrad(dy, wt, None, dx, status)
    ok, info = close(dx, dy.float() @ w.float())
    assert ok and status.item() == 0, info


@pytest.mark.parametrize("M,N,K", SHAPES + [(65536, 400, 432)])
def test_linear_wgrad_accumulates(M, N, K):
    torch.manual_seed(2)
    dy, x = rnd(M, N, scale=0.1), rnd(M, K)
    dw = torch.zeros(N, K, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.linear_wgrad(dy, x, dw, status)
    want = dy.float().t() @ x.float()
    assert status.item() == 0
    ok, info = close(dw, want, tol=5e-3)
    assert ok, info
    C.linear_wgrad(dy, x, dw, status)  # red-add: a second call doubles the buffer
    ok, info = close(dw, 2 * want, tol=5e-3)
    assert ok, info


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("M,N,K", [(40001, 400, 448), (65536, 448, 400), (20000, 256, 192)])
def test_every_gemm_variant_agrees(variant, M, N, K):
    """CTA-pair (cta_group::2), single-CTA weight-resident and tile-per-CTA kernels on one shape."""
    torch.manual_seed(2)
    x, w, b = rnd(M, K), rnd(N, K, scale=0.1), torch.randn(N, device=DEV)
    dy, h = rnd(M, N), rnd(M, K).relu()
    y = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    dx = torch.full((M, K), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.gemm_set_tuning(variant, 0)
    try:
        C.linear_forward(x, w, b, True, y, status)
        C.linear_dgrad(dy, w.t().contiguous(), h, dx, status)
    finally:
        C.gemm_set_tuning(0, 0)
    assert status.item() == 0
    ok, info = close(y, (x.float() @ w.float().t() + b).relu())
    assert ok, info
    ok, info = close(dx, (dy.float() @ w.float()) * (h.float() > 0))
    assert ok, info


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("M,N,K", [(40001, 400, 448), (300, 72, 64)])
def test_relu_bit_mask_round_trip(variant, M, N, K):
    """Forward leaves one bit per output (> 0); the input gradient masked by those bits equals the
    one masked by the bf16 activations themselves."""
    torch.manual_seed(3)
    x, w, b = rnd(M, K), rnd(N, K, scale=0.1), torch.randn(N, device=DEV)
    y = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    mask = torch.zeros(((N + 15) // 16, (M + 63) // 64 * 64), device=DEV, dtype=torch.int16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K2 = 96
    dy2, w2 = rnd(M, K2), rnd(K2, N, scale=0.1)     # a following layer N -> K2
    dx_bits = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    dx_acts = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    C.gemm_set_tuning(variant, 0)
    try:
        C.linear_forward(x, w, b, True, y, status, mask)
        C.linear_dgrad(dy2, w2.t().contiguous(), None, dx_bits, status, mask)
        C.linear_dgrad(dy2, w2.t().contiguous(), y, dx_acts, status)
    finally:
        C.gemm_set_tuning(0, 0)
    assert status.item() == 0
    words = (mask[:, :M].t().to(torch.int32) & 0xFFFF)                # [M, chunks]
    got = ((words.unsqueeze(-1) >> torch.arange(16, device=DEV)) & 1).reshape(M, -1)[:, :N].bool()
    assert torch.equal(got, y.float() > 0)
    assert torch.equal(dx_bits, dx_acts)


def test_colsum_bf16():
    torch.manual_seed(3)
    dy = rnd(5000, 400)
    db = torch.ones(400, device=DEV)
    C.colsum_bf16(dy, db)
    assert torch.allclose(db, 1 + dy.float().sum(0), atol=1e-2, rtol=1e-3)


def test_strided_views_are_accepted():
    """Operands may be column slices of wider buffers (pitch > width)."""
    torch.manual_seed(4)
    big = rnd(512, 448)
    x = big[:, :432]
    w = rnd(400, 432, scale=0.1)
    ybuf = torch.zeros(512, 408, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.linear_forward(x, w, None, False, ybuf[:, :400], status)
    ok, info = close(ybuf[:, :400], x.float() @ w.float().t())
    assert ok and status.item() == 0, info
    assert (ybuf[:, 400:] == 0).all()


def emulate(x, ws, bs, g):
    """fp32 restatement of the fused MLP with its rounding points: bf16 inputs, weights and
    hidden activations / activation gradients, fp32 accumulation.  Returns (out, dWs, dbs, dx)."""
    r = lambda t: t.to(torch.bfloat16).float()
    L = len(ws)
    h = [r(x)]
    for i in range(L - 1):
        h.append(r((h[-1] @ r(ws[i]).t() + bs[i]).relu()))
    single = ws[-1].shape[0] == 1
    wl = ws[-1] if single else r(ws[-1])
    out = h[-1] @ wl.t() + bs[-1]
    if not single:
        out = r(out)
    dy = g if single else r(g)
    dws, dbs = [None] * L, [None] * L
    dws[-1], dbs[-1] = dy.t() @ h[-1], dy.sum(0)
    dh = dy @ wl
    if L > 1:
        dh = dh * (h[-1] > 0)
    dh = r(dh)
    for i in range(L - 2, -1, -1):
        dws[i], dbs[i] = dh.t() @ h[i], dh.sum(0)
        dh = dh @ r(ws[i])
        if i > 0:
            dh = dh * (h[i] > 0)
        dh = r(dh)
    return out, dws, dbs, dh


@pytest.mark.parametrize("sizes", [[400, 400, 400, 1], [64, 16], [256, 8]])
def test_fused_mlp_matches_fp32_restatement(sizes):
    from kraken_b200.models.mlp import MLP
    from kraken_b200.ops.mlp import check_gemm_status
    torch.manual_seed(5)
    K, M = 432, 1000
    mlp = MLP(K, sizes).to(DEV)
    assert mlp.use_tensor_cores
    ws = [l.weight.detach().clone() for l in mlp.layers]
    bs = [l.bias.detach().clone() for l in mlp.layers]
    x = torch.randn(M, K, device=DEV)
    x1 = x.clone().requires_grad_(True)
    out = mlp(x1)
    g = torch.randn_like(out)
    want, dws, dbs, dx = emulate(x, ws, bs, g)
    assert out.dtype == torch.float32 and out.shape == want.shape
    ok, info = close(out, want, tol=3e-2, row_tol=0.15)
    assert ok, info
    out.backward(g)
    check_gemm_status(torch.device(DEV, torch.cuda.current_device()))
    for layer, dw, db in zip(mlp.layers, dws, dbs):
        ok, info = close(layer.weight.grad, dw, tol=3e-2, row_tol=0.15)
        assert ok, info
        ok, info = close(layer.bias.grad, db, tol=3e-2, row_tol=0.15)
        assert ok, info
    ok, info = close(x1.grad, dx, tol=3e-2, row_tol=0.15)
    assert ok, info
    # against plain fp32 torch the only extra differences are ReLU gates that flip for
    # pre-activations within bf16 rounding of zero: compare in the Frobenius norm
    ref = MLP(K, sizes, use_tensor_cores=False).to(DEV)
    ref.load_state_dict(mlp.state_dict())
    ref(x).backward(g)
    for a, b in zip(mlp.parameters(), ref.parameters()):
        assert (a.grad - b.grad).norm().item() <= 0.15 * b.grad.norm().item()
    # a second backward accumulates into the same gradient buffers
    mlp(x).backward(g)
    for layer, dw in zip(mlp.layers, dws):
        ok, info = close(layer.weight.grad, 2 * dw, tol=3e-2, row_tol=0.15)
        assert ok, info


def test_fused_mlp_with_odd_width_head():
    """A 10-class head: hidden layers on the tensor cores, the head as a small fp32 matmul."""
    from kraken_b200.models.mlp import MLP
    torch.manual_seed(6)
    mlp = MLP(784, [256, 128, 10]).to(DEV)
    assert mlp.use_tensor_cores
    ws = [l.weight.detach().clone() for l in mlp.layers]
    bs = [l.bias.detach().clone() for l in mlp.layers]
    x = torch.randn(500, 784, device=DEV)
    out = mlp(x)
    g = torch.randn_like(out)
    r = lambda t: t.to(torch.bfloat16).float()
    h0 = r(x)
    h1 = r((h0 @ r(ws[0]).t() + bs[0]).relu())
    h2 = r((h1 @ r(ws[1]).t() + bs[1]).relu())
    want = h2 @ ws[2].t() + bs[2]
    ok, info = close(out, want, tol=1e-2)
    assert ok, info
    out.backward(g)
    ok, info = close(mlp.layers[2].weight.grad, g.t() @ h2, tol=1e-2)
    assert ok, info
    dh2 = r((g @ ws[2]) * (h2 > 0))
    ok, info = close(mlp.layers[1].weight.grad, dh2.t() @ h1, tol=2e-2)
    assert ok, info


@pytest.mark.parametrize("M,K", [(5000, 400), (8192, 32), (300, 20), (65536, 400)])
@pytest.mark.parametrize("relu", [False, True])
def test_rowdot_backward(M, K, relu):
    """Head layer (K -> 1) backward: wide (16-byte) kernel for K % 8 == 0, narrow kernel otherwise."""
    torch.manual_seed(4)
    x = rnd(M, K)
    w = torch.randn(K, device=DEV) * 0.1
    dy = torch.randn(M, device=DEV) * 0.01
    dx = torch.empty_like(x)
    dw = torch.zeros(K, device=DEV)
    db = torch.zeros(1, device=DEV)
    C.rowdot_backward(x, w, dy, relu, dx, dw, db)
    want_dx = dy[:, None] * w[None, :]
    if relu:
        want_dx = want_dx * (x.float() > 0)
    ok, info = close(dx, want_dx)
    assert ok, info
    want_dw = dy @ x.float()
    assert (dw - want_dw).abs().max().item() <= 1e-3 * (want_dw.abs().max().item() + 1e-6) + 1e-5
    assert abs(db.item() - dy.sum().item()) < 1e-3

"""Small driver that launches the MLP GEMM kernels a few times on one shape; used as the
command under ``ncu`` when profiling them (python -m kraken_b200.benchmarks.gemm_case)."""
import argparse

import torch

from kraken_b200._native import C


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--m", type=int, default=65536)
    p.add_argument("--n", type=int, default=400)
    p.add_argument("--k", type=int, default=432)
    p.add_argument("--op", default="forward", choices=["forward", "dgrad", "wgrad"])
    p.add_argument("--reps", type=int, default=3)
    p.add_argument("--bits", action="store_true", help="dgrad: ReLU mask as one bit per element instead of the activations")
    p.add_argument("--rotate", type=int, default=1, help="number of operand sets to rotate over")
    p.add_argument("--n-tiles", type=int, default=0, help="column tiles of the weight-resident variants (0 = auto)")
    p.add_argument("--variant", type=int, default=0, help="0 auto, 1 CTA pair, 2 single-CTA resident, 3 tile per CTA")
    a = p.parse_args()
    dev = "cuda"
    C.gemm_set_tuning(a.variant, a.n_tiles)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    x = torch.randn(a.m, a.k, device=dev).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device=dev) * 0.05).to(torch.bfloat16)
    b = torch.randn(a.n, device=dev)
    y = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(a.m, a.n, device=dev).to(torch.bfloat16)
    wt = w.t().contiguous()
    dx = torch.empty(a.m, a.k, device=dev, dtype=torch.bfloat16)
    dw = torch.zeros(a.n, a.k, device=dev)
    # back-to-back launches inside one event pair (the host runs ahead of the device, so launch latency
    # is not in the figure), rotating over several input/output sets so every launch finds its operands
    # in HBM rather than in the 126 MB L2
    sets = max(1, a.rotate)
    xs = [x] + [x.clone() for _ in range(sets - 1)]
    ys = [y] + [torch.empty_like(y) for _ in range(sets - 1)]
    dys = [dy] + [dy.clone() for _ in range(sets - 1)]
    dxs = [dx] + [torch.empty_like(dx) for _ in range(sets - 1)]

    masks = [torch.randint(-32768, 32767, ((a.k + 15) // 16, (a.m + 63) // 64 * 64), dtype=torch.int16, device=dev) for _ in range(sets)]

    def run(i):
        j = i % sets
        if a.op == "forward":
            C.linear_forward(xs[j], w, b, True, ys[j], st)
        elif a.op == "dgrad":
            if a.bits:
                C.linear_dgrad(dys[j], wt, None, dxs[j], st, masks[j])
            else:
                C.linear_dgrad(dys[j], wt, xs[j], dxs[j], st)
        else:
            C.linear_wgrad(dys[j], xs[j], dw, st)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    e0.record()
    for i in range(a.reps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.reps
    flops = 2.0 * a.m * a.n * a.k
    print(f"{a.op} M={a.m} N={a.n} K={a.k} variant={a.variant} n_tiles={a.n_tiles}: {us:.1f} us per launch over {a.reps} "
          f"launches, {flops / us / 1e6:.0f} TFLOP/s, status {st.item()}")


if __name__ == "__main__":
    main()

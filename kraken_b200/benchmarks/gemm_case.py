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
    a = p.parse_args()
    dev = "cuda"
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    x = torch.randn(a.m, a.k, device=dev).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device=dev) * 0.05).to(torch.bfloat16)
    b = torch.randn(a.n, device=dev)
    y = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(a.m, a.n, device=dev).to(torch.bfloat16)
    wt = w.t().contiguous()
    dx = torch.empty(a.m, a.k, device=dev, dtype=torch.bfloat16)
    dw = torch.zeros(a.n, a.k, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(a.reps):
        e0.record()
        if a.op == "forward":
            C.linear_forward(x, w, b, True, y, st)
        elif a.op == "dgrad":
            C.linear_dgrad(dy, wt, x, dx, st)
        else:
            C.linear_wgrad(dy, x, dw, st)
        e1.record()
        torch.cuda.synchronize()
    print(f"{a.op} M={a.m} N={a.n} K={a.k}: {e0.elapsed_time(e1) * 1e3:.1f} us, status {st.item()}")


if __name__ == "__main__":
    main()

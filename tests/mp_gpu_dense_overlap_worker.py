"""Child process of test_gpu_multi.py / test_gpu_engine.py: a dense MLP trained for a few steps with its
parameters in several buckets that are stepped DURING the backward pass (overlap_dense_step=True, small
dense_bucket_elems) must end with the same weights as the same run with one bucket stepped after it."""
import sys

import torch

import kraken_b200.pytorch as kk
from kraken_b200.models.mlp import MLP


def run(overlap: bool, bucket_elems: int):
    kk.initialize("gpu", seed=0, overlap_dense_step=overlap, dense_bucket_elems=bucket_elems)
    eng = kk.native.engine()
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model = MLP(64, [128, 96, 72, 10]).to(dev)       # hidden layers on the tcgen05 path, a 10-wide head on torch ops
    assert model.use_tensor_cores
    opt = kk.Optimizer("mlp", model.named_parameters(), 0.05, kk.SGD(momentum=0.9))
    g = torch.Generator().manual_seed(100 + eng.rank)
    for _ in range(4):
        x = torch.randn(512, 64, generator=g).to(dev)
        y = torch.randint(0, 10, (512,), generator=g).to(dev)
        loss = torch.nn.functional.cross_entropy(model(x), y) / eng.world
        loss.backward()
        opt.step()
    torch.cuda.synchronize()
    eng.check()
    n_buckets = len(eng.bucket.buckets)
    out = [p.detach().clone() for p in model.parameters()]
    kk.stop(keep_process_group=True)   # the second run reuses the NCCL group of the first
    return out, n_buckets


base, nb0 = run(False, 1 << 30)
over, nb1 = run(True, 1 << 10)
assert nb0 == 1 and nb1 >= 4, (nb0, nb1)
worst = max(float((a - b).abs().max()) for a, b in zip(base, over))
assert worst < 2e-5, worst
moved = max(float(p.abs().max()) for p in base)
assert moved > 0
print(f"DENSE_OVERLAP ok buckets={nb1} worst_diff={worst:.2e}", flush=True)
kk.stop()
sys.exit(0)

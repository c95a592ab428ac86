"""Child process of test_gpu_multi.py: the combined (several tables, one exchange) calls on N GPU ranks;
every table must equal one CPU shard fed all ranks' ids and gradients."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import kraken_b200.pytorch as kk  # noqa: E402
from test_gpu_engine import _combined_scenario  # noqa: E402

kk.initialize("gpu", table_capacity=1 << 12, seed=0)
eng = kk.native.engine()
_combined_scenario(torch.device("cuda", torch.cuda.current_device()), eng.rank, eng.world, steps=4)
if eng.rank == 0:
    print("MULTI_GPU_COMBINED ok", flush=True)
kk.stop()

"""Multi-GPU runs of the fused exchange kernels (need >= 2 GPUs in one box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(script, world, *args, timeout=600):
    port = 29800 + (os.getpid() % 150)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(REPO, "tests", script), *args]
    env = dict(os.environ, PYTHONPATH=REPO, NCCL_NVLS_ENABLE="0", KRAKEN_B200_NO_BUILD="1")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-5000:]
    return res.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gpu_ranks_match_one_shard(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = run_ranks("mp_gpu_worker.py", world, str(tmp_path))
    for tag in ("MULTI_GPU_MATCHES_SINGLE ok", "MULTI_GPU_BAGS ok", "MULTI_GPU_CHECKPOINT_LOAD ok",
                "MULTI_GPU_CHECKPOINT_RESHARD ok"):
        assert tag in out, out[-2000:]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_back_to_back_exchanges_match_one_shard(world):
    """50 pull/push steps on two tables with no dense step, host sync or other collective between them
    (half eager, half CUDA-graph replays), 200 k skewed ids per rank: every row must match the CPU shard."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = run_ranks("mp_gpu_stress_worker.py", world, "200000", "50", timeout=900)
    assert "MULTI_GPU_STRESS ok" in out, out[-2000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_combined_tables_one_exchange_across_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = run_ranks("mp_gpu_combined_worker.py", world)
    assert "MULTI_GPU_COMBINED ok" in out, out[-2000:]


@pytest.mark.parametrize("world", [1, 2, 4])
def test_bucketed_dense_step_during_backward_matches_single_bucket(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = run_ranks("mp_gpu_dense_overlap_worker.py", world)
    assert "DENSE_OVERLAP ok" in out, out[-2000:]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_live_reshard_halves_and_restores_the_owners(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = run_ranks("mp_gpu_reshard_worker.py", world)
    assert "LIVE_RESHARD ok" in out, out[-2000:]


def test_nccl_baseline_exchange_matches_one_shard(tmp_path):
    """The NCCL-only path must give the same tables as the fused path's oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = run_ranks("mp_gpu_worker.py", 2, str(tmp_path), "nccl")
    assert "MULTI_GPU_MATCHES_SINGLE ok" in out, out[-2000:]

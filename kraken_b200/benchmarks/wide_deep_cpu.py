"""Wide&Deep on the CPU: 1 parameter-server shard + 1 worker, fp32, 200 steps, batch 512, 26 single-hot
fields with Zipf(1.05) ids over 1e5 per field, server-side Adagrad lr 0.01 with initial accumulator 0.1.
Prints train samples/s.

    python -m kraken_b200.benchmarks.wide_deep_cpu [--steps 200] [--deployment inproc|tcp] [--impl ours|reference]

``--deployment inproc``: shard and worker in one process (the gloo engine at world size 1).
``--deployment tcp``: ``scheduler_server`` and one ``ps_server`` as separate processes on localhost, the worker
reaches them through ``initialize("tcp://...")`` - the topology of the reference's deployment.
``--impl reference``: the same configuration on the unmodified reference (its scheduler, one ps_server and one
worker over localhost ZeroMQ; needs ``python baseline/build_reference.py`` to have been run).
"""
import argparse
import os
import socket
import subprocess
import sys
import time

import torch

import kraken_b200.pytorch as kk
from kraken_b200.benchmarks.common import emit
from kraken_b200.models import ClickDataset, WideAndDeep
from kraken_b200.ops import bce_with_logits

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _start_servers():
    """scheduler_server + one ps_server as child processes; returns (scheduler address, processes)."""
    from kraken_b200.runtime.rpc import Connecter, Rpc
    # the servers' work per request is small: two threads each, so that they do not fight the worker's
    # math threads for the same cores (the worker keeps two cores free for them, see main)
    env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", OMP_NUM_THREADS="2",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    sp, pp = _free_port(), _free_port()
    procs = [subprocess.Popen([sys.executable, "-m", "kraken_b200.launch.scheduler_server", "--port", str(sp)], env=env)]

    def nodes() -> int:
        c = Connecter(f"127.0.0.1:{sp}", timeout_ms=1000)
        try:
            return len(c.call(Rpc.FETCH_ROUTER)[0]["nodes"])
        finally:
            c.close()

    def wait(cond):
        t0 = time.monotonic()
        while time.monotonic() - t0 < 120:
            try:
                if cond():
                    return
            except (ConnectionError, OSError):
                pass
            time.sleep(0.2)
        raise RuntimeError("the server processes did not come up")

    wait(lambda: nodes() >= 0)
    procs.append(subprocess.Popen([sys.executable, "-m", "kraken_b200.launch.ps_server", "--port", str(pp), "--addr",
                                   f"127.0.0.1:{pp}", "--s_addr", f"127.0.0.1:{sp}"], env=env))
    wait(lambda: nodes() == 1)
    return f"127.0.0.1:{sp}", procs


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--batch", type=int, default=512)
    p.add_argument("--deployment", choices=("inproc", "tcp"), default="inproc")
    p.add_argument("--impl", choices=("ours", "reference"), default="ours")
    p.add_argument("--combine", action="store_true",
                   help="wide and deep tables through one CombineEmbedding (one request round per step and direction, as "
                        "the reference arm's model does)")
    p.add_argument("--async-push", action="store_true",
                   help="tcp deployment: pushes are applied behind the worker's back (the reference's fire-and-forget mode)")
    a = p.parse_args()
    if a.impl == "reference":
        sys.path.insert(0, ROOT)
        from baseline.reference_arm import run_wide_deep_cpu
        emit(run_wide_deep_cpu(a.steps, a.batch))
        return
    torch.manual_seed(0)
    procs = []
    try:
        if a.deployment == "tcp":
            s_addr, procs = _start_servers()
            if "OMP_NUM_THREADS" not in os.environ:
                torch.set_num_threads(max(1, (os.cpu_count() or 4) - 2))   # worker and servers share this host
            kk.initialize(f"tcp://{s_addr}", seed=0, async_push=a.async_push)
        else:
            kk.initialize("cpu", seed=0)
        model = WideAndDeep(26, 13, 8, (256, 128), combine=a.combine)
        opt = kk.Optimizer("wide_deep", model.named_parameters(), 0.01, kk.Adagrad(initial_accumulator_value=0.1))
        data = ClickDataset(26, 13, 100_000, 1.05, seed=0)
        batches = [data.batch(a.batch) for _ in range(a.steps)]
        losses = []
        t0 = time.perf_counter()
        for dense, ids, labels in batches:
            loss = bce_with_logits(model(dense, ids), labels)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        dt = time.perf_counter() - t0
        emit({"benchmark": "wide_deep_cpu", "impl": "ours",
              "engine": "cpu, shard and worker in one process" if a.deployment == "inproc" else
                        "scheduler_server + 1 ps_server + 1 worker as processes, localhost TCP" + (", async pushes" if a.async_push else ""),
              "steps": a.steps, "batch": a.batch, "samples_per_sec": a.steps * a.batch / dt,
              "ms_per_step": dt / a.steps * 1e3, "loss_first10": sum(losses[:10]) / 10,
              "loss_last10": sum(losses[-10:]) / 10, "torch_threads": torch.get_num_threads()})
    finally:
        kk.stop()
        for pr in procs:
            pr.terminate()
        for pr in procs:
            try:
                pr.wait(timeout=20)
            except subprocess.TimeoutExpired:
                pr.kill()


if __name__ == "__main__":
    main()

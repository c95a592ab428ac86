"""Reference arm of bench.py: the UNMODIFIED reference, installed offline under baseline/_ref by
``baseline/build_reference.py``, trained on the benchmark's metric and configuration through its own
public API and stock code path.

What runs: the reference's ``scheduler_server`` and ``--gpus N`` ``ps_server`` processes (its two
executables, kraken/executable/*_main.cc) on localhost, and one worker process
(``baseline/ref_deepfm_worker.py``) that drives ``kraken.pytorch`` the way the reference's DeepFM
example does.  The reference has no GPU code (every entry point rejects CUDA tensors), so all of it
runs on the host CPU in fp32; N only sets the number of parameter-server shards.  None of this
repository's models, kernels or engine is on that path: the worker is a separate process that
imports only baseline/_ref.
"""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import tempfile
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
METRIC = "deepfm_train_samples_per_sec"


def _free_ports(n: int):
    socks, ports = [], []
    for _ in range(n):
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        socks.append(s)
        ports.append(s.getsockname()[1])
    for s in socks:
        s.close()
    return ports


def _installed() -> str:
    for need in ("kraken_native.so", os.path.join("bin", "ps_server"), os.path.join("bin", "scheduler_server"),
                 os.path.join("kraken", "pytorch", "__init__.py")):
        if not os.path.exists(os.path.join(_REF, need)):
            return f"baseline/_ref/{need} is missing (run python baseline/build_reference.py)"
    return ""


def _emit(obj) -> None:
    print(json.dumps(obj), flush=True)


def run(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return  # launched once per GPU: one line for the whole job
    why = _installed()
    if why:
        _emit({"impl": "reference", "unavailable": why})
        return
    steps = args.steps
    n_ps = max(1, int(args.gpus))
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(_REF, "lib") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    env.pop("PYTHONPATH", None)
    ports = _free_ports(1 + n_ps)
    s_addr = f"127.0.0.1:{ports[0]}"
    procs = []
    logdir = os.environ.get("KRAKEN_REF_LOG_DIR") or os.path.join(tempfile.gettempdir(), "kraken_reference_logs")
    os.makedirs(logdir, exist_ok=True)
    logs = []

    def spawn(cmd, name):
        f = open(os.path.join(logdir, f"reference_{name}.log"), "w")
        logs.append(f)
        p = subprocess.Popen(cmd, env=env, stdout=f, stderr=subprocess.STDOUT)
        procs.append(p)
        return p

    try:
        spawn([os.path.join(_REF, "bin", "scheduler_server"), f"--port={ports[0]}"], "scheduler")
        time.sleep(1.0)
        for k in range(n_ps):
            # servers join one at a time: the reference's scheduler refuses a join while another is in flight
            spawn([os.path.join(_REF, "bin", "ps_server"), f"--port={ports[1 + k]}", "--thread_nums=8",
                   f"--addr=127.0.0.1:{ports[1 + k]}", f"--s_addr={s_addr}"], f"ps{k}")
            time.sleep(2.0)
        for p in procs:
            if p.poll() is not None:
                _emit({"impl": "reference", "unavailable": f"a reference server process exited at start-up (code {p.returncode})"})
                return
        cores = os.cpu_count() or 8
        n_workers = int(os.environ.get("KRAKEN_REF_WORKERS", "0")) or max(1, min(8, cores // 8))
        micro = int(os.environ.get("KRAKEN_REF_MICRO_BATCH", "4096"))
        # warm-up plus timed steps stop after this long (a step is a whole 65536-sample batch: 7-8 s on one server);
        # the record then carries the steps that were finished and says so
        deadline = float(os.environ.get("KRAKEN_REF_DEADLINE_S", "600"))
        threads = max(1, min(16, (cores - 4 * n_ps) // n_workers))
        t0 = time.perf_counter()
        workers = []
        for w in range(n_workers):
            workers.append(subprocess.Popen(
                [sys.executable, os.path.join(_HERE, "ref_deepfm_worker.py"), "--ref-path", _REF, "--s-addr", s_addr,
                 "--steps", str(steps), "--warmup", str(args.warmup), "--global-batch", str(args.global_batch),
                 "--workers", str(n_workers), "--worker-index", str(w), "--micro-batch", str(micro),
                 "--deadline-s", str(deadline), "--torch-threads", str(threads)],
                env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        lines, fails = [], []
        for w, p in enumerate(workers):
            out, err = p.communicate()
            line = None
            for ln in out.splitlines():
                if ln.startswith("{") and '"worker"' in ln:
                    line = json.loads(ln)
            if p.returncode != 0 or line is None:
                tail = [t for t in (err or out or "").strip().splitlines() if "Error" in t or "error" in t][-2:]
                fails.append(f"worker {w} exit {p.returncode}: " + " | ".join(tail)[:300])
            else:
                lines.append(line)
        wall = time.perf_counter() - t0
        if fails:
            _emit({"impl": "reference", "unavailable": "reference worker failed: " + "; ".join(fails)[:600]})
            return
        # every worker trained `samples` samples in `seconds`; the job's rate is the sum of the workers' rates
        # over the slowest worker's time (max over ranks)
        sec = max(l["seconds"] for l in lines)
        done = min(l["steps"] for l in lines)
        samples = sum(l["samples"] for l in lines)
        value = samples / sec
        ms = sec / max(1, done) * 1e3
        rec = {
            "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": int(args.gpus),
            "steps": done, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"model": "DeepFM 26x1e7 dim16 + MLP 400-400-400-1, Adam lr 1e-3",
                       "tables": "dim-16 embedding + dim-1 first-order, one CombineEmbedding request round",
                       "global_batch": args.global_batch, "seq_len": 26,
                       "parallelism": f"{n_workers} workers x micro-batch {lines[0]['micro_batch']} "
                                      f"({lines[0]['micro_steps_per_step']} per worker and step) + {n_ps} parameter-server "
                                      "processes + scheduler over localhost ZeroMQ, CPU only",
                       "why_micro_batches": "the reference's 5000 ms RPC timeout rejects a pull for a whole 65536-sample batch",
                       "device": "host CPU (the reference has no GPU code)", "torch_threads_per_worker": lines[0].get("torch_threads"),
                       "build": "offline against the dependency stand-ins under baseline/standins; reference sources unmodified"},
            # the reference's inputs never leave the host, so the end-to-end figure is the same wall-clock measurement
            "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "ms_per_step": ms},
            "gpu_launches": 0, "final_loss": lines[0].get("final_loss"), "wall_s_including_setup": wall,
        }
        if done < steps:
            rec["truncated"] = f"stopped after {done} of {steps} steps at the {deadline:.0f} s deadline"
        _emit(rec)
    finally:
        for p in procs:
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                p.kill()
        for f in logs:
            f.close()


def run_wide_deep_cpu(steps: int = 200, batch: int = 512, torch_threads: int = 0) -> dict:
    """The CPU Wide&Deep configuration on the reference: its scheduler, ONE ps_server and one worker process
    (baseline/ref_wide_deep_worker.py) over localhost.  Returns the worker's record, or {"unavailable": why}."""
    why = _installed()
    if why:
        return {"impl": "reference", "unavailable": why}
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(_REF, "lib") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    env.pop("PYTHONPATH", None)
    ports = _free_ports(2)
    s_addr = f"127.0.0.1:{ports[0]}"
    procs = []
    try:
        procs.append(subprocess.Popen([os.path.join(_REF, "bin", "scheduler_server"), f"--port={ports[0]}"], env=env,
                                      stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL))
        time.sleep(1.0)
        procs.append(subprocess.Popen([os.path.join(_REF, "bin", "ps_server"), f"--port={ports[1]}", "--thread_nums=2",
                                       f"--addr=127.0.0.1:{ports[1]}", f"--s_addr={s_addr}"], env=env,
                                      stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL))
        time.sleep(2.0)
        if any(p.poll() is not None for p in procs):
            return {"impl": "reference", "unavailable": "a reference server process exited at start-up"}
        w = subprocess.run([sys.executable, os.path.join(_HERE, "ref_wide_deep_worker.py"), "--ref-path", _REF,
                            "--s-addr", s_addr, "--steps", str(steps), "--batch", str(batch),
                            "--torch-threads", str(torch_threads)], env=env, capture_output=True, text=True, timeout=1800)
        for ln in w.stdout.splitlines():
            if ln.startswith("{") and "wide_deep_cpu" in ln:
                return json.loads(ln)
        tail = [t for t in (w.stderr or w.stdout).strip().splitlines() if "rror" in t][-2:]
        return {"impl": "reference", "unavailable": f"reference worker exit {w.returncode}: " + " | ".join(tail)[:400]}
    finally:
        for p in procs:
            if p.poll() is None:
                p.terminate()
        for p in procs:
            try:
                p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                p.kill()

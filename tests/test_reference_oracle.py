"""Optimizers, bag pooling and DCT compression against the reference itself.  Optimizers: the same pushes go to the UNMODIFIED reference
(one cluster per configuration, baseline/ref_optim_worker.py) and to this framework's CPU shard, whose
element-wise math (csrc/core/optim_math.h) is the one the CUDA kernels compile too.  Needs the offline
reference build; skipped where that is absent.  Reference math: kraken/ps/optim/{sgd,adagrad,adam,rmsprop}.cc."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from kraken_b200._native import C
from test_reference_checkpoint_compat import REF, ROOT, ReferenceCluster

pytestmark = pytest.mark.skipif(
    not (os.path.exists(os.path.join(REF, "bin", "ps_server")) and os.path.exists(os.path.join(REF, "kraken_native.so"))),
    reason="the reference is not built here (python baseline/build_reference.py)")

CASES = [
    ("SGD", {}),
    ("SGD", {"momentum": "0.9", "dampening": "0.1", "weight_decay": "0.01"}),
    ("SGD", {"momentum": "0.9", "nesterov": "true"}),
    ("Adagrad", {"weight_decay": "0.01", "eps": "1e-6"}),
    ("Adam", {}),
    ("Adam", {"amsgrad": "true", "weight_decay": "0.02", "beta1": "0.8", "beta2": "0.99"}),
    ("RMSprop", {}),
    ("RMSprop", {"centered": "true", "momentum": "0.9", "weight_decay": "0.01", "alpha": "0.95"}),
]


@pytest.mark.parametrize("optim,conf", CASES, ids=[f"{o}-{'-'.join(sorted(c)) or 'default'}" for o, c in CASES])
def test_optimizer_follows_the_reference_step_by_step(optim, conf, tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_optim_worker as w
    finally:
        sys.path.pop(0)
    cluster = ReferenceCluster(str(tmp_path / "scratch"), n_ps=1)
    try:
        import subprocess
        out = str(tmp_path / "oracle.npz")
        run = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "ref_optim_worker.py"), "--ref-path", REF,
                              "--s-addr", cluster.s_addr, "--optim", optim, "--conf", json.dumps(conf), "--out", out],
                             env=cluster.env, capture_output=True, text=True, timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
        want = dict(np.load(out))
    finally:
        cluster.stop()

    shard = C.CpuShard(0)
    shard.init_model("oracle", getattr(C.OptimType, "k" + optim), conf)
    shard.create_sparse_table(0, "e", w.DIM, C.InitializerType.kConstant, {"value": "0.5"})
    shard.create_dense_table(1, "w", torch.linspace(-1, 1, 15).view(3, 5))
    ids, sparse, dense, lrs = w.inputs()
    probe = torch.arange(w.ROWS, dtype=torch.int64) * 11
    shard.pull_sparse(0, probe)
    for k in range(w.STEPS):
        uniq, inv = C.cpu_dedup(ids[k])
        shard.push_sparse(0, uniq, C.cpu_segment_sum(sparse[k], inv, uniq.numel()), lrs[k])
        shard.push_dense(1, dense[k].reshape(-1), lrs[k])
        got_rows = shard.pull_sparse(0, probe).numpy()
        got_dense = shard.pull_dense(1).numpy().reshape(3, 5)
        assert np.allclose(got_rows, want[f"rows_{k}"], rtol=2e-5, atol=2e-6), (optim, conf, k)
        assert np.allclose(got_dense, want[f"dense_{k}"], rtol=2e-5, atol=2e-6), (optim, conf, k)


def test_jagged_pooling_follows_the_reference(tmp_path):
    """Bag pooling against the reference's own CPU ops (kraken/pytorch/py/jagged_ops.cc): sum and mean forward
    with an empty bag and a patch value, mean backward.  The reference's sum backward writes only the first
    row of every bag and leaves the rest uninitialised (jagged_ops.cc:147-200); here every row of a bag gets the
    bag's gradient, so only those first rows are compared."""
    import subprocess
    out = str(tmp_path / "jagged.npz")
    code = f"""
import sys, numpy as np, torch
sys.path.insert(0, {REF!r})
import kraken_native as kn
g = torch.Generator().manual_seed(3)
values = torch.randn(23, 6, generator=g)
offsets = torch.tensor([0, 4, 4, 9, 10, 23], dtype=torch.int64)
grads = torch.randn(5, 6, generator=g)
np.savez({out!r}, sum_f=kn.jagged_sum_forward(values, offsets, -2.5).numpy(),
         mean_f=kn.jagged_mean_forward(values, offsets, 0.25).numpy(),
         mean_b=kn.jagged_mean_backward(offsets, grads).numpy(),
         sum_b=kn.jagged_sum_backward(offsets, grads).numpy())
"""
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(REF, "lib") + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
    env.pop("PYTHONPATH", None)
    run = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
    want = dict(np.load(out))
    g = torch.Generator().manual_seed(3)
    values = torch.randn(23, 6, generator=g)
    offsets = torch.tensor([0, 4, 4, 9, 10, 23], dtype=torch.int64)
    grads = torch.randn(5, 6, generator=g)
    assert np.allclose(C.jagged_sum_forward(values, offsets, -2.5).numpy(), want["sum_f"], atol=1e-6)
    assert np.allclose(C.jagged_mean_forward(values, offsets, 0.25).numpy(), want["mean_f"], atol=1e-6)
    assert np.allclose(C.jagged_mean_backward(offsets, grads).numpy(), want["mean_b"], atol=1e-6)
    ours = C.jagged_sum_backward(offsets, grads).numpy()
    firsts = [0, 4, 9, 10]                      # first row of every non-empty bag
    assert np.allclose(ours[firsts], want["sum_b"][firsts], atol=1e-6)
    assert np.allclose(ours[5], grads[2].numpy(), atol=1e-6)    # a later row of bag 2 carries the bag's gradient too


def test_dct_compression_follows_the_reference(tmp_path):
    """Dynamic communication thresholding against the reference's own emitter (kraken/worker/dct_emitter.cc:16-43):
    the same 8 gradients through both, life span 3, eta 0.75, SGD on the server.  After every push the table
    must hold the same values - which entries crossed, what stayed behind as error feedback, when the threshold
    was refreshed - for a table above the 256-element limit and one below it."""
    import subprocess

    import kraken_b200.pytorch as kk
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_dct_worker as w
    finally:
        sys.path.pop(0)
    cluster = ReferenceCluster(str(tmp_path / "scratch"), n_ps=1)
    try:
        out = str(tmp_path / "dct.npz")
        run = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "ref_dct_worker.py"), "--ref-path", REF,
                              "--s-addr", cluster.s_addr, "--out", out], env=cluster.env, capture_output=True, text=True,
                             timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
        want = dict(np.load(out))
    finally:
        cluster.stop()

    kk.initialize("cpu", kk.EmitterType.kDCT, w.LIFE_SPAN, w.ETA)
    try:
        kk.init_model("dct", kk.OptimType.kSGD, {})
        kk.update_lr(w.LR)
        tb = kk.register_dense_table("big", torch.zeros(*w.BIG))
        ts = kk.register_dense_table("small", torch.zeros(*w.SMALL))
        for k, (gb, gs) in enumerate(w.inputs()):
            kk.push_dense_table(tb, gb)
            kk.push_dense_table(ts, gs)
            assert np.allclose(kk.pull_dense_table(tb).numpy(), want[f"big_{k}"], atol=1e-6), k
            assert np.allclose(kk.pull_dense_table(ts).numpy(), want[f"small_{k}"], atol=1e-6), k
        moved = np.count_nonzero(want["big_0"])
        assert 0 < moved < 0.3 * 1200        # the first push really was sparse: about (1 - eta) of the entries
    finally:
        kk.stop()


def test_row_initialisers_draw_from_the_reference_distributions(tmp_path):
    """The reference seeds its random initialisers from std::random_device (kraken/t/math.cc:455-517), so rows
    cannot be compared one by one; 20 000 new rows of width 16 per initialiser are compared by mean, spread and
    range instead - in particular the Xavier bounds, which depend on how fan-in and fan-out are read off a row."""
    import subprocess

    import kraken_b200.pytorch as kk
    specs = [("constant", "kConstant", {"value": "0.75"}), ("uniform", "kUniform", {"lower": "-0.5", "upper": "1.5"}),
             ("normal", "kNormal", {"mean": "0.3", "stddev": "0.2"}), ("xu", "kXavierUniform", {"gain": "2.0"}),
             ("xn", "kXavierNormal", {"gain": "0.5"})]
    out = str(tmp_path / "init.npz")
    code = f"""
import sys, numpy as np, torch
sys.path.insert(0, {REF!r})
import kraken.pytorch as kk
kk.initialize(sys.argv[1])
kk.init_model("init", kk.OptimType.kSGD, {{}})
res = {{}}
for name, kind, conf in {specs!r}:
    t = kk.register_sparse_table(name, 16, torch.float32, getattr(kk.InitializerType, kind), conf)
    res[name] = kk.pull_sparse_table(t, torch.arange(20000, dtype=torch.int64)).numpy()
np.savez({out!r}, **res)
kk.stop()
"""
    cluster = ReferenceCluster(str(tmp_path / "scratch"), n_ps=1)
    try:
        run = subprocess.run([sys.executable, "-c", code, cluster.s_addr], env=cluster.env, capture_output=True, text=True,
                             timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
        want = dict(np.load(out))
    finally:
        cluster.stop()

    kk.initialize("cpu", seed=4)
    try:
        kk.init_model("init", kk.OptimType.kSGD, {})
        for name, kind, conf in specs:
            t = kk.register_sparse_table(name, 16, torch.float32, getattr(kk.InitializerType, kind), conf)
            got = kk.pull_sparse_table(t, torch.arange(20000)).numpy()
            ref = want[name]
            assert got.shape == ref.shape
            if name == "constant":
                assert np.array_equal(got, ref)
                continue
            n = got.size
            tol = 6 * ref.std() / np.sqrt(n)                   # six standard errors of a mean of n draws
            assert abs(got.mean() - ref.mean()) < 2 * tol, (name, got.mean(), ref.mean())
            assert abs(got.std() / ref.std() - 1) < 0.02, (name, got.std(), ref.std())
            if name in ("uniform", "xu"):                       # bounded: the same support
                assert abs(got.min() - ref.min()) < 0.01 * (ref.max() - ref.min()), (name, got.min(), ref.min())
                assert abs(got.max() - ref.max()) < 0.01 * (ref.max() - ref.min()), (name, got.max(), ref.max())
    finally:
        kk.stop()


def test_the_same_script_trains_the_same_under_both_packages(tmp_path):
    """baseline/dropin_train.py is written against the reference's public API and run twice: once with
    ``kraken.pytorch`` = the unmodified reference (scheduler + server processes), once with ``kraken.pytorch`` =
    this framework behind ``install_alias()``.  Same data, same torch seed, Adam on the servers: the loss of
    every one of the 25 steps and the final dense layers must agree."""
    import subprocess
    script = os.path.join(ROOT, "baseline", "dropin_train.py")
    cluster = ReferenceCluster(str(tmp_path / "scratch"), n_ps=1)
    try:
        ref_out = str(tmp_path / "ref.npz")
        run = subprocess.run([sys.executable, script, "--impl", "reference", "--ref-path", REF, "--s-addr", cluster.s_addr,
                              "--out", ref_out], env=cluster.env, capture_output=True, text=True, timeout=300)
        assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
    finally:
        cluster.stop()
    our_out = str(tmp_path / "ours.npz")
    env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    run = subprocess.run([sys.executable, script, "--impl", "ours", "--s-addr", "cpu", "--out", our_out], env=env,
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
    ref, ours = dict(np.load(ref_out)), dict(np.load(our_out))
    assert ref["losses"].shape == ours["losses"].shape == (25,)
    assert ref["losses"][0] > ref["losses"][-1]                  # it did train
    assert np.allclose(ours["losses"], ref["losses"], rtol=1e-4, atol=1e-5), (ours["losses"], ref["losses"])
    for k in range(6):
        assert np.allclose(ours[f"param_{k}"], ref[f"param_{k}"], rtol=1e-3, atol=1e-5), k


def test_the_references_own_example_model_runs_unmodified_under_the_alias():
    """examples/DeepFM/model/DeepFM.py of the reference - 39 + 39 ``kk.Embedding`` tables, ``kk.Optimizer`` with
    ``kk.Adam()``, its own ``fit`` loop - is imported from the reference checkout as it is and trained on the CPU
    engine behind ``install_alias()``.  (Its ``main.py`` cannot run anywhere: the data file it reads,
    ``feature_sizes.txt``, is empty in the checkout.)"""
    import importlib.util
    src = os.path.join(os.environ.get("KRAKEN_REFERENCE_SRC", "/root/reference"), "examples", "DeepFM", "model", "DeepFM.py")
    if not os.path.exists(src):
        pytest.skip("no checkout of the reference here")
    import kraken_b200
    kraken_b200.install_alias()
    import kraken.pytorch as kk
    spec = importlib.util.spec_from_file_location("reference_example_deepfm", src)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    torch.manual_seed(0)
    g = torch.Generator().manual_seed(5)
    fields, n = 39, 64
    batches = []
    for _ in range(6):
        xi = torch.randint(0, 50, (n, fields, 1), generator=g)
        xv = torch.ones(n, fields)
        y = ((xi[:, 0, 0] % 2) == 0).float()            # learnable from the first field
        batches.append((xi, xv, y))

    class Loader(list):
        class dataset:
            train = True

    kk.initialize("cpu", seed=0)
    try:
        model = mod.DeepFM([50] * fields, use_cuda=False)
        optimizer = kk.Optimizer(model_name="DeepFM", named_parameters=model.named_parameters(), optim=kk.Adam(), lr=1e-2)
        assert len(kk.native.engine().tables) >= 2 * fields          # every Embedding became a sparse table
        crit = torch.nn.functional.binary_cross_entropy_with_logits
        model.eval()
        with torch.no_grad():
            before = float(sum(crit(model(xi, xv.float()), y) for xi, xv, y in batches)) / len(batches)
        model.fit(Loader(batches), Loader(batches), optimizer, epochs=15, verbose=False)
        model.eval()
        with torch.no_grad():
            after = float(sum(crit(model(xi, xv.float()), y) for xi, xv, y in batches)) / len(batches)
        assert after < 0.7 * before, (before, after)
    finally:
        kk.stop()

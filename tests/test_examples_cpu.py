"""The example programs (counterparts of the reference's examples/DeepFM, examples/WideAndDeep,
examples/WideAndDeep_Combine and examples/Mnist/kraken) run a few steps on the CPU engine."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,extra", [("deepfm", []), ("wide_deep", []), ("wide_deep_combine", []), ("mnist", []),
                                        ("mnist", ["--dct"])])
def test_example_trains_a_few_steps(name, extra):
    env = dict(os.environ, KRAKEN_B200_NO_BUILD="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    run = subprocess.run([sys.executable, os.path.join(ROOT, "examples", name, "main.py"), "--s_addr", "cpu", "--steps", "6",
                          *extra], env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, (run.stdout + run.stderr)[-2000:]
    assert "loss" in run.stdout

"""Host-side C++ (router, serializer, checkpoint files, CPU shard, reference kernels, task queue, TCP transport)
built with AddressSanitizer + UBSan and with ThreadSanitizer and run as a stand-alone program.
The reference has no sanitizer job (its CMakeLists.txt:54-55 sets -O3 / -O0 -g only)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "kraken_b200", "csrc")
SOURCES = [os.path.join(ROOT, "tests", "host_selftest_src", "host_selftest.cc"), "core/router.cc", "core/checkpoint.cc", "core/net.cc", "cpu/cpu_shard.cc", "cpu/cpu_ops.cc"]


@pytest.mark.parametrize("name,flags", [("asan_ubsan", "-fsanitize=address,undefined"), ("tsan", "-fsanitize=thread")])
def test_host_code_is_clean_under_sanitizers(tmp_path, name, flags):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = tmp_path / f"host_selftest_{name}"
    cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-Wno-unknown-pragmas", "-I", CSRC, *flags.split(),
           *SOURCES, "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "cannot find" in build.stderr and "san" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1",
               TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([str(exe), str(tmp_path / "ckpt")], capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "host selftest: ok" in run.stdout
    assert "Sanitizer" not in run.stderr, run.stderr[-3000:]

#!/usr/bin/env python
"""Offline install of the UNMODIFIED reference into baseline/_ref.

The reference's CMake build fetches its third-party projects from the network at configure time
(cmake/*.cmake use FetchContent with SOURCE_DIR third_party/<name>).  Here a copy of the reference
tree is made under /tmp, its ``third_party/`` directory - which the reference itself does not ship -
is populated with the stand-ins of ``baseline/standins`` (dependencies only; every reference source
file stays byte-identical, which the recorded tree hash shows), FetchContent is told through a
toolchain file to use what is there, and the documented pip command installs the result:

    python -m pip install --no-index --no-build-isolation --find-links /opt/wheelhouse \
        --target baseline/_ref /tmp/<copy>

The reference's setup.py installs only the Python extension; the two server executables and the
reference's own test binary are copied from its build tree into baseline/_ref/bin afterwards.

Usage: python baseline/build_reference.py [--reference <checkout of the reference>] [--keep-build]
"""
from __future__ import annotations

import argparse
import glob
import hashlib
import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
STANDINS = os.path.join(HERE, "standins")
TARGET = os.path.join(HERE, "_ref")
NAMES = ["eigen", "libzmq", "snappy", "gflags", "googletest", "configor", "libcuckoo", "pybind11"]


def tree_hash(root: str) -> str:
    """SHA-256 over (relative path, content) of every file below ``root``, in sorted order."""
    h = hashlib.sha256()
    for dirpath, dirnames, filenames in os.walk(root):
        dirnames.sort()
        rel = os.path.relpath(dirpath, root)
        if rel.split(os.sep)[0] in ("third_party", "build", "kraken.egg-info"):
            dirnames[:] = []
            continue
        for fn in sorted(filenames):
            p = os.path.join(dirpath, fn)
            h.update(os.path.relpath(p, root).encode())
            with open(p, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KRAKEN_REFERENCE_SRC", "/root/reference"),
                    help="checkout of the reference (read only; copied before the build)")
    ap.add_argument("--work", default="/tmp/kraken_reference_build")
    ap.add_argument("--keep-build", action="store_true")
    args = ap.parse_args()

    src = os.path.join(args.work, "src")
    if os.path.isdir(args.work):
        shutil.rmtree(args.work)
    os.makedirs(args.work)
    shutil.copytree(args.reference, src, symlinks=True)
    subprocess.check_call(["chmod", "-R", "u+w", src])
    want = tree_hash(args.reference)
    tp = os.path.join(src, "third_party")
    os.makedirs(tp, exist_ok=True)
    for n in NAMES:
        shutil.copytree(os.path.join(STANDINS, n), os.path.join(tp, n))

    env = dict(os.environ)
    env["CMAKE_TOOLCHAIN_FILE"] = os.path.join(STANDINS, "toolchain.cmake")
    # an empty libstdc++fs.a, found before the compiler's own (see toolchain.cmake for the reason)
    libdir0 = os.path.join(args.work, "empty_libs")
    os.makedirs(libdir0)
    subprocess.check_call(["ar", "rcs", os.path.join(libdir0, "libstdc++fs.a")])
    env["KRAKEN_BASELINE_LIBDIR"] = libdir0
    # the distribution's own compiler driver: a wrapper that CC/CXX may name on a build box was seen to
    # link libstdc++ statically into the extension, which then crashed inside the Python process
    if os.path.exists("/usr/bin/g++") and os.path.exists("/usr/bin/gcc"):
        env["CC"], env["CXX"] = "/usr/bin/gcc", "/usr/bin/g++"
    if os.path.isdir(TARGET):
        shutil.rmtree(TARGET)
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
           "/opt/wheelhouse", "--target", TARGET, src]
    log = os.path.join(args.work, "pip_install.log")
    with open(log, "w") as f:
        rc = subprocess.call(cmd, env=env, stdout=f, stderr=subprocess.STDOUT)
    if rc != 0:
        print(f"pip install failed (exit {rc}); see {log}")
        return rc
    got = tree_hash(src)
    if got != want:
        print("reference sources changed during the build: refusing to use the result")
        return 2

    bindir = os.path.join(TARGET, "bin")
    os.makedirs(bindir, exist_ok=True)
    found = {}
    for exe in ("ps_server", "scheduler_server", "kraken_test"):
        hits = glob.glob(os.path.join(src, "build", "**", exe), recursive=True)
        hits = [h for h in hits if os.path.isfile(h) and os.access(h, os.X_OK)]
        if hits:
            shutil.copy2(hits[0], os.path.join(bindir, exe))
            found[exe] = True
    # the shared libraries the stand-in libzmq target links to, kept beside the binaries as a fallback
    # for a machine whose Python environment sits elsewhere
    import zmq  # noqa: PLC0415  (the pyzmq wheel bundles libzmq + libsodium)
    libs = os.path.join(os.path.dirname(os.path.dirname(zmq.__file__)), "pyzmq.libs")
    libdir = os.path.join(TARGET, "lib")
    os.makedirs(libdir, exist_ok=True)
    for p in glob.glob(os.path.join(libs, "*.so*")):
        shutil.copy2(p, libdir)
    with open(os.path.join(TARGET, "BUILD_INFO.json"), "w") as f:
        json.dump({"reference_tree_sha256": want, "standins": NAMES, "executables": sorted(found),
                   "pip_command": " ".join(cmd[1:]), "toolchain_file": "baseline/standins/toolchain.cmake"}, f, indent=1)
    print(f"installed into {TARGET}: kraken_native + {sorted(found)}; reference tree sha256 {want[:16]}... unchanged")
    if not args.keep_build:
        shutil.rmtree(args.work, ignore_errors=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())

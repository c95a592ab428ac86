"""In-tree build of the native extension ``kraken_b200._C``.

Host C++ (hash, router, serializer, checkpoint, CPU shard) and the sm_100a CUDA
kernels are compiled with ninja through ``torch.utils.cpp_extension`` into
``kraken_b200/_ext/_C.so``; a source tree that has been built once can be
moved to another machine and imported without a compiler.

Run ``python -m kraken_b200._build`` (or ``__graft_entry__.build()``).
"""
from __future__ import annotations

import glob
import os
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
_EXT_DIR = os.path.join(_PKG, "_ext")
EXT_NAME = "_C"
SO_PATH = os.path.join(_EXT_DIR, EXT_NAME + ".so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-Wall", "-Wno-unknown-pragmas", "-Wno-unused-function", "-Wno-sign-compare"]


def sources():
    out = []
    for pat in ("*.cc", "core/*.cc", "cpu/*.cc", "cuda/*.cu"):
        out += sorted(glob.glob(os.path.join(_CSRC, pat)))
    return out


def cutlass_include():
    """CUTLASS/CuTe headers vendored inside site-packages (used for reference
    constants only; the kernels are written with inline PTX)."""
    import site

    for sp in site.getsitepackages():
        cand = os.path.join(sp, "flashinfer", "data", "cutlass", "include")
        if os.path.isdir(cand):
            return cand
    return None


def build(verbose: bool = False) -> str:
    from torch.utils import cpp_extension

    os.makedirs(_EXT_DIR, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name=EXT_NAME,
        sources=sources(),
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=["-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lstdc++"],
        extra_include_paths=[_CSRC],
        build_directory=_EXT_DIR,
        with_cuda=True,
        is_python_module=False,
        verbose=verbose,
    )
    if not os.path.exists(SO_PATH):
        raise RuntimeError(f"build did not produce {SO_PATH}")
    return SO_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))

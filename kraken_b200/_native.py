"""Loader of the native extension.

``kraken_b200._C`` is compiled in-tree by ``kraken_b200._build``; importing the
package loads the existing shared object and, if there is none, builds it.
Nothing falls back to pure Python: a missing extension is an error, so a GPU
run can never silently use a slower path.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch  # noqa: F401  (libtorch must be loaded before the extension)

from . import _build


def _load():
    name = __package__ + "._C"
    if name in sys.modules:
        return sys.modules[name]
    if not os.path.exists(_build.SO_PATH):
        if os.environ.get("KRAKEN_B200_NO_BUILD") == "1":
            raise ImportError(f"{_build.SO_PATH} is missing and KRAKEN_B200_NO_BUILD=1")
        _build.build()
    spec = importlib.util.spec_from_file_location(name, _build.SO_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[name] = mod
    return mod


C = _load()

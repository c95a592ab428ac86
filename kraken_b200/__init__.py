"""kraken_b200: a Blackwell-native sparse-embedding training framework with the
capabilities, Python API and checkpoint format of amazingyyc/Kraken.

``import kraken_b200.pytorch as kk`` is the counterpart of the reference's
``import kraken.pytorch as kk``; ``kraken_b200.install_alias()`` additionally
registers the package under the name ``kraken`` so that existing scripts run
unchanged.
"""
import importlib
import importlib.abc
import importlib.util
import sys

__version__ = "0.2.0"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Resolves ``kraken`` / ``kraken.<anything>`` / ``kraken_native`` to the module of the same path in this
    package - the SAME module object, not a second copy of it (a second copy of a submodule would import the
    native library twice)."""

    def _target(self, fullname: str):
        if fullname == "kraken_native":
            return __name__ + ".pytorch.native"
        if fullname == "kraken" or fullname.startswith("kraken."):
            return __name__ + fullname[len("kraken"):]
        return None

    def find_spec(self, fullname, path=None, target=None):
        real = self._target(fullname)
        if real is None:
            return None
        try:
            module = importlib.import_module(real)
        except ModuleNotFoundError:
            return None
        spec = importlib.util.spec_from_loader(fullname, self, is_package=hasattr(module, "__path__"))
        spec._kraken_b200_module = module
        return spec

    def create_module(self, spec):
        return spec._kraken_b200_module

    def exec_module(self, module):   # already executed under its own name
        pass


_finder = _AliasFinder()


def install_alias() -> None:
    """Makes ``import kraken``, ``import kraken.pytorch``, any ``kraken.pytorch.<module>`` of the reference's layout
    and ``import kraken_native`` resolve to this package (a ``kraken`` that was imported before this call stays)."""
    from . import pytorch
    from .pytorch import native

    sys.modules.setdefault("kraken", sys.modules[__name__])
    sys.modules.setdefault("kraken.pytorch", pytorch)
    sys.modules.setdefault("kraken_native", native)
    if _finder not in sys.meta_path:
        sys.meta_path.insert(0, _finder)

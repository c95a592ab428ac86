"""kraken_b200: a Blackwell-native sparse-embedding training framework with the
capabilities, Python API and checkpoint format of amazingyyc/Kraken.

``import kraken_b200.pytorch as kk`` is the counterpart of the reference's
``import kraken.pytorch as kk``; ``kraken_b200.install_alias()`` additionally
registers the package under the name ``kraken`` so that existing scripts run
unchanged.
"""
import sys

__version__ = "0.1.0"


def install_alias() -> None:
    """Makes ``import kraken.pytorch`` and ``import kraken_native`` resolve to this package."""
    from . import pytorch
    from .pytorch import native

    sys.modules.setdefault("kraken", sys.modules[__name__])
    sys.modules.setdefault("kraken.pytorch", pytorch)
    sys.modules.setdefault("kraken_native", native)

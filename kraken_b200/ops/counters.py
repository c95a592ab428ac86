"""Count of this package's own kernel launches made through the ops wrappers
(model kernels and tcgen05 GEMMs); the engines count their exchange kernels."""
_n = [0]


def add(k: int = 1) -> None:
    _n[0] += k


def launches() -> int:
    return _n[0]

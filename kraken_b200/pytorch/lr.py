"""Learning-rate schedules (interface of kraken/pytorch/lr.py:4-26)."""


class LR(object):
    def step(self):
        raise NotImplementedError

    def lr(self) -> float:
        raise NotImplementedError


class ConstantLR(LR):
    def __init__(self, lr: float):
        self._lr = float(lr)

    def step(self):
        pass

    def lr(self) -> float:
        return self._lr


class StepLR(LR):
    """lr * gamma ** (steps // step_size)."""

    def __init__(self, lr: float, step_size: int, gamma: float = 0.1):
        self._base, self._size, self._gamma, self._n = float(lr), int(step_size), float(gamma), 0

    def step(self):
        self._n += 1

    def lr(self) -> float:
        return self._base * self._gamma ** (self._n // self._size)

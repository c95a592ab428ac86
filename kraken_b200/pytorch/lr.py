"""Learning-rate schedules.  The worker owns the rate and sends it along with every push; a schedule is an
object with ``step()`` (called once per optimizer step) and ``lr()`` (the rate to use next) - the interface of
the reference's kraken/pytorch/lr.py:4-26, which ships the constant schedule only."""
import math
from typing import Callable


class LR:
    """Base class: counts steps; subclasses turn the count into a rate in ``rate_at``."""

    def __init__(self) -> None:
        self.steps_done = 0

    def step(self) -> None:
        self.steps_done += 1

    def rate_at(self, n: int) -> float:
        raise NotImplementedError

    def lr(self) -> float:
        return float(self.rate_at(self.steps_done))


class ConstantLR(LR):
    def __init__(self, lr: float) -> None:
        super().__init__()
        self._lr = float(lr)

    def rate_at(self, n: int) -> float:
        return self._lr


class StepLR(LR):
    """lr * gamma ** (n // step_size)."""

    def __init__(self, lr: float, step_size: int, gamma: float = 0.1) -> None:
        super().__init__()
        self._base, self._size, self._gamma = float(lr), int(step_size), float(gamma)

    def rate_at(self, n: int) -> float:
        return self._base * self._gamma ** (n // self._size)


class ExponentialLR(LR):
    """lr * gamma ** n."""

    def __init__(self, lr: float, gamma: float) -> None:
        super().__init__()
        self._base, self._gamma = float(lr), float(gamma)

    def rate_at(self, n: int) -> float:
        return self._base * self._gamma ** n


class WarmupCosineLR(LR):
    """Linear warm-up from 0 to ``lr`` over ``warmup`` steps, then a cosine down to ``floor`` at ``total`` steps."""

    def __init__(self, lr: float, warmup: int, total: int, floor: float = 0.0) -> None:
        super().__init__()
        self._base, self._warm, self._total, self._floor = float(lr), int(warmup), int(total), float(floor)

    def rate_at(self, n: int) -> float:
        if n < self._warm:
            return self._base * (n + 1) / self._warm
        span = max(1, self._total - self._warm)
        t = min(1.0, (n - self._warm) / span)
        return self._floor + 0.5 * (self._base - self._floor) * (1.0 + math.cos(math.pi * t))


class LambdaLR(LR):
    """lr * fn(n) for a user function of the step count."""

    def __init__(self, lr: float, fn: Callable[[int], float]) -> None:
        super().__init__()
        self._base, self._fn = float(lr), fn

    def rate_at(self, n: int) -> float:
        return self._base * float(self._fn(n))

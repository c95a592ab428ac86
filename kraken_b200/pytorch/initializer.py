"""Row initializer descriptors: (type, string conf) pairs that travel to the
shards and into checkpoints (same classes and conf keys as
kraken/pytorch/initializer.py:16-78)."""
from typing import Dict

from .native import InitializerType


class Initializer(object):
    def type(self):
        raise NotImplementedError

    def conf(self) -> Dict[str, str]:
        raise NotImplementedError


class ConstantInitializer(Initializer):
    def __init__(self, value: float = 0.0):
        self._value = value

    def type(self):
        return InitializerType.kConstant

    def conf(self):
        return {"value": str(self._value)}


class UniformInitializer(Initializer):
    def __init__(self, lower: float = 0.0, upper: float = 1.0):
        self._lower, self._upper = lower, upper

    def type(self):
        return InitializerType.kUniform

    def conf(self):
        return {"lower": str(self._lower), "upper": str(self._upper)}


class NormalInitializer(Initializer):
    def __init__(self, mean: float = 0.0, stddev: float = 1.0):
        self._mean, self._stddev = mean, stddev

    def type(self):
        return InitializerType.kNormal

    def conf(self):
        return {"mean": str(self._mean), "stddev": str(self._stddev)}


class XavierUniformInitializer(Initializer):
    def __init__(self, gain: float = 1.0):
        self._gain = gain

    def type(self):
        return InitializerType.kXavierUniform

    def conf(self):
        return {"gain": str(self._gain)}


class XavierNormalInitializer(Initializer):
    def __init__(self, gain: float = 1.0):
        self._gain = gain

    def type(self):
        return InitializerType.kXavierNormal

    def conf(self):
        return {"gain": str(self._gain)}

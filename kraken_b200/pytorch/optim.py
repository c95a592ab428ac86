"""Server-side optimizer descriptors (classes and conf keys of
kraken/pytorch/optim.py:16-143).  Optional keys are emitted only when set, as
the reference does; Adagrad additionally accepts ``initial_accumulator_value``."""
from typing import Dict

from .native import OptimType


def _b(v: bool) -> str:
    return "true" if v else "false"


class Optim(object):
    def type(self):
        raise NotImplementedError

    def conf(self) -> Dict[str, str]:
        raise NotImplementedError


class Adagrad(Optim):
    def __init__(self, weight_decay=None, eps: float = 1e-10, initial_accumulator_value: float = 0.0):
        self._weight_decay, self._eps, self._init_acc = weight_decay, eps, initial_accumulator_value

    def type(self):
        return OptimType.kAdagrad

    def conf(self):
        c = {"eps": str(self._eps)}
        if self._weight_decay:
            c["weight_decay"] = str(self._weight_decay)
        if self._init_acc:
            c["initial_accumulator_value"] = str(self._init_acc)
        return c


class Adam(Optim):
    def __init__(self, weight_decay=None, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-08,
                 amsgrad: bool = False):
        self._weight_decay, self._beta1, self._beta2, self._eps, self._amsgrad = weight_decay, beta1, beta2, eps, amsgrad

    def type(self):
        return OptimType.kAdam

    def conf(self):
        c = {"beta1": str(self._beta1), "beta2": str(self._beta2), "eps": str(self._eps),
             "amsgrad": _b(self._amsgrad)}
        if self._weight_decay:
            c["weight_decay"] = str(self._weight_decay)
        return c


class RMSprop(Optim):
    def __init__(self, weight_decay=None, momentum=None, alpha: float = 0.99, eps: float = 1e-8,
                 centered: bool = False):
        self._weight_decay, self._momentum, self._alpha, self._eps, self._centered = (weight_decay, momentum, alpha,
                                                                                      eps, centered)

    def type(self):
        return OptimType.kRMSprop

    def conf(self):
        c = {"alpha": str(self._alpha), "eps": str(self._eps), "centered": _b(self._centered)}
        if self._weight_decay:
            c["weight_decay"] = str(self._weight_decay)
        if self._momentum:
            c["momentum"] = str(self._momentum)
        return c


class SGD(Optim):
    def __init__(self, momentum=None, dampening=None, weight_decay=None, nesterov: bool = False):
        self._momentum, self._dampening, self._weight_decay, self._nesterov = momentum, dampening, weight_decay, nesterov

    def type(self):
        return OptimType.kSGD

    def conf(self):
        c = {"nesterov": _b(self._nesterov)}
        if self._momentum:
            c["momentum"] = str(self._momentum)
        if self._dampening:
            c["dampening"] = str(self._dampening)
        if self._weight_decay:
            c["weight_decay"] = str(self._weight_decay)
        return c

"""Row initializer descriptors: a kind and string-valued options that travel to the shards and into
checkpoints.  Same class names, constructor arguments and option keys as the reference's
kraken/pytorch/initializer.py:16-78, so model code written for it constructs them unchanged."""
from typing import Dict

from .native import InitializerType


class Initializer:
    """A kind plus named options; subclasses only name their options and defaults."""

    KIND = None

    def __init__(self, **options: float) -> None:
        self._options = dict(options)

    def type(self):
        if self.KIND is None:
            raise NotImplementedError("Initializer is abstract: use one of its subclasses")
        return self.KIND

    def conf(self) -> Dict[str, str]:
        """Options as strings, the form in which the shards and the checkpoint files keep them."""
        return {name: str(value) for name, value in self._options.items()}

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v}" for k, v in self._options.items())
        return f"{type(self).__name__}({inner})"


class ConstantInitializer(Initializer):
    KIND = InitializerType.kConstant

    def __init__(self, value: float = 0.0) -> None:
        super().__init__(value=value)


class UniformInitializer(Initializer):
    KIND = InitializerType.kUniform

    def __init__(self, lower: float = 0.0, upper: float = 1.0) -> None:
        super().__init__(lower=lower, upper=upper)


class NormalInitializer(Initializer):
    KIND = InitializerType.kNormal

    def __init__(self, mean: float = 0.0, stddev: float = 1.0) -> None:
        super().__init__(mean=mean, stddev=stddev)


class XavierUniformInitializer(Initializer):
    KIND = InitializerType.kXavierUniform

    def __init__(self, gain: float = 1.0) -> None:
        super().__init__(gain=gain)


class XavierNormalInitializer(Initializer):
    KIND = InitializerType.kXavierNormal

    def __init__(self, gain: float = 1.0) -> None:
        super().__init__(gain=gain)

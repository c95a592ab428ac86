"""The optimizer facade a training script talks to.

Construction registers the model and every parameter with the engine: sparse
tables by description, dense parameters by value (kraken/pytorch/optimizer.py:16-139).
The optimizer itself runs where the parameters live - on the shard - so
``step()`` only has to make the dense update happen and refresh the local
dense values; ``zero_grad()`` is a no-op (kraken/pytorch/optimizer.py:151-176).

On the GPU engine dense parameters are bound to the engine's flat bucket
(``.data`` and ``.grad`` alias it) and ``step()`` launches one fused
reduce-scatter + optimizer + all-gather kernel.  On the other engines each
dense parameter gets a gradient hook that pushes its gradient, and ``step()``
pulls the updated values, exactly like the reference.
"""
import logging
from typing import Union

import torch

from . import native
from .lr import LR, ConstantLR
from .optim import Optim
from .sparse_table import CombineSparseTable, SparseTable

log = logging.getLogger("kraken_b200")


class Optimizer:
    def __init__(self, model_name: str, named_parameters, lr: Union[float, LR], optim: Optim):
        self._model_name = model_name
        self._lr = ConstantLR(lr=lr) if isinstance(lr, (float, int)) else lr
        self._optim = optim
        self._param_table_id = {}
        self._dense = []  # (param, table_id)
        eng = native.engine()

        native.init_model(model_name, optim.type(), optim.conf())
        log.info("Register model:[%s], optim_type:%s, optim_conf:%s", model_name, optim.type(), optim.conf())
        native.update_lr(self._lr.lr())

        for name, param in named_parameters:
            if not param.requires_grad:
                continue
            if isinstance(param, SparseTable):
                real = param.name() if param.name() is not None else name
                init = param.initializer()
                tid = native.register_sparse_table(name=real, dimension=param.dimension(), dtype=param.dtype(),
                                                   init_type=init.type(), init_conf=init.conf())
                param.set_table_id(tid)
                param.set_name(real)
                self._param_table_id[param] = tid
                log.info("Register SparseTable:[%s], table id:[%d], dimension:[%d]", real, tid, param.dimension())
            elif isinstance(param, CombineSparseTable):
                names, ids = [], []
                for i, dim in enumerate(param.dimensions()):
                    real = param.names()[i] if param.names() is not None else f"{name}.{i}"
                    init = param.initializers()[i]
                    tid = native.register_sparse_table(name=real, dimension=dim, dtype=param.dtypes()[i],
                                                       init_type=init.type(), init_conf=init.conf())
                    names.append(real)
                    ids.append(tid)
                    log.info("Register SparseTable:[%s], table id:[%d], dimension:[%d]", real, tid, dim)
                param.set_names(names)
                param.set_table_ids(ids)
                self._param_table_id[param] = ids
            else:
                tid = native.register_dense_table(name, param.data)
                self._param_table_id[param] = tid
                self._dense.append((param, tid))
                log.info("Register DenseTable:[%s], table id:[%d]", name, tid)

        self._bound = hasattr(eng, "bind_dense_params") and len(self._dense) > 0
        if self._bound:
            eng.bind_dense_params([(tid, p) for p, tid in self._dense])
        else:
            for p, tid in self._dense:
                p.register_hook(self._make_hook(tid))
            self._pull_dense()

    @staticmethod
    def _make_hook(table_id):
        def hook(grad):
            native.push_dense_table(table_id, grad)
            return grad

        return hook

    def _pull_dense(self):
        if not self._dense:
            return
        values = native.combine_pull_dense_table([tid for _, tid in self._dense])
        for (p, _), v in zip(self._dense, values):
            p.data = v.to(p.device) if v.device != p.device else v

    def step(self):
        eng = native.engine()
        if self._bound:
            eng.dense_step()
        else:
            for p, _ in self._dense:
                p.grad = None
            self._pull_dense()
        self.host_step()

    def host_step(self) -> bool:
        """The part of ``step()`` that runs on the host: advances the learning-rate schedule (the new
        value reaches the kernels through the engine's device-side copy) and lets the engine do its
        between-step work (table growth, error words).  A CUDA-graph replay of a step repeats the
        kernels only, so ``GraphedStep`` calls this after every replay; True means a table was
        reallocated and captured graphs must be rebuilt."""
        self._lr.step()
        native.update_lr(self._lr.lr())
        return bool(native.engine().end_step())

    def zero_grad(self):
        pass

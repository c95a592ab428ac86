"""Parameter stand-ins for sparse tables.

A sparse table has no local storage: these are EMPTY ``nn.Parameter``s that
only carry the table description, so that the tables show up in
``model.named_parameters()`` and the ``Optimizer`` can register them (the
device used by kraken/pytorch/sparse_table.py:7-42 and
kraken/pytorch/combine_sparse_table.py:8-57).
"""
from typing import List, Optional

import torch

from .initializer import Initializer, NormalInitializer


class SparseTable(torch.nn.Parameter):
    def __new__(cls, dimension: int, dtype: torch.dtype = torch.float32, initializer: Optional[Initializer] = None,
                name: Optional[str] = None):
        self = super().__new__(cls)
        self._dimension = int(dimension)
        self._dtype = dtype
        self._initializer = initializer if initializer is not None else NormalInitializer()
        self._name = name
        self._table_id = None
        return self

    def dimension(self):
        return self._dimension

    def dtype(self):
        return self._dtype

    def initializer(self):
        return self._initializer

    def name(self):
        return self._name

    def table_id(self):
        return self._table_id

    def set_name(self, name: str):
        self._name = name

    def set_table_id(self, table_id: int):
        self._table_id = table_id

    def __deepcopy__(self, memo):
        return self

    def __repr__(self):
        return f"SparseTable(name={self._name!r}, dimension={self._dimension}, table_id={self._table_id})"


class CombineSparseTable(torch.nn.Parameter):
    def __new__(cls, dimensions: List[int], dtypes: Optional[List[torch.dtype]] = None,
                initializers: Optional[List[Initializer]] = None, names: Optional[List[str]] = None):
        self = super().__new__(cls)
        n = len(dimensions)
        if dtypes is not None and len(dtypes) != n:
            raise ValueError("dtypes must have one entry per table")
        if initializers is not None and len(initializers) != n:
            raise ValueError("initializers must have one entry per table")
        if names is not None and len(names) != n:
            raise ValueError("names must have one entry per table")
        self._dimensions = [int(d) for d in dimensions]
        self._dtypes = list(dtypes) if dtypes is not None else [torch.float32] * n
        self._initializers = list(initializers) if initializers is not None else [NormalInitializer() for _ in range(n)]
        self._names = list(names) if names is not None else None
        self._table_ids = None
        return self

    def dimensions(self):
        return self._dimensions

    def dtypes(self):
        return self._dtypes

    def initializers(self):
        return self._initializers

    def names(self):
        return self._names

    def table_ids(self):
        return self._table_ids

    def set_names(self, names: List[str]):
        self._names = list(names)

    def set_table_ids(self, table_ids: List[int]):
        self._table_ids = list(table_ids)

    def __deepcopy__(self, memo):
        return self

    def __repr__(self):
        return f"CombineSparseTable(names={self._names!r}, dimensions={self._dimensions})"

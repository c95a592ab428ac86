"""``CombineSparseTable`` under the module path the reference keeps it at
(kraken/pytorch/combine_sparse_table.py)."""
from .sparse_table import CombineSparseTable  # noqa: F401

"""``CombineJaggedEmbedding`` under the module path the reference keeps it at
(kraken/pytorch/combine_jagged_embedding.py)."""
from .jagged_embedding import CombineJaggedEmbedding  # noqa: F401

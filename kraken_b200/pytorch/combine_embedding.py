"""``CombineEmbedding`` under the module path the reference keeps it at (kraken/pytorch/combine_embedding.py)."""
from .embedding import CombineEmbedding, CombineEmbeddingFunction  # noqa: F401

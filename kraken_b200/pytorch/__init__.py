"""Drop-in counterpart of the reference's ``kraken.pytorch`` package
(kraken/pytorch/__init__.py:3-35): same names, same call signatures."""
from .native import (CompressType, EmitterType, InitializerType, KrakenError, OptimType, combine_pull_dense_table,
                     combine_pull_sparse_table, combine_push_sparse_table, init_model, initialize, is_initialized,
                     jagged_mean_backward, jagged_mean_forward, jagged_sum_backward, jagged_sum_forward,
                     pull_dense_table, pull_sparse_table, push_dense_table, push_sparse_table, register_dense_table,
                     register_sparse_table, stop, try_load_model_blocked, try_save_model, update_lr)
from .embedding import CombineEmbedding, Embedding
from .initializer import (ConstantInitializer, NormalInitializer, UniformInitializer, XavierNormalInitializer,
                          XavierUniformInitializer)
from .jagged_embedding import CombineJaggedEmbedding, JaggedEmbedding
from .jagged_tensor import JaggedTensor
from .lr import LR, ConstantLR, ExponentialLR, LambdaLR, StepLR, WarmupCosineLR
from .optim import SGD, Adagrad, Adam, RMSprop
from .optimizer import Optimizer
from .sparse_table import CombineSparseTable, SparseTable

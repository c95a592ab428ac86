from .deepfm import DeepFM
from .mlp import MLP
from .synthetic import ClickDataset, MultiHotDataset, mnist_like
from .wide_deep import MultiHotWideAndDeep, WideAndDeep

from .deepfm import DeepFM
from .mlp import MLP
from .synthetic import ClickDataset

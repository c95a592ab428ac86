from .functional import bce_with_logits, fm_interaction

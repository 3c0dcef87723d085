"""Triangle (protein-folding) ops, B200 implementation."""

from ._attention_pair_bias import attention_pair_bias
from ._project import attention_input_projection
from ._triattn import triangle_attention, triangle_attention_b200
from ._trimul import triangle_multiplicative_update, trimul_b200

__all__ = [
    "attention_input_projection",
    "attention_pair_bias",
    "triangle_attention",
    "triangle_attention_b200",
    "triangle_multiplicative_update",
    "trimul_b200",
]

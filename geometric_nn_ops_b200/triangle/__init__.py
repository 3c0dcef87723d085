"""Triangle (protein-folding) ops, B200 implementation."""

from ._triattn import triangle_attention, triangle_attention_b200
from ._trimul import triangle_multiplicative_update, trimul_b200

__all__ = [
    "triangle_attention",
    "triangle_attention_b200",
    "triangle_multiplicative_update",
    "trimul_b200",
]

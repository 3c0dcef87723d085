"""``geometric_nn_ops_torch.triangle``: the reference's three public ops, computed by the B200 library."""

from geometric_nn_ops_b200.triangle import (
    attention_pair_bias,
    triangle_attention,
    triangle_multiplicative_update,
)

from . import _masking  # noqa: F401

__all__ = [
    "attention_pair_bias",
    "triangle_attention",
    "triangle_multiplicative_update",
]

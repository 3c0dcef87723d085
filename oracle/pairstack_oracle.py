"""CPU oracle of the pair stack (geometric_nn_ops_b200/pairstack.py): TEST INFRASTRUCTURE, not a product path.

A composition of the two pinned oracle functions (``triangle_oracle.trimul_fwd`` and ``triangle_attention_fwd``,
which restate the reference's ``_reference/trimul.py:57-97`` and ``_reference/triangle_attention.py:11-44``)
with the stack's own glue in numpy fp64: LayerNorm without affine parameters, q/k/v/bias projections, residual
adds in the reference's ``x = x + layer(x, mask)`` convention (``testutil/trimul.py:161-164``).  The glue has no
counterpart in the reference (its attention takes pre-projected tensors), so for the glue this file is the
definition; parity of the two ops inside it is pinned through ``triangle_oracle``.
"""

import numpy as np

from oracle import triangle_oracle as orc

HEADS, HEAD_DIM = 4, 32


def _ln(t, eps=1e-5):
    mu = t.mean(axis=-1, keepdims=True)
    var = ((t - mu) ** 2).mean(axis=-1, keepdims=True)
    return (t - mu) / np.sqrt(var + eps)


def attention_update(z, pair_mask, w):
    """Starting-node attention update of ``z`` ``[B, N, N, C]``; ``w``: wq, wk, wv ``[C, H*D]``, wb ``[C, H]``."""
    B, N = z.shape[0], z.shape[1]
    zn = _ln(z)
    q, k, v = ((zn @ w[m]).reshape(B, N, N, HEADS, HEAD_DIM) for m in ("wq", "wk", "wv"))
    bias = np.transpose(zn @ w["wb"], (0, 3, 1, 2))[:, None]          # [B, 1, H, N, N]
    keep = (pair_mask != 0).reshape(B, N, 1, 1, N)
    o = orc.triangle_attention_fwd(q, k, v, bias, keep, HEAD_DIM ** -0.5)   # fully masked rows come out uniform
    return o.reshape(B, N, N, HEADS * HEAD_DIM)


def pair_block(z, pair_mask, w):
    """``w``: dict with trimul_out, trimul_in (weight dicts) and attn_start, attn_end (projection dicts), float64."""
    z = z + orc.trimul_fwd(z, "outgoing", pair_mask, **w["trimul_out"])
    z = z + orc.trimul_fwd(z, "incoming", pair_mask, **w["trimul_in"])
    z = z + attention_update(z, pair_mask, w["attn_start"])
    zt, mt = np.swapaxes(z, 1, 2), np.swapaxes(pair_mask, 1, 2)
    return z + np.swapaxes(attention_update(zt, mt, w["attn_end"]), 1, 2)


def pair_stack(z, pair_mask, blocks):
    z = np.asarray(z, dtype=np.float64)
    pair_mask = np.asarray(pair_mask, dtype=np.float64)
    for w in blocks:
        z = pair_block(z, pair_mask, w)
    return z

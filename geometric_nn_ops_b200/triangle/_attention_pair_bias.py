"""attention_pair_bias: attention over a token axis with a per-head bias projected from the pair representation.

Same signature, layouts and results as the reference's functional op
(``geometric_nn_ops_torch/triangle/_attention_pair_bias.py:11-98``), whose arithmetic is stock PyTorch
(``_reference/attention_pair_bias.py:26-89``).  Here the softmax core -- the part that is a flash-attention
problem -- runs on this package's CUDA triangle-attention kernels whenever it has their shape:

    queries and keys of one length (U == V), CUDA tensors, a kernel dtype, and the default key-mask sentinel.

Viewed as triangle attention, a batch entry is ``B``, the multiplicity ``M`` (the copies of one pair bias that
share a batch entry) is the row axis, and the per-head bias ``(B, H, U, V)`` is the pair bias shared by all
rows.  Every other case (cross attention with U != V, an explicit ``inf`` other than the dtype's sentinel, CPU
tensors, fp64) is evaluated with the same torch operations the reference uses, on whatever device the tensors
live.  The LayerNorm and projection of ``z`` before the core, and the gate and output projection after it, are
torch operations in both cases.
"""

import torch
import torch.nn.functional as F

from ._masking import mask_val
from ._triattn import _DTYPES, triangle_attention_b200


def _pair_bias(z, ln_z_weight, proj_z_weight, eps):
    """``(B, U, V, Zc)`` -> LayerNorm (weight only) -> ``Zc -> H`` projection -> ``(B, H, U, V)`` contiguous."""
    zn = F.layer_norm(z, z.shape[-1:], ln_z_weight, None, eps)
    return F.linear(zn, proj_z_weight).permute(0, 3, 1, 2).contiguous()


def _core_torch(q, k, v, pz, mask, scale, inf, B, M):
    BM, H, U, DH = q.shape
    V = k.shape[2]
    qm, km, vm = q.view(B, M, H, U, DH), k.reshape(B, M, H, V, DH), v.reshape(B, M, H, V, DH)
    logits = torch.matmul(qm, km.transpose(-1, -2)) * scale + pz[:, None]
    if mask is not None:
        keep = mask.reshape(B, -1, 1, 1, V)          # (B, 1 or M, 1, 1, V)
        sentinel = mask_val(logits.dtype) if inf is None else inf
        logits = logits + (keep.to(logits.dtype) - 1.0) * sentinel
    return torch.matmul(torch.softmax(logits, dim=-1), vm).reshape(BM, H, U, DH)


def _core_kernel(q, k, v, pz, mask, scale, B, M):
    BM, H, U, DH = q.shape
    # (BM, H, U, DH) -> rows = multiplicity: [B, M, U, H, DH] as a strided view (no copy)
    as_rows = lambda t: t.reshape(B, M, H, U, DH).transpose(2, 3)  # noqa: E731
    keep = None
    if mask is not None:
        keep = (mask != 0).reshape(B, -1, 1, 1, U).expand(B, M, 1, 1, U)
    o = triangle_attention_b200(as_rows(q), as_rows(k), as_rows(v), pz.unsqueeze(1), keep, scale)
    return o.transpose(2, 3).reshape(BM, H, U, DH)


def attention_pair_bias(s, q, k, v, z, *, proj_g_weight, proj_o_weight, proj_z_weight=None, ln_z_weight=None,
                        proj_g_bias=None, proj_o_bias=None, mask=None, scale=None, inf=None, eps=1e-5,
                        z_is_projected=False, return_z_proj=False):
    """Attention with pair bias on pre-projected q, k, v.

    Args (the reference's, same meaning):
        s: ``(BM, S, D)`` token representation the gate is projected from; the output has this shape.
        q: ``(BM, H, U, DH)``; k, v: ``(BM, H, V, DH)``.
        z: pair representation ``(B, U, V, Zc)``, or the projected bias ``(B, H, U, V)`` with ``z_is_projected``.
        proj_g_weight, proj_o_weight: ``(D, D)``; proj_z_weight: ``(H, Zc)``; ln_z_weight: ``(Zc,)``.
        mask: ``(B, V)`` or ``(BM, V)``, 1 keeps; scale: default ``DH ** -0.5``; inf: key-mask sentinel
        (default: the logits dtype's); eps: LayerNorm epsilon.

    Returns ``(out, proj_z)``: ``out`` ``(BM, S, D)``; ``proj_z`` the ``(B, H, U, V)`` bias when
    ``return_z_proj`` (reusable with ``z_is_projected``), else ``None``.
    """
    BM, H, U, DH = q.shape
    V = k.shape[2]
    B = z.shape[0]
    if BM % B != 0:
        raise ValueError(f"q batch {BM} is not a multiple of z batch {B}")
    M = BM // B
    if mask is not None and mask.shape[0] not in (B, BM):
        raise ValueError(f"mask batch {mask.shape[0]} must be B={B} or BM={BM}")
    if scale is None:
        scale = DH ** -0.5
    pz = z if z_is_projected else _pair_bias(z, ln_z_weight, proj_z_weight, eps)

    on_kernel = (q.is_cuda and U == V and q.dtype in _DTYPES and k.dtype == q.dtype and v.dtype == q.dtype
                 and DH <= 128 and (inf is None or float(inf) == mask_val(q.dtype)))
    if on_kernel:
        o = _core_kernel(q, k, v, pz.to(q.dtype), mask, float(scale), B, M)
    else:
        o = _core_torch(q, k, v, pz, mask, scale, inf, B, M)
    o = o.transpose(1, 2).reshape(BM, U, H * DH).to(s.dtype)
    gate = torch.sigmoid(F.linear(s, proj_g_weight, proj_g_bias))
    out = F.linear(o * gate, proj_o_weight, proj_o_bias)
    return out, (pz if return_z_proj else None)

"""Pairformer-style pair stack built from the two triangle ops: inference, one GPU or rows sharded over GPUs.

One block updates the pair representation ``z`` ``[B, N, N, C]`` four times, each with a residual add (the
reference's stack convention, ``testutil/trimul.py:161-164``)::

    z += triangle_multiplicative_update(z, "outgoing")
    z += triangle_multiplicative_update(z, "incoming")
    z += triangle_attention around the starting node   (row i attends over the keys j of its own row)
    z += triangle_attention around the ending node     (the same op on z transposed, result transposed back)

The reference ships the two ops, not this glue: its attention takes pre-projected tensors
(``geometric_nn_ops_torch/triangle/_triattn.py:36-44``).  The glue here is the plain one: ``zn = LayerNorm(z)``
without affine parameters, ``q, k, v = zn W_{q,k,v}`` (``[C, H*D]``, split into H heads), pair bias
``= zn W_b`` (``[C, H]``) laid out ``[B, 1, H, N, N]``, key mask of row i = row i of the pair mask, and the
attention output ``[B, N, N, H*D]`` is what is added back (H*D = C).

Sharded over P GPUs, every rank holds rows ``[r N/P, (r+1) N/P)`` of ``z``: the multiplicative updates use the
row <-> channel exchanges of :mod:`geometric_nn_ops_b200.sharded`, the starting-node attention is local once the
pair bias has been all-gathered, and the ending-node attention runs between two all-to-all transposes.
"""

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import sharded
from .triangle import attention_input_projection, triangle_attention, triangle_multiplicative_update

HEADS, HEAD_DIM = 4, 32
TRIMUL_NAMES = ("norm_in_weight", "norm_in_bias", "p_in_weight", "g_in_weight", "norm_out_weight", "norm_out_bias",
                "p_out_weight", "g_out_weight")


@dataclass
class BlockWeights:
    trimul_out: dict
    trimul_in: dict
    attn_start: dict      # {"wq", "wk", "wv": [C, H*D], "wb": [C, H]}
    attn_end: dict

    def to(self, device=None, dtype=None):
        mv = lambda d: {k: v.to(device=device, dtype=dtype) for k, v in d.items() if not k.startswith("_")}  # noqa: E731
        return BlockWeights(mv(self.trimul_out), mv(self.trimul_in), mv(self.attn_start), mv(self.attn_end))


def make_block_weights(seed, c=128, dtype=torch.bfloat16, device="cpu"):
    """Random weights of one block drawn on the CPU from ``seed`` (BASELINE distributions: LayerNorm weights
    1 + N(0, 0.02), LayerNorm biases N(0, 0.02), projections N(0, 1/sqrt(fan_in)), no projection biases)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc  # noqa: E731

    def trimul():
        return {"norm_in_weight": 1 + rn(c, sc=0.02), "norm_in_bias": rn(c, sc=0.02),
                "p_in_weight": rn(2 * c, c, sc=c ** -0.5), "g_in_weight": rn(2 * c, c, sc=c ** -0.5),
                "norm_out_weight": 1 + rn(c, sc=0.02), "norm_out_bias": rn(c, sc=0.02),
                "p_out_weight": rn(c, c, sc=c ** -0.5), "g_out_weight": rn(c, c, sc=c ** -0.5)}

    def attn():
        return {"wq": rn(c, HEADS * HEAD_DIM, sc=c ** -0.5), "wk": rn(c, HEADS * HEAD_DIM, sc=c ** -0.5),
                "wv": rn(c, HEADS * HEAD_DIM, sc=c ** -0.5), "wb": rn(c, HEADS, sc=c ** -0.5)}

    return BlockWeights(trimul(), trimul(), attn(), attn()).to(device, dtype)


def make_inputs(n, c=128, masked_tail=64, dtype=torch.bfloat16, seed=100):
    """``z ~ N(0, 1)`` ``[1, n, n, c]`` and the pair mask: outer product of a residue mask whose last
    ``masked_tail`` residues are 0."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(1, n, n, c, generator=g).to(dtype)
    res = torch.ones(n)
    if masked_tail:
        res[-masked_tail:] = 0
    return z, (res[:, None] * res[None, :]).reshape(1, n, n).to(dtype)


def _fused_weights(w):
    """The projection weights in the layout the fused kernel takes, built once per block and kept with it."""
    if "_w_qkv" not in w:
        w["_w_qkv"] = torch.cat([w["wq"].t(), w["wk"].t(), w["wv"].t()]).contiguous()    # [3*H*D, C]
        w["_w_bias"] = w["wb"].t().contiguous()                                            # [H, C]
    return w["_w_qkv"], w["_w_bias"]


def project_attention_inputs(z, w):
    """``z`` ``[B, R, N, C]`` (R rows) -> q, k, v ``[B, R, N, H, D]`` and this rows' bias ``[B, H, R, N]``.

    On the GPU with C = 128 this is the library's fused projection (one LayerNorm + bias kernel, one GEMM); the
    torch composition below it defines what that computes and serves every other case."""
    if z.is_cuda and z.shape[-1] == 128 and z.dtype in (torch.bfloat16, torch.float16) and not torch.is_grad_enabled():
        w_qkv, w_bias = _fused_weights(w)
        q, k, v, bias = attention_input_projection(z, w_qkv, w_bias, HEADS)
        return q, k, v, bias.contiguous()
    zn = F.layer_norm(z, z.shape[-1:])
    B, R, N, _ = z.shape
    q, k, v = ((zn @ w[m]).view(B, R, N, HEADS, HEAD_DIM) for m in ("wq", "wk", "wv"))
    bias = (zn @ w["wb"]).permute(0, 3, 1, 2).contiguous()
    return q, k, v, bias


def _ending_node_update(z, pair_mask, w):
    """Ending-node triangle attention of a whole ``z`` ``[B, N, N, C]`` on one GPU, without transposing ``z``.

    The projections act on single pair positions, so q, k, v of the transposed pair representation are transposed
    *views* of the ones projected from ``z`` as it lies; the kernels take the strides.  Only the ``[B, H, N, N]``
    bias and the mask (both small) are copied transposed, and the result comes back through a transposed view.
    Returns the update in ``z``'s orientation, ``[B, N, N, C]``."""
    q, k, v, bias = project_attention_inputs(z, w)                    # [B, i, j, H, D], [B, H, i, j]
    B, N = z.shape[0], z.shape[1]
    keep = (pair_mask.transpose(1, 2) != 0).reshape(B, N, 1, 1, N)     # row j of the transposed problem masks keys i
    o = triangle_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                           bias.transpose(2, 3).contiguous().unsqueeze(1), keep)   # [B, j, i, H, D]
    return o.transpose(1, 2).reshape(B, N, N, HEADS * HEAD_DIM)


def _attention_update(z, pair_mask, w, group):
    """Starting-node triangle attention on the rows held here; returns ``[B, R, N, C]``."""
    q, k, v, bias = project_attention_inputs(z, w)
    B, R, N, _ = z.shape
    if group is not None and sharded._world(group)[0] > 1:
        parts = [torch.empty_like(bias) for _ in range(sharded._world(group)[0])]
        torch.distributed.all_gather(parts, bias, group=group)       # every rank needs the whole [H, N, N] bias
        bias = torch.cat(parts, dim=2)
    keep = (pair_mask != 0).view(B, R, 1, 1, N)
    o = triangle_attention(q, k, v, bias.unsqueeze(1), keep)
    return o.reshape(B, R, N, HEADS * HEAD_DIM)


def pair_block(z, pair_mask, w: BlockWeights, group=None):
    """One block on ``z`` ``[B, R, N, C]`` (R = N on one GPU, N/P rows when sharded), ``pair_mask`` ``[B, R, N]``."""
    multi = group is not None and sharded._world(group)[0] > 1
    for direction, tw in (("outgoing", w.trimul_out), ("incoming", w.trimul_in)):
        if multi:
            z = z + sharded.sharded_triangle_multiplicative_update(z, direction, pair_mask, group=group, **tw)
        else:
            z = z + triangle_multiplicative_update(z, direction, pair_mask, **tw)
    z = z + _attention_update(z, pair_mask, w.attn_start, group)
    if multi:
        zt = sharded.all_to_all_transpose(z.contiguous(), group)
        mt = sharded.all_to_all_transpose(pair_mask.contiguous(), group)
        z = z + sharded.all_to_all_transpose(_attention_update(zt, mt, w.attn_end, group).contiguous(), group)
    else:
        z = z + _ending_node_update(z, pair_mask, w.attn_end)
    return z


@torch.no_grad()
def pair_stack(z, pair_mask, blocks, group=None):
    """Run ``blocks`` (a list of :class:`BlockWeights`) in order; inference only."""
    for w in blocks:
        z = pair_block(z, pair_mask, w, group)
    return z


def stack_flops(n, n_blocks, c=128):
    """Algorithmic forward FLOPs: per block two multiplicative updates, two attentions and their projections."""
    m = float(n) * n
    trimul = 2.0 * m * c * 4 * c + 2.0 * m * c * c + 2.0 * m * c * c + 2.0 * float(n) ** 3 * c
    attn = 4.0 * n * HEADS * m * HEAD_DIM
    proj = 2.0 * m * c * (3 * HEADS * HEAD_DIM + HEADS)
    return n_blocks * 2.0 * (trimul + attn + proj)

"""Fused input projection of triangle attention in a pair stack: LayerNorm(z) -> q, k, v and the pair bias.

Two launches of the CUDA library (``tri_attn_project``): a LayerNorm kernel that also projects the per-head pair
bias while the normalised row is in registers, and one tcgen05 GEMM that writes q, k and v side by side in a single
``[pixels, 3*H*D]`` buffer.  The returned q, k, v are strided views of that buffer in the ``[B, rows, N, H, D]``
layout :func:`triangle_attention` takes (its kernels read strides, so nothing is copied), and the bias comes back
head-major, ready to be used as ``[B, 1, H, N, N]``.

The reference has no such op: its attention takes pre-projected tensors
(``geometric_nn_ops_torch/triangle/_triattn.py:36-44``) and callers project with eager torch.  Forward only.
"""

import ctypes

import torch

from .. import _lib, _precision
from ._triattn import _DTYPES


def attention_input_projection(z, w_qkv, w_bias, heads, ln_weight=None, ln_bias=None, eps=1e-5):
    """``z``: ``[B, R, N, 128]``; ``w_qkv``: ``[3*H*D, 128]`` (rows: q, then k, then v, ``F.linear`` layout);
    ``w_bias``: ``[H, 128]``.  Returns ``q, k, v`` ``[B, R, N, H, D]`` and ``bias`` ``[B, H, R, N]``
    (``bias[b, h, r, n] = LayerNorm(z)[b, r, n] . w_bias[h]``).  Inference only: no gradient is recorded."""
    lib = _lib.load()
    if not z.is_cuda:
        raise RuntimeError("attention_input_projection needs CUDA tensors: there is no CPU implementation")
    if z.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {z.dtype}")
    if any(t is not None and t.requires_grad for t in (z, w_qkv, w_bias, ln_weight, ln_bias)) and torch.is_grad_enabled():
        raise RuntimeError("attention_input_projection is forward only: call it under torch.no_grad()")
    B, R, N, C = z.shape
    n_out = w_qkv.shape[0]
    if n_out % (3 * heads) != 0 or w_qkv.shape[1] != C or tuple(w_bias.shape) != (heads, C):
        raise ValueError(f"w_qkv must be [3*H*D, {C}] and w_bias [{heads}, {C}], got {tuple(w_qkv.shape)} and {tuple(w_bias.shape)}")
    D = n_out // (3 * heads)
    d = _lib.TriAttnProjDesc()
    d.M, d.C, d.H, d.D = B * R * N, C, heads, D
    d.dtype = _DTYPES[z.dtype]
    precision = _precision.matmul_precision(fp32_operands=z.dtype == torch.float32)
    d.precision = _lib.PREC_TF32 if precision == _precision.TF32 else _lib.PREC_IEEE
    d.eps = eps
    ws_bytes = lib.tri_attn_project_ws_bytes(ctypes.byref(d))
    if ws_bytes == 0:
        raise RuntimeError("attention_input_projection: " + lib.tri_last_error().decode(errors="replace"))
    cv = lambda t: None if t is None else t.detach().to(z.dtype).contiguous()  # noqa: E731
    zc, wq, wb, lw, lb = cv(z), cv(w_qkv), cv(w_bias), cv(ln_weight), cv(ln_bias)
    qkv = torch.empty(B, R, N, 3, heads, D, dtype=z.dtype, device=z.device)
    bias = torch.empty(heads, B, R, N, dtype=z.dtype, device=z.device)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=z.device)
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream(z.device).cuda_stream)
    with torch.cuda.device(z.device):
        _lib.check(lib.tri_attn_project(ctypes.byref(d), p(zc), p(lw), p(lb), p(wq), p(wb), p(qkv), p(bias), p(ws), ws_bytes,
                                        stream), "tri_attn_project")
        _lib.check_device_status(ws, stream)
    return qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2], bias.permute(1, 0, 2, 3)

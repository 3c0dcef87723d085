"""triangle_attention on B200: public wrapper, kernel-level entry and autograd glue.

The public function keeps the signature and argument handling of the reference's
``geometric_nn_ops_torch/triangle/_triattn.py:23-106``; the kernel-level entry
``triangle_attention_b200`` stands where the reference has
``triangle_attention_triton`` (``_kernels/triangle_attention.py:1447-1484``).
All arithmetic happens in libtri_b200.so; q/k/v/o are passed with their strides,
so both the native ``[B, N_seq, N_res, H, D]`` layout and the cuequivariance
``(B, N, H, S, D)`` layout (a transposed view) run without a copy.
"""

import ctypes

import torch

from .. import _lib, _precision

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _inner_contiguous(t):
    """A tensor whose last axis has stride 1 (copy only if it does not)."""
    return t if t.stride(-1) == 1 or t.shape[-1] == 1 else t.contiguous()


def _dense(t):
    """True when ``t``'s strides describe a permutation of a contiguous block."""
    if t.stride(-1) != 1:
        return False
    expect = 1
    for size, stride in sorted(zip(t.shape, t.stride()), key=lambda p: p[1]):
        if size == 1:
            continue
        if stride != expect:
            return False
        expect *= size
    return True


def _like(t):
    return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device) if _dense(t) else torch.empty_like(
        t, memory_format=torch.contiguous_format)


def _st4(t):
    s = t.stride()
    return (ctypes.c_int64 * 4)(s[0], s[1], s[2], s[3])


def _desc(q, k, v, o, bias, mask, scale, precision):
    B, S, N, H, D = q.shape
    d = _lib.TriAttnDesc()
    d.B, d.n_seq, d.n_res, d.H, d.D = B, S, N, H, D
    d.dtype = _DTYPES[q.dtype]
    d.precision = _lib.PREC_TF32 if precision == _precision.TF32 else _lib.PREC_IEEE
    d.scale = scale
    d.q_st, d.k_st, d.v_st, d.o_st = _st4(q), _st4(k), _st4(v), _st4(o)
    if bias is not None:
        bs = bias.stride()
        d.bias_st = (ctypes.c_int64 * 3)(bs[0], bs[2], bs[3])
    if mask is not None:
        ms = mask.stride()
        d.mask_st = (ctypes.c_int64 * 2)(ms[0], ms[1])
    return d


class _TriangleAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, mask, scale):
        lib = _lib.load()
        if not q.is_cuda:
            raise RuntimeError("triangle_attention needs CUDA tensors: there is no CPU implementation")
        if q.dtype not in _DTYPES:
            raise TypeError(f"unsupported dtype {q.dtype}")
        q, k, v = _inner_contiguous(q), _inner_contiguous(k), _inner_contiguous(v)
        B, S, N, H, D = q.shape
        if bias is not None:
            bias = _inner_contiguous(bias)
        mask_u8 = None
        if mask is not None:
            mask_u8 = mask.reshape(B, S, N).contiguous().view(torch.uint8)
        precision = _precision.matmul_precision(fp32_operands=q.dtype == torch.float32)
        o = _like(q)
        lse = torch.empty(2, B, S, H, N, dtype=torch.float32, device=q.device)
        d = _desc(q, k, v, o, bias, mask_u8, scale, precision)
        ws_bytes = lib.tri_attn_ws_bytes(ctypes.byref(d), 0)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=q.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        with torch.cuda.device(q.device):
            _lib.check(lib.tri_attn_fwd(ctypes.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask_u8),
                                        _ptr(o), _ptr(lse), _ptr(ws), ws_bytes, stream), "tri_attn_fwd")
            _lib.check_device_status(ws, stream)
        ctx.save_for_backward(q, k, v, bias, mask_u8, o, lse)
        ctx.scale, ctx.precision = scale, precision
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _d_stats=None):
        lib = _lib.load()
        q, k, v, bias, mask_u8, o, lse = ctx.saved_tensors
        B, S, N, H, D = q.shape
        d_o = _inner_contiguous(d_o)
        dq, dk, dv = _like(q), _like(k), _like(v)
        want_dbias = bias is not None and ctx.needs_input_grad[3]
        dbias = torch.empty(B, H, N, N, dtype=torch.float32, device=q.device) if want_dbias else None
        d = _desc(q, k, v, o, bias, mask_u8, ctx.scale, ctx.precision)
        d.do_st, d.dq_st, d.dk_st, d.dv_st = _st4(d_o), _st4(dq), _st4(dk), _st4(dv)
        ws_bytes = lib.tri_attn_ws_bytes(ctypes.byref(d), 1)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=q.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        with torch.cuda.device(q.device):
            _lib.check(lib.tri_attn_bwd(ctypes.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mask_u8),
                                        _ptr(o), _ptr(lse), _ptr(d_o), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbias),
                                        _ptr(ws), ws_bytes, stream), "tri_attn_bwd")
            _lib.check_device_status(ws, stream)
        grad_bias = None
        if want_dbias:
            grad_bias = dbias.to(bias.dtype).reshape(B, 1, H, N, N)
        return dq, dk, dv, grad_bias, None, None


def _aux(stats):
    """Softmax statistics ``[2, B, N_seq, H, N_res]`` (row maximum, log row sum) -> ``(lse, max)``, each
    ``[B, N_seq, H, N_res, 1]`` fp32, the cuequivariance ``(B, N, H, Q, 1)`` layout.

    ``lse`` is exact.  ``max`` is the reference point the kernel used for the exponentials: the exact row maximum on
    the CUDA-core path; on the tensor-core path, which rescales its accumulator only when the maximum grows by more
    than ``8 ln 2``, a value between ``max - 8 ln 2`` and ``max``."""
    m, log_l = stats[0], stats[1]
    return (m + log_l).unsqueeze(-1), m.unsqueeze(-1)


def triangle_attention_b200(q, k, v, bias=None, mask=None, scale=None, dynamic=False, use_exp2=False,
                            return_aux=False):
    """Kernel-level entry on canonical 5-D shapes.

    ``q, k, v``: ``[B, N_seq, N_res, H, D]``; ``bias``: ``[B, 1, H, N_res, N_res]`` (batch may be
    a broadcast view); ``mask``: bool ``[B, N_seq, 1, 1, N_res]``, ``True`` keeps.
    ``dynamic`` and ``use_exp2`` are accepted for signature compatibility; the CUDA kernels
    take shapes at run time, so both settings give the same result.
    ``return_aux=True`` returns ``(out, lse, max)``: the log-sum-exp and the maximum of each query's
    logits, fp32 ``[B, N_seq, H, N_res, 1]``, not differentiable.  (The reference's kernels do not expose
    them and its cuequivariance shim raises for ``return_aux``,
    ``cuequivariance_ops_torch/triangle_attention.py:34-38``; these kernels write them anyway.)
    """
    del dynamic, use_exp2
    if scale is None:
        scale = q.shape[-1] ** -0.5
    o, stats = _TriangleAttention.apply(q, k, v, bias, mask, float(scale))
    if return_aux:
        return (o, *_aux(stats))
    return o


def triangle_attention(q, k, v, bias=None, mask=None, scale=None, dynamic=False, use_exp2=False, return_aux=False):
    """Triangle attention with the reference's (cuequivariance-compatible) signature.

    Args:
        q, k, v: ``[..., N_seq, N_res, H, D]``; rank 4, 5 or 6 (leading dims fold into one batch).
        bias: broadcastable to ``[B, 1, H, N_res, N_res]``, or ``None``.
        mask: bool, ``True`` keeps; broadcastable to ``[B, N_seq, 1, 1, N_res]``, or ``None``.
        scale: softmax scale, default ``D ** -0.5``.

    Returns a tensor of q's shape and dtype; with ``return_aux=True`` also the log-sum-exp and the
    maximum of every query's logits (fp32, ``[B, N_seq, H, N_res, 1]``).  fp32 matmuls follow
    ``torch.backends.cuda.matmul.fp32_precision``.
    """
    if mask is not None and mask.dtype != torch.bool:
        raise ValueError(f"mask must be bool (keep=True/mask=False), got {mask.dtype}")

    orig_shape, orig_dtype = q.shape, q.dtype
    if q.dim() < 5:
        pad = (1,) * (5 - q.dim())
        q, k, v = (t.reshape(pad + tuple(t.shape)) for t in (q, k, v))
    elif q.dim() > 5:
        q, k, v = (t.reshape(-1, *t.shape[-4:]) for t in (q, k, v))
    B, S, N, H, D = q.shape

    if bias is not None:
        if bias.dim() == 4:
            bias = bias.unsqueeze(-4)
        elif bias.dim() > 5:
            bias = bias.reshape(-1, *bias.shape[-4:])
        bias = bias.broadcast_to(B, 1, H, N, N)
    if mask is not None:
        if mask.dim() > 5:
            mask = mask.reshape(-1, *mask.shape[-4:])
        mask = mask.broadcast_to(B, S, 1, 1, N)

    compute = orig_dtype if orig_dtype in _DTYPES else torch.float32
    res = triangle_attention_b200(
        q.to(compute), k.to(compute), v.to(compute),
        None if bias is None else bias.to(compute), mask, scale, dynamic, use_exp2, return_aux,
    )
    if return_aux:
        o, lse, amax = res
        return o.to(orig_dtype).reshape(orig_shape), lse, amax
    return res.to(orig_dtype).reshape(orig_shape)

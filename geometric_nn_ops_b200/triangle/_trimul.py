"""triangle_multiplicative_update on B200: public wrapper, kernel-level entry, autograd glue.

Keeps the signature of the reference's public op
(``geometric_nn_ops_torch/triangle/_trimul.py:39-88``) and of its kernel-level
functions ``impl(x, direction, mask, *, eps, **weights)``
(``_kernels/trimul.py:404-422``, ``_reference/trimul.py:57-75``).  Unlike the
reference, whose kernels are forward-only and which sends every grad-requiring call
to eager torch, forward AND backward run in libtri_b200.so.  CPU tensors are
rejected: there is no CPU implementation in this package.
"""

import ctypes

import torch

from .. import _lib, _precision

DIRECTIONS = ("outgoing", "incoming")
_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def is_outgoing(direction: str) -> bool:
    if direction not in DIRECTIONS:
        raise ValueError(f"direction must be one of {DIRECTIONS}, got {direction!r}")
    return direction == "outgoing"


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _aligned(t):
    """Contiguous and 16-byte aligned (TMA and the vector loads need it); copies only if it must."""
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


class _TriMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, outgoing, eps, *weights):
        lib = _lib.load()
        if not x.is_cuda:
            raise RuntimeError("triangle_multiplicative_update needs CUDA tensors: there is no CPU implementation")
        named = dict(zip(_lib.WEIGHT_NAMES, weights))
        for req in ("p_in_weight", "g_in_weight", "p_out_weight", "g_out_weight"):
            if named[req] is None:
                raise ValueError(f"{req} is required")
        N, C = x.shape[-2], x.shape[-1]
        if x.shape[-3] != N:
            raise ValueError(f"x must be [*, N, N, C], got {tuple(x.shape)}")
        xc = _aligned(x.reshape(-1, N, N, C))
        B = xc.shape[0]
        mc = None
        if mask is not None:
            mc = _aligned(mask.to(x.dtype).broadcast_to(x.shape[:-1]).reshape(B, N, N))
        wc = {n: (None if t is None else _aligned(t.detach().to(x.dtype))) for n, t in named.items()}
        Ch = wc["p_in_weight"].shape[0] // 2
        expect = {"p_in_weight": (2 * Ch, C), "g_in_weight": (2 * Ch, C), "p_out_weight": (C, Ch),
                  "g_out_weight": (C, C), "norm_in_weight": (C,), "norm_in_bias": (C,), "norm_out_weight": (Ch,),
                  "norm_out_bias": (Ch,), "p_in_bias": (2 * Ch,), "g_in_bias": (2 * Ch,), "p_out_bias": (C,),
                  "g_out_bias": (C,)}
        for n, t in wc.items():
            if t is not None and tuple(t.shape) != expect[n]:
                raise ValueError(f"{n} has shape {tuple(t.shape)}, expected {expect[n]}")

        d = _lib.TriMulDesc()
        d.B, d.N, d.C, d.Ch = B, N, C, Ch
        d.dtype = _DTYPES[x.dtype]
        precision = _precision.matmul_precision(fp32_operands=x.dtype == torch.float32)
        d.precision = _lib.PREC_TF32 if precision == _precision.TF32 else _lib.PREC_IEEE
        d.direction = _lib.OUTGOING if outgoing else _lib.INCOMING
        d.eps = eps
        w = _lib.TriMulWeights()
        for n, t in wc.items():
            setattr(w, _lib.abi_field(n), None if t is None else t.data_ptr())

        need_grad = any(ctx.needs_input_grad)
        saved = None
        if need_grad:
            saved = torch.empty(lib.tri_mul_saved_bytes(ctypes.byref(d)), dtype=torch.uint8, device=x.device)
        ws_bytes = lib.tri_mul_ws_bytes(ctypes.byref(d), 0)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
        out = torch.empty_like(xc)
        stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        with torch.cuda.device(x.device):
            _lib.check(lib.tri_mul_fwd(ctypes.byref(d), _ptr(xc), _ptr(mc), ctypes.byref(w), _ptr(out), _ptr(saved),
                                       _ptr(ws), ws_bytes, stream), "tri_mul_fwd")
            _lib.check_device_status(ws, stream)
        if need_grad:
            ctx.save_for_backward(xc, mc, saved, *[t for t in wc.values() if t is not None])
            ctx.present = [t is not None for t in wc.values()]
            ctx.desc = d
            ctx.x_shape = x.shape
            ctx.weight_dtypes = [None if t is None else t.dtype for t in weights]
        return out.reshape(x.shape)

    @staticmethod
    def backward(ctx, d_out):
        lib = _lib.load()
        xc, mc, saved, *present_w = ctx.saved_tensors
        it = iter(present_w)
        wc = {n: (next(it) if has else None) for n, has in zip(_lib.WEIGHT_NAMES, ctx.present)}
        d = ctx.desc
        w = _lib.TriMulWeights()
        g = _lib.TriMulWeightGrads()
        grads = {}
        for i, (n, t) in enumerate(wc.items()):
            setattr(w, _lib.abi_field(n), None if t is None else t.data_ptr())
            if t is not None and ctx.needs_input_grad[4 + i]:
                grads[n] = torch.empty(t.shape, dtype=torch.float32, device=xc.device)
                setattr(g, _lib.abi_field(n), grads[n].data_ptr())
        dc = _aligned(d_out.reshape(xc.shape).to(xc.dtype))
        dx = torch.empty_like(xc)
        ws_bytes = lib.tri_mul_ws_bytes(ctypes.byref(d), 1)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=xc.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(xc.device).cuda_stream)
        with torch.cuda.device(xc.device):
            _lib.check(lib.tri_mul_bwd(ctypes.byref(d), _ptr(xc), _ptr(mc), ctypes.byref(w), _ptr(saved), _ptr(dc),
                                       _ptr(dx), ctypes.byref(g), _ptr(ws), ws_bytes, stream), "tri_mul_bwd")
            _lib.check_device_status(ws, stream)
        out = [dx.reshape(ctx.x_shape) if ctx.needs_input_grad[0] else None, None, None, None]
        for n, dt in zip(_lib.WEIGHT_NAMES, ctx.weight_dtypes):
            out.append(grads[n].to(dt) if n in grads else None)
        return tuple(out)


def trimul_b200(x, direction="outgoing", mask=None, *, eps=1e-5, norm_in_weight=None, norm_in_bias=None,
                p_in_weight=None, p_in_bias=None, g_in_weight=None, g_in_bias=None, norm_out_weight=None,
                norm_out_bias=None, p_out_weight=None, p_out_bias=None, g_out_weight=None, g_out_bias=None):
    """Kernel-level triangle multiplicative update, forward and backward on the GPU.

    ``x`` is ``[*, N, N, C_z]``, ``mask`` broadcastable to ``[*, N, N]`` (1 = keep);
    ``p_in_weight`` / ``g_in_weight`` are the concatenated ``[a; b]`` projections.
    """
    outgoing = is_outgoing(direction)
    return _TriMul.apply(x, mask, outgoing, float(eps), norm_in_weight, norm_in_bias, p_in_weight, p_in_bias,
                         g_in_weight, g_in_bias, norm_out_weight, norm_out_bias, p_out_weight, p_out_bias,
                         g_out_weight, g_out_bias)


def triangle_multiplicative_update(x, direction="outgoing", mask=None, norm_in_weight=None, norm_in_bias=None,
                                   p_in_weight=None, p_in_bias=None, g_in_weight=None, g_in_bias=None,
                                   norm_out_weight=None, norm_out_bias=None, p_out_weight=None, p_out_bias=None,
                                   g_out_weight=None, g_out_bias=None, eps=1e-5):
    """Triangle multiplicative update over a pair representation (reference signature).

    Returns ``[*, N, N, C_z]``.  fp32 matmuls follow
    ``torch.backends.cuda.matmul.fp32_precision``.  Dtypes without a kernel (fp64) are
    computed in fp32 and cast back.
    """
    is_outgoing(direction)
    kw = dict(norm_in_weight=norm_in_weight, norm_in_bias=norm_in_bias, p_in_weight=p_in_weight,
              p_in_bias=p_in_bias, g_in_weight=g_in_weight, g_in_bias=g_in_bias, norm_out_weight=norm_out_weight,
              norm_out_bias=norm_out_bias, p_out_weight=p_out_weight, p_out_bias=p_out_bias,
              g_out_weight=g_out_weight, g_out_bias=g_out_bias)
    if x.dtype in _DTYPES:
        return trimul_b200(x, direction, mask, eps=eps, **kw)
    out = trimul_b200(x.float(), direction, mask, eps=eps,
                      **{n: (None if t is None else t.float()) for n, t in kw.items()})
    return out.to(x.dtype)

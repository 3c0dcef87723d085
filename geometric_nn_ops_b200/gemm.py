"""Batched tensor-core GEMM ``C[b] = A[b] @ B[b]^T`` (the trimul "combine" step) as a torch-callable.

Stands where the reference calls ``torch.einsum`` on permuted views
(``geometric_nn_ops_torch/triangle/_reference/trimul.py:44-54``).
"""

import ctypes

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def bgemm(a, b, *, a_mn_major=False, b_mn_major=False, out_dtype=None, check=False):
    """``a``: ``[batch, M, K]`` (K-major) or ``[batch, K, M]`` (MN-major); ``b`` likewise with N.

    Returns ``[batch, M, N]`` in ``out_dtype`` (the input dtype, or ``torch.float32``).  fp32 inputs are
    multiplied in tf32.  ``check=True`` reads the kernel's status word back (synchronises).
    """
    lib = _lib.load()
    if not a.is_cuda:
        raise RuntimeError("bgemm needs CUDA tensors: there is no CPU implementation")
    a, b = a.contiguous(), b.contiguous()
    batch = a.shape[0]
    M, K = (a.shape[2], a.shape[1]) if a_mn_major else (a.shape[1], a.shape[2])
    N = b.shape[2] if b_mn_major else b.shape[1]
    out_dtype = out_dtype or a.dtype
    c = torch.empty(batch, M, N, dtype=out_dtype, device=a.device)
    d = _lib.TriGemmDesc()
    d.M, d.N, d.K, d.batch, d.dtype = M, N, K, batch, _DTYPES[a.dtype]
    d.a_mn_major, d.b_mn_major = int(a_mn_major), int(b_mn_major)
    d.out_f32 = int(out_dtype == torch.float32)
    d.lda, d.ldb, d.ldc = a.stride(1), b.stride(1), N
    d.batch_a, d.batch_b, d.batch_c = a.stride(0), b.stride(0), M * N
    ws = torch.empty(256, dtype=torch.uint8, device=a.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    with torch.cuda.device(a.device):
        _lib.check(lib.tri_bgemm(ctypes.byref(d), p(a), p(b), p(c), p(ws), 256, stream), "tri_bgemm")
        if check:
            _lib.check(lib.tri_ws_status(p(ws), stream), "tri_bgemm (device status)")
    return c

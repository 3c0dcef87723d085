"""CPU-only checks: the C-ABI library loads and exports what the header declares; host-side argument
handling raises the reference's errors; nothing computes without a GPU."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "tri_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tri_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    names = _header_functions()
    assert {"tri_attn_fwd", "tri_attn_bwd", "tri_mul_fwd", "tri_mul_bwd"} <= set(names)
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.EXPORTS, f"{name} has no ctypes prototype"
    assert lib.tri_abi_version() >= 1


def test_struct_layouts_match_header():
    from geometric_nn_ops_b200 import _lib
    assert ctypes.sizeof(_lib.TriAttnDesc) == 8 * 4 + 8 * 4 * 8 + 3 * 8 + 2 * 8
    assert ctypes.sizeof(_lib.TriMulDesc) == 32
    assert ctypes.sizeof(_lib.TriMulWeights) == 12 * 8 == ctypes.sizeof(_lib.TriMulWeightGrads)


def test_argument_checks_need_no_gpu():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    d = _lib.TriMulDesc()
    assert lib.tri_mul_ws_bytes(ctypes.byref(d), 0) == 0
    assert b"positive" in lib.tri_last_error()
    d.B, d.N, d.C, d.Ch, d.dtype = 1, 8, 16, 8, _lib.F32
    assert lib.tri_mul_ws_bytes(ctypes.byref(d), 1) > lib.tri_mul_ws_bytes(ctypes.byref(d), 0) > 0
    assert lib.tri_mul_saved_bytes(ctypes.byref(d)) > 0
    d.direction = 7
    assert lib.tri_mul_fwd(ctypes.byref(d), None, None, None, None, None, None, 0, None) == -1
    a = _lib.TriAttnDesc()
    a.B, a.n_seq, a.n_res, a.H, a.D = 1, 4, 4, 1, 256
    assert lib.tri_attn_fwd(ctypes.byref(a), *([None] * 8), 0, None) == -3


def test_host_errors():
    from geometric_nn_ops_b200.triangle import triangle_attention, triangle_multiplicative_update
    q = torch.zeros(1, 2, 4, 1, 8)
    with pytest.raises(ValueError, match="mask must be bool"):
        triangle_attention(q, q, q, None, torch.ones(1, 2, 1, 1, 4))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        triangle_attention(q, q, q)
    x = torch.zeros(1, 4, 4, 8)
    w = dict(p_in_weight=torch.zeros(8, 8), g_in_weight=torch.zeros(8, 8), p_out_weight=torch.zeros(8, 4),
             g_out_weight=torch.zeros(8, 8))
    with pytest.raises(ValueError, match="direction must be one of"):
        triangle_multiplicative_update(x, "sideways", None, **w)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        triangle_multiplicative_update(x, "outgoing", None, **w)


def test_precision_follows_torch_global():
    from geometric_nn_ops_b200 import _precision
    matmul = torch.backends.cuda.matmul
    prev = matmul.fp32_precision
    try:
        matmul.fp32_precision = "tf32"
        assert _precision.torch_precision() == "tf32"
        assert _precision.matmul_precision(fp32_operands=False) == "ieee"
        matmul.fp32_precision = "ieee"
        assert _precision.torch_precision() == "ieee"
    finally:
        matmul.fp32_precision = prev
    assert _precision.torch_precision() in ("ieee", "tf32")

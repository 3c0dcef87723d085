"""tri_attn_bwd_noalloc: the attention backward for callers that may not allocate device memory.

Collected last on purpose (file name), so a run that stops at the first failure has already seen every
other test.  The entry point keeps its scratch in an array built into the library, so the test calls it
straight through the C ABI with nothing but inputs and outputs, twice in a row, and compares each result
with what the regular workspace-taking entry point returns for the same inputs and with the fp64 oracle.
"""

import ctypes

import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu


def _run(dtype, shape, seed):
    from geometric_nn_ops_b200 import _lib
    from geometric_nn_ops_b200.triangle import _triattn

    lib = _lib.load()
    t, mask, d_o = util.attn_inputs(*shape, dtype, seed=seed)
    q, k, v, bias = t["q"], t["k"], t["v"], t["bias"]
    B, S, N, H, D = q.shape
    mask_u8 = mask.reshape(B, S, N).contiguous().view(torch.uint8)
    o = torch.empty_like(q)
    lse = torch.empty(2, B, S, H, N, dtype=torch.float32, device="cuda")
    d = _triattn._desc(q, k, v, o, bias, mask_u8, D ** -0.5, "ieee")
    d.do_st = d.dq_st = d.dk_st = d.dv_st = _triattn._st4(q)
    p = lambda x: None if x is None else ctypes.c_void_p(x.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fws = lib.tri_attn_ws_bytes(ctypes.byref(d), 0)
    ws = torch.empty(max(fws, 1), dtype=torch.uint8, device="cuda")
    _lib.check(lib.tri_attn_fwd(ctypes.byref(d), p(q), p(k), p(v), p(bias), p(mask_u8), p(o), p(lse), p(ws), fws,
                                stream), "tri_attn_fwd")

    def grads():
        return [torch.empty_like(q), torch.empty_like(q), torch.empty_like(q),
                torch.empty(B, H, N, N, dtype=torch.float32, device="cuda")]

    want = grads()
    bws = lib.tri_attn_ws_bytes(ctypes.byref(d), 1)
    ws = torch.empty(max(bws, 1), dtype=torch.uint8, device="cuda")
    _lib.check(lib.tri_attn_bwd(ctypes.byref(d), p(q), p(k), p(v), p(bias), p(mask_u8), p(o), p(lse), p(d_o),
                                *[p(g) for g in want], p(ws), bws, stream), "tri_attn_bwd")
    got = grads()
    _lib.check(lib.tri_attn_bwd_noalloc(ctypes.byref(d), p(q), p(k), p(v), p(bias), p(mask_u8), p(o), p(lse), p(d_o),
                                        *[p(g) for g in got], stream), "tri_attn_bwd_noalloc")
    torch.cuda.synchronize()
    cos_min, fro = util.ATTN_TOL[dtype, "ieee"]
    for name, a, b in zip(("dq", "dk", "dv", "dbias"), got, want):
        util.check_close(name, a, util.f64(b), cos_min, util.IEEE_REL_FRO if dtype == torch.float32 else fro)
    # and on its own feet: against the oracle (the softmax statistics it consumed came from the forward above)
    _, g_ref = util.attn_oracle(t, mask, None, d_o)
    for name, a, key in zip(("dq", "dk", "dv", "dbias"), got, ("q", "k", "v", "bias")):
        util.check_close(name + " vs oracle", a, g_ref[key].reshape(a.shape), cos_min,
                         util.IEEE_REL_FRO if dtype == torch.float32 else fro)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_two_calls_in_a_row_match_the_workspace_entry_point(dtype):
    # the second call finds the shared scratch full of the first call's values, and a different shape
    _run(dtype, (1, 16, 96, 4, 32), seed=1)
    _run(dtype, (2, 5, 37, 2, 16), seed=2)


def test_sizes_beyond_the_built_in_scratch_are_refused():
    from geometric_nn_ops_b200 import _lib

    lib = _lib.load()
    d = _lib.TriAttnDesc()
    d.B, d.n_seq, d.n_res, d.H, d.D, d.dtype = 1, 1024, 1024, 4, 32, _lib.F32
    one = torch.zeros(8, device="cuda")
    p = ctypes.c_void_p(one.data_ptr())
    rc = lib.tri_attn_bwd_noalloc(ctypes.byref(d), *([p] * 12), None)
    assert rc == -3
    assert b"exceeds the built-in scratch" in lib.tri_last_error()

"""triangle_attention on the GPU against the oracle, golden fixtures and known answers.

Known-answer and structural cases mirror the reference's tests/test_triangle_attention.py
(single unmasked key :88-104, uniform softmax :107-126, mask=None == all-keep :129-141,
masked perturbations :144-216, no-bias == zero-bias :219-232, fully masked row :235-300,
mask dtype :303-313, default scale :341-355, ranks :358-426, dynamic :429-443,
precision :451-484, accuracy grid :491-509).
"""

import glob
import os

import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu

GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "attn_*.npz")))


@pytest.fixture(scope="module")
def ta():
    from geometric_nn_ops_b200.triangle import triangle_attention
    return triangle_attention


def _tol(dtype, precision):
    cos_min, fro = util.ATTN_TOL[dtype, precision]
    if dtype == torch.float32 and precision == "ieee":
        return cos_min, util.IEEE_REL_FRO, util.MAX_ABS_REL["ieee32"]
    if dtype == torch.float32:
        return cos_min, fro, util.MAX_ABS_REL["tf32"]
    return cos_min, fro, util.MAX_ABS_REL[dtype]


@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p) for p in GOLD])
def test_golden_fp32_ieee(ta, path):
    g = dict(np.load(path))
    scale = None if g["scale"] < 0 else float(g["scale"])
    dev = lambda n: torch.from_numpy(g[n]).cuda() if n in g else None  # noqa: E731
    t = {"q": dev("q"), "k": dev("k"), "v": dev("v"), "bias": dev("bias")}
    mask = dev("mask")
    with util.matmul_precision("ieee"):
        out, grads = util.attn_fwd_bwd(ta, t, mask, scale, dev("d_out"))
    util.check_close("out", out, g["out"], 1 - 1e-9, util.IEEE_REL_FRO, 1e-4)
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g["grad_" + name], 1 - 1e-9, util.IEEE_REL_FRO, 1e-4)


SHAPES = [(1, 8, 8, 2, 8), (2, 5, 37, 3, 16), (1, 16, 100, 4, 32), (1, 3, 130, 2, 64), (1, 4, 65, 1, 48),
          (1, 4, 64, 4, 32), (1, 6, 136, 4, 32), (2, 3, 256, 2, 64), (1, 2, 384, 4, 32),
          (1, 9, 72, 2, 32),     # 9 rows: the bias gradient is summed over four row chunks, the last one empty
          (1, 3, 200, 2, 64)]    # head dim 64 with a ragged second key tile
MODES = [(torch.float32, "ieee"), (torch.float32, "tf32"), (torch.bfloat16, "ieee"), (torch.float16, "ieee")]


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("dtype,precision", MODES, ids=lambda v: str(v).replace("torch.", ""))
def test_oracle_fwd_bwd(ta, shape, dtype, precision):
    t, mask, d_out = util.attn_inputs(*shape, dtype, seed=sum(shape))
    from geometric_nn_ops_b200 import _lib
    with util.matmul_precision(precision):
        with torch.no_grad():
            ta(t["q"], t["k"], t["v"], t["bias"], mask)
        tensor_core = dtype != torch.float32 and shape[4] in (32, 64) and shape[2] % 8 == 0
        assert _lib.last_path() == ("tcgen05" if tensor_core else "simt")
        out, grads = util.attn_fwd_bwd(ta, t, mask, None, d_out)
        torch.cuda.synchronize()
        assert _lib.last_path() == ("tcgen05" if tensor_core else "simt")  # the backward ran last
    o_ref, g_ref = util.attn_oracle(t, mask, None, d_out)
    cos_min, fro, mar = _tol(dtype, precision)
    util.check_close("out", out, o_ref, cos_min, fro, mar)
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro, mar)


@pytest.mark.parametrize("n,dtype", [(256, torch.bfloat16), (128, torch.float32)])
def test_baseline_config_forward(ta, n, dtype):
    """BASELINE config 1 (bf16, B=1, N=256, H=4, D=32, keep 0.95) in the cuequivariance layout."""
    t, mask, _ = util.attn_inputs(1, n, n, 4, 32, dtype, seed=1, keep=0.95)
    cueq = {k: (v.transpose(-2, -3).contiguous().transpose(-2, -3) if k != "bias" else v) for k, v in t.items()}
    with torch.no_grad():
        out = ta(cueq["q"], cueq["k"], cueq["v"], cueq["bias"], mask, 32 ** -0.5)
    assert out.stride() == cueq["q"].stride()
    o_ref, _ = util.attn_oracle(t, mask, 32 ** -0.5, torch.zeros_like(t["q"]))
    util.check_close("out", out, o_ref, *_tol(dtype, "ieee"))


def test_single_unmasked_key_returns_its_value(ta):
    t, _, _ = util.attn_inputs(1, 3, 19, 2, 16, torch.float32, seed=3)
    mask = torch.zeros(1, 3, 1, 1, 19, dtype=torch.bool, device="cuda")
    mask[..., 7] = True
    out = ta(t["q"], t["k"], t["v"], t["bias"], mask)
    want = t["v"][:, :, 7:8].expand_as(out)
    assert torch.equal(out, want)


def test_zero_query_gives_mean_of_values(ta):
    B, S, N, H, D = 1, 2, 24, 2, 8
    g = torch.Generator().manual_seed(0)
    v = torch.randint(-4, 5, (B, S, N, H, D), generator=g).float().cuda()
    q = torch.zeros_like(v)
    k = torch.randn(B, S, N, H, D, generator=g).cuda()
    out = ta(q, k, v)
    want = v.mean(dim=2, keepdim=True).expand_as(out)
    assert (out - want).abs().max() <= 2 * torch.finfo(torch.float32).eps * want.abs().max()


@pytest.mark.parametrize("n", [70, 136])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_structural_bit_exact(ta, dtype, n):
    t, mask, _ = util.attn_inputs(1, 4, n, 2, 32, dtype, seed=5)
    base = ta(t["q"], t["k"], t["v"], t["bias"], mask)
    # mask=None equals an all-keep mask
    keep = torch.ones_like(mask)
    assert torch.equal(ta(t["q"], t["k"], t["v"], t["bias"], None), ta(t["q"], t["k"], t["v"], t["bias"], keep))
    # bias=None equals a zero bias
    assert torch.equal(ta(t["q"], t["k"], t["v"], None, mask),
                       ta(t["q"], t["k"], t["v"], torch.zeros_like(t["bias"]), mask))
    # noise on masked keys / values changes nothing
    dropped = ~mask.reshape(1, 4, n, 1, 1).expand_as(t["v"])
    noise = 1e3 * torch.randn_like(t["v"].float()).to(dtype)
    v2 = torch.where(dropped, t["v"] + noise, t["v"])
    k2 = torch.where(dropped, t["k"] + noise, t["k"])
    assert torch.equal(ta(t["q"], t["k"], v2, t["bias"], mask), base)
    assert torch.equal(ta(t["q"], k2, t["v"], t["bias"], mask), base)
    # dynamic / use_exp2 flags are accepted and change nothing
    assert torch.equal(ta(t["q"], t["k"], t["v"], t["bias"], mask, None, True, False), base)
    # run twice: deterministic
    assert torch.equal(ta(t["q"], t["k"], t["v"], t["bias"], mask), base)


@pytest.mark.parametrize("n,d", [(40, 16), (136, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fully_masked_row_is_uniform(ta, dtype, n, d):
    t, mask, d_out = util.attn_inputs(1, 3, n, 2, d, dtype, seed=6, bias_scale=0.1)
    mask[0, 1] = False
    out, grads = util.attn_fwd_bwd(ta, t, mask, None, d_out)
    want = t["v"][0, 1].float().mean(dim=0)
    got = out[0, 1].float()
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)
    o_ref, g_ref = util.attn_oracle(t, mask, None, d_out)
    cos_min, fro, _ = _tol(dtype, "ieee")
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro)


def test_mask_must_be_bool(ta):
    t, mask, _ = util.attn_inputs(1, 2, 8, 1, 8, torch.float32)
    with pytest.raises(ValueError, match="mask must be bool"):
        ta(t["q"], t["k"], t["v"], t["bias"], mask.float())


def test_ranks_and_broadcasts(ta):
    t, mask, _ = util.attn_inputs(2, 3, 20, 2, 8, torch.float32, seed=7)
    full = ta(t["q"], t["k"], t["v"], t["bias"], mask, 0.5)
    # rank 4 (no batch) with 4-D bias and lower-rank mask
    o4 = ta(t["q"][0], t["k"][0], t["v"][0], t["bias"][0], mask[0], 0.5)
    assert o4.shape == t["q"][0].shape and torch.equal(o4, full[0])
    # rank 6: two leading dims fold into the batch
    r6 = lambda x: x.reshape(2, 1, *x.shape[1:])  # noqa: E731
    o6 = ta(r6(t["q"]), r6(t["k"]), r6(t["v"]), r6(t["bias"]), r6(mask), 0.5)
    assert o6.shape == r6(t["q"]).shape and torch.equal(o6.reshape(full.shape), full)
    # batch-broadcast bias: its gradient is the batch sum
    b1 = t["bias"][:1].clone().requires_grad_()
    out = ta(t["q"], t["k"], t["v"], b1, mask, 0.5)
    (gb,) = torch.autograd.grad(out, [b1], grad_outputs=torch.ones_like(out))
    tt = dict(t, bias=t["bias"][:1].expand(2, -1, -1, -1, -1).contiguous())
    _, g_ref = util.attn_oracle(tt, mask, 0.5, torch.ones_like(out))
    util.check_close("grad_bias", gb, g_ref["bias"].sum(axis=0, keepdims=True), 1 - 1e-9, 1e-5)
    # fp64 inputs are computed in fp32 and cast back
    o64 = ta(t["q"].double(), t["k"].double(), t["v"].double(), t["bias"].double(), mask, 0.5)
    assert o64.dtype == torch.float64 and torch.equal(o64.float(), full)


def test_tf32_differs_from_ieee(ta):
    t, mask, d_out = util.attn_inputs(1, 4, 64, 2, 32, torch.float32, seed=8)
    with util.matmul_precision("ieee"):
        o1, g1 = util.attn_fwd_bwd(ta, t, mask, None, d_out)
    with util.matmul_precision("tf32"):
        o2, g2 = util.attn_fwd_bwd(ta, t, mask, None, d_out)
    assert not torch.equal(o1, o2)
    for name in g1:
        assert not torch.equal(g1[name], g2[name]), name


def test_rows_are_independent_at_full_size(ta):
    """Size-independent property at the headline size: a row's result does not depend on the others."""
    t, mask, _ = util.attn_inputs(1, 768, 768, 4, 32, torch.bfloat16, seed=9, keep=0.95)
    with torch.no_grad():
        full = ta(t["q"], t["k"], t["v"], t["bias"], mask)
        part = ta(t["q"][:, 100:164], t["k"][:, 100:164], t["v"][:, 100:164], t["bias"], mask[:, 100:164])
    assert torch.equal(full[:, 100:164], part)
    assert torch.isfinite(full.float()).all()
    # every output is a convex combination of that row's values
    vmax = t["v"].float().amax(dim=2, keepdim=True)
    vmin = t["v"].float().amin(dim=2, keepdim=True)
    assert (full.float() <= vmax + 1e-2).all() and (full.float() >= vmin - 1e-2).all()


# ---- the sizes BASELINE.json times, against the oracle -------------------------------------------------------
# Rows are independent in triangle attention (a row only shares the pair bias with the others), so a slice of rows at
# the full N_res = N_seq size runs exactly the tile loops, masks and key counts of the full problem while the fp64
# oracle stays cheap; the bias gradient is the sum over the rows of the slice.
@pytest.mark.parametrize("n,rows", [(512, 16), (768, 16), (768, 64)], ids=lambda v: str(v))
def test_baseline_sizes_row_slice_fwd_bwd(ta, n, rows):
    """BASELINE config 2 (N=512) and the headline size (N=768): bf16, H=4, D=32, keep 0.95, first key kept."""
    from geometric_nn_ops_b200 import _lib
    t, mask, d_out = util.attn_inputs(1, rows, n, 4, 32, torch.bfloat16, seed=n + rows, keep=0.95)
    out, grads = util.attn_fwd_bwd(ta, t, mask, 32 ** -0.5, d_out)
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05"
    cos_min, fro, mar = _tol(torch.bfloat16, "ieee")
    o_ref = np.empty(out.shape)
    g_ref = {k: np.empty(v.shape) for k, v in grads.items()}
    g_ref["bias"][:] = 0.0
    for r0 in range(0, rows, 8):      # oracle in row chunks: the fp64 logits of 8 rows are 150 MB at N=768
        sl = slice(r0, r0 + 8)
        tt = {k: (v[:, sl] if k != "bias" else v) for k, v in t.items()}
        o_c, g_c = util.attn_oracle(tt, mask[:, sl], 32 ** -0.5, d_out[:, sl])
        o_ref[:, sl] = o_c
        for k in ("q", "k", "v"):
            g_ref[k][:, sl] = g_c[k]
        g_ref["bias"] += g_c["bias"]
    util.check_close("out", out, o_ref, cos_min, fro, mar)
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro, mar)


def test_headline_full_size_against_oracle_rows_and_row_additivity(ta):
    """The full N_seq = N_res = 768 problem bench.py times: a slice of rows of out / dq / dk / dv against the fp64
    oracle, and the full bias gradient against the sum of the bias gradients of row blocks run on their own."""
    from geometric_nn_ops_b200 import _lib
    n = 768
    t, mask, d_out = util.attn_inputs(1, n, n, 4, 32, torch.bfloat16, seed=11, keep=0.95)
    out, grads = util.attn_fwd_bwd(ta, t, mask, None, d_out)
    torch.cuda.synchronize()
    assert _lib.last_path() == "tcgen05"
    cos_min, fro, mar = _tol(torch.bfloat16, "ieee")
    for r0 in (0, 377, 760):
        sl = slice(r0, r0 + 8)
        tt = {k: (v[:, sl] if k != "bias" else v) for k, v in t.items()}
        o_ref, g_ref = util.attn_oracle(tt, mask[:, sl], None, d_out[:, sl])
        util.check_close("out", out[:, sl], o_ref, cos_min, fro, mar)
        for name in ("q", "k", "v"):
            util.check_close("grad_" + name, grads[name][:, sl], g_ref[name], cos_min, fro, mar)
    acc = torch.zeros_like(grads["bias"], dtype=torch.float32)
    for r0 in range(0, n, 192):
        sl = slice(r0, r0 + 192)
        tt = {k: (v[:, sl].contiguous() if k != "bias" else v) for k, v in t.items()}
        _, g = util.attn_fwd_bwd(ta, tt, mask[:, sl].contiguous(), None, d_out[:, sl].contiguous())
        acc += g["bias"].float()
    # each block's gradient is rounded to bf16 before it is summed here: four roundings against one
    util.check_close("grad_bias", grads["bias"], util.f64(acc), 1 - 1e-5, 6e-3)


@pytest.mark.parametrize("broadcast", ["heads", "queries", "heads+queries"])
def test_broadcast_bias_views_bf16(ta, broadcast):
    """A bias handed in as a broadcast view over heads or queries (zero strides) has no tensor map: the call must run
    (on the CUDA-core kernels) and agree with the oracle, forward and backward, not fail."""
    B, S, N, H, D = 1, 4, 64, 4, 32
    t, mask, d_out = util.attn_inputs(B, S, N, H, D, torch.bfloat16, seed=12)
    shape = {"heads": (B, 1, 1, N, N), "queries": (B, 1, H, 1, N), "heads+queries": (B, 1, 1, 1, N)}[broadcast]
    small = torch.randn(shape, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda().requires_grad_()
    q, k, v = (t[n].clone().requires_grad_() for n in ("q", "k", "v"))
    out = ta(q, k, v, small, mask)
    gq, gk, gv, gb = torch.autograd.grad(out, [q, k, v, small], grad_outputs=d_out)
    tt = dict(t, bias=small.detach().expand(B, 1, H, N, N).contiguous())
    o_ref, g_ref = util.attn_oracle(tt, mask, None, d_out)
    cos_min, fro, mar = _tol(torch.bfloat16, "ieee")
    util.check_close("out", out, o_ref, cos_min, fro, mar)
    for name, val in (("q", gq), ("k", gk), ("v", gv)):
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro, mar)
    dims = tuple(i for i, (a, b) in enumerate(zip(shape, (B, 1, H, N, N))) if a != b)
    util.check_close("grad_bias", gb, g_ref["bias"].sum(axis=dims, keepdims=True), cos_min, fro, mar)


def test_pairformer_point_h16_d48(ta):
    """The pairformer-style point of the reference's grid (tests/test_triangle_attention.py:591-608): H=16, D=48."""
    t, mask, d_out = util.attn_inputs(1, 4, 384, 16, 48, torch.bfloat16, seed=13, keep=0.9)
    out, grads = util.attn_fwd_bwd(ta, t, mask, None, d_out)
    o_ref, g_ref = util.attn_oracle(t, mask, None, d_out)
    cos_min, fro, mar = _tol(torch.bfloat16, "ieee")
    util.check_close("out", out, o_ref, cos_min, fro, mar)
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro, mar)


def test_rows_and_residues_swapped_in_memory_bit_exact(ta):
    """q, k, v handed in as transposed views of ``[B, N_res, N_seq, H, D]`` storage (the ending-node attention of a
    pair stack reads the projections of the untransposed pair representation this way; one of them a column
    slice of a wider buffer, as the fused projection produces it): same kernels, same bits as the contiguous call,
    forward and backward."""
    from geometric_nn_ops_b200 import _lib

    B, S, N, H, D = 1, 136, 136, 4, 32
    t, mask, d_out = util.attn_inputs(B, S, N, H, D, torch.bfloat16, seed=14)
    base = {n: t[n].clone().requires_grad_() for n in ("q", "k", "v", "bias")}
    out = ta(base["q"], base["k"], base["v"], base["bias"], mask)
    g0 = torch.autograd.grad(out, list(base.values()), grad_outputs=d_out)

    def stored_transposed(x, wide):
        y = x.detach().transpose(1, 2).contiguous()                    # [B, N_res, N_seq, H, D] in memory
        if wide:                                                       # a slice of a [..., 3*H*D] buffer
            buf = torch.zeros(B, N, S, 3 * H * D, dtype=x.dtype, device=x.device)
            buf[..., H * D:2 * H * D] = y.reshape(B, N, S, H * D)
            y = buf[..., H * D:2 * H * D].view(B, N, S, H, D)
        return y.requires_grad_()
    store = {"q": stored_transposed(t["q"], False), "k": stored_transposed(t["k"], True),
             "v": stored_transposed(t["v"], False)}
    bias = t["bias"].clone().requires_grad_()
    _lib.profile_enable(True)
    out_t = ta(store["q"].transpose(1, 2), store["k"].transpose(1, 2), store["v"].transpose(1, 2), bias, mask)
    names = set(_lib.profile_summary())
    _lib.profile_enable(False)
    assert "tc_attn_fwd" in names, names                               # the tensor-core kernels took the strides
    g1 = torch.autograd.grad(out_t, [store["q"], store["k"], store["v"], bias], grad_outputs=d_out)
    assert torch.equal(out_t, out)
    for a, b in zip(g1[:3], g0[:3]):
        assert torch.equal(a.transpose(1, 2), b)
    assert torch.equal(g1[3], g0[3])

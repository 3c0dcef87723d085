"""The drop-in ``geometric_nn_ops_torch`` facade (``dropin/``) and the route of the cuequivariance shim through it.

The reference's ``cuequivariance_ops_torch`` shim is unmodified reference code: it is imported from a checkout
named by the environment variable ``TRI_REFERENCE_CHECKOUT`` when that is set (the test is skipped otherwise,
e.g. on a GPU box that has no checkout).  What the shim imports from the facade
(cuequivariance_ops_torch/triangle_attention.py:16, triangle_multiplicative_update.py:9-10,
attention_pair_bias_torch.py:21) is checked without it too, and the GPU test calls the facade exactly the way
the shim does (cuequivariance layout in, transposes, bool cast, rank-5 result: triangle_attention.py:39-52).
"""

import importlib
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from tests import util

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "dropin")


@pytest.fixture()
def facade():
    saved_path, saved_mods = list(sys.path), {k: v for k, v in sys.modules.items() if k.startswith("geometric_nn_ops_torch")}
    for k in saved_mods:
        del sys.modules[k]
    sys.path.insert(0, DROPIN)
    try:
        yield importlib.import_module("geometric_nn_ops_torch")
    finally:
        sys.path[:] = saved_path
        for k in [k for k in sys.modules if k.startswith("geometric_nn_ops_torch")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)


def test_facade_exports_what_the_shim_imports(facade):
    import geometric_nn_ops_b200.triangle as b200
    from geometric_nn_ops_torch import _precision
    from geometric_nn_ops_torch.triangle import attention_pair_bias, triangle_attention, triangle_multiplicative_update
    from geometric_nn_ops_torch.triangle._masking import mask_val, masked_key_bias
    assert facade.__file__.startswith(DROPIN)
    assert triangle_attention is b200.triangle_attention
    assert triangle_multiplicative_update is b200.triangle_multiplicative_update
    assert attention_pair_bias is b200.attention_pair_bias
    assert _precision.IEEE == "ieee" and _precision.TF32 == "tf32" and _precision.torch_precision() in ("ieee", "tf32")
    assert mask_val(torch.bfloat16) == 1e9 and masked_key_bias(torch.tensor([True, False]), torch.float32).tolist() == [0.0, -1e9]


@pytest.mark.skipif(not os.environ.get("TRI_REFERENCE_CHECKOUT"), reason="TRI_REFERENCE_CHECKOUT names no reference checkout")
def test_unmodified_shim_routes_into_this_library():
    """In a fresh interpreter: dropin/ first on sys.path, then the reference's shim directory; the shim's three
    functions must end in this library (a CPU tensor reaches its 'no CPU implementation' error), with the
    reference's own geometric_nn_ops_torch package never imported."""
    ref = os.environ["TRI_REFERENCE_CHECKOUT"]
    code = textwrap.dedent(f"""
        import sys, warnings
        sys.path[:0] = [{DROPIN!r}, {os.path.join(ref, "hipequivariance_ops_torch")!r}]
        import torch
        import cuequivariance_ops_torch as shim
        import geometric_nn_ops_torch
        assert geometric_nn_ops_torch.__file__.startswith({DROPIN!r}), geometric_nn_ops_torch.__file__
        assert shim.__file__.startswith({ref!r}), shim.__file__
        q = torch.zeros(1, 2, 1, 4, 8)                      # cuequivariance layout (B, N, H, S, D)
        for call in (lambda: shim.triangle_attention(q, q, q, torch.zeros(1, 1, 1, 4, 4)),
                     lambda: shim.triangle_multiplicative_update(torch.zeros(1, 4, 4, 8), p_in_weight=torch.zeros(8, 8),
                         g_in_weight=torch.zeros(8, 8), p_out_weight=torch.zeros(8, 4), g_out_weight=torch.zeros(8, 8))):
            try:
                call()
            except RuntimeError as exc:
                assert "no CPU implementation" in str(exc), exc
            else:
                raise AssertionError("the call did not reach the B200 library")
        try:
            shim.triangle_multiplicative_update(torch.zeros(1, 4, 4, 8), "sideways")
        except ValueError as exc:
            assert "direction must be one of" in str(exc)
        # attention_pair_bias has a torch route for CPU tensors: it must run and return the documented pair
        s = torch.randn(2, 4, 8); qq = torch.randn(2, 2, 4, 4); z = torch.randn(1, 4, 4, 6)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            out, pz = shim.attention_pair_bias(s, qq, qq, qq, z, torch.ones(1, 4), 2, torch.randn(2, 6), torch.randn(8, 8),
                                               torch.randn(8, 8), w_ln_z=torch.ones(6))
        assert out.shape == s.shape and pz.shape == (1, 2, 4, 4)
        print("shim-ok")
    """)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0 and "shim-ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cuequivariance_layout_call_through_the_facade(facade):
    """What the shim does around the facade call, on the GPU against the oracle: (B, N, H, S, D) tensors, an int
    mask cast to bool, transposed views in, transposed view out, rank restored to 5."""
    from geometric_nn_ops_torch.triangle import triangle_attention, triangle_multiplicative_update
    t, mask, d_out = util.attn_inputs(1, 8, 128, 4, 32, torch.bfloat16, seed=21, keep=0.9)
    cueq = {k: (v.transpose(-2, -3).contiguous() if k != "bias" else v) for k, v in t.items()}   # (B, N, H, S, D)
    leaves = {k: v.clone().requires_grad_() for k, v in cueq.items()}
    out = triangle_attention(leaves["q"].transpose(-2, -3), leaves["k"].transpose(-2, -3), leaves["v"].transpose(-2, -3),
                             leaves["bias"], mask.int().bool(), None).transpose(-2, -3)
    assert out.shape == cueq["q"].shape
    grads = torch.autograd.grad(out, list(leaves.values()), grad_outputs=d_out.transpose(-2, -3))
    o_ref, g_ref = util.attn_oracle(t, mask, None, d_out)
    cos_min, fro = util.ATTN_TOL[torch.bfloat16, "ieee"]
    util.check_close("out", out.transpose(-2, -3), o_ref, cos_min, fro)
    for name, val in zip(leaves, grads):
        util.check_close("grad_" + name, val if name == "bias" else val.transpose(-2, -3), g_ref[name], cos_min, fro)
    # rank-4 input: the op returns rank 4 (the shim pads it back to 5)
    o4 = triangle_attention(cueq["q"][0].transpose(-2, -3), cueq["k"][0].transpose(-2, -3), cueq["v"][0].transpose(-2, -3),
                            cueq["bias"][0], mask[0], None)
    assert o4.dim() == 4 and torch.equal(o4, out.detach().transpose(-2, -3)[0])
    # return_aux: the statistics the reference's kernels do not expose
    o, lse, amax = triangle_attention(t["q"], t["k"], t["v"], t["bias"], mask, None, return_aux=True)
    from oracle import triangle_oracle as orc
    logits = (util.f64(t["q"]).transpose(0, 1, 3, 2, 4) * 32 ** -0.5) @ util.f64(t["k"]).transpose(0, 1, 3, 4, 2)
    logits = logits + util.f64(t["bias"]) + orc.masked_key_bias(mask.cpu().numpy(), "bfloat16")
    import numpy as np
    want_max = logits.max(axis=-1, keepdims=True)
    want_lse = want_max + np.log(np.exp(logits - want_max).sum(axis=-1, keepdims=True))
    assert lse.shape == (1, 8, 4, 128, 1) and lse.dtype == torch.float32
    assert np.abs(util.f64(lse) - want_lse).max() < 2e-2 and np.abs(util.f64(amax) - want_max).max() < 5e-2 + 5.6
    # trimul keyword call, as the shim forwards it
    x, pm, w, _ = util.trimul_inputs(1, 64, 128, 128, torch.bfloat16, seed=22)
    with torch.no_grad():
        y = triangle_multiplicative_update(x, direction="incoming", mask=pm, eps=1e-5, **w)
    y_ref = util.trimul_oracle(x, pm, w, "incoming", torch.zeros_like(x))[0]
    util.check_close("trimul out", y, y_ref, *util.TRIMUL_TOL[torch.bfloat16, "ieee"])

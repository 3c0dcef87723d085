"""attention_pair_bias against fixtures produced by the reference itself (tests/golden/apb_*.npz).

CPU: the torch-operation route in fp64, every output and gradient to 1e-10.  GPU: the route whose softmax core
runs on the CUDA triangle-attention kernels (self attention, default sentinel) in fp32 and bf16, and the
torch route for the cross-attention / explicit-``inf`` fixture.
"""

import glob
import os

import numpy as np
import pytest
import torch

GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "apb_*.npz")))
POS = ("s", "q", "k", "v", "z")


def _run(g, dtype, device):
    from geometric_nn_ops_b200.triangle import attention_pair_bias
    t = {n[3:]: torch.from_numpy(v).to(dtype).to(device).requires_grad_() for n, v in g.items() if n.startswith("in_")}
    mask = torch.from_numpy(g["mask"]).to(dtype).to(device) if "mask" in g else None
    inf = None if g["inf"] < 0 else float(g["inf"])
    kw = {n: v for n, v in t.items() if n not in POS}
    out, pz = attention_pair_bias(*[t[n] for n in POS], mask=mask, inf=inf, return_z_proj=True, **kw)
    grads = torch.autograd.grad(out, list(t.values()), grad_outputs=torch.from_numpy(g["d_out"]).to(dtype).to(device))
    return out, pz, dict(zip(t, grads))


def _rel(a, b):
    a, b = a.detach().double().cpu().numpy(), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm((a - b).ravel()) / max(np.linalg.norm(b.ravel()), 1e-30))


def test_fixtures_present():
    assert len(GOLD) == 4


@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p) for p in GOLD])
def test_torch_route_matches_reference_fp64(path):
    g = dict(np.load(path))
    out, pz, grads = _run(g, torch.float64, "cpu")
    assert _rel(out, g["out"]) < 1e-10 and _rel(pz, g["proj_z"]) < 1e-10
    for name, val in grads.items():
        assert _rel(val, g["grad_" + name]) < 1e-10, name


def test_cached_projection_and_errors():
    from geometric_nn_ops_b200.triangle import attention_pair_bias
    g = dict(np.load(os.path.join(os.path.dirname(GOLD[0]), "apb_self.npz")))     # B=2, multiplicity 3
    t = {n[3:]: torch.from_numpy(v).double() for n, v in g.items() if n.startswith("in_")}
    mask = torch.from_numpy(g["mask"]).double()
    kw = {n: v for n, v in t.items() if n not in POS}
    out, pz = attention_pair_bias(*[t[n] for n in POS], mask=mask, return_z_proj=True, **kw)
    again, none = attention_pair_bias(t["s"], t["q"], t["k"], t["v"], pz, mask=mask, z_is_projected=True,
                                      proj_g_weight=t["proj_g_weight"], proj_o_weight=t["proj_o_weight"])
    assert none is None and torch.equal(again, out)
    with pytest.raises(ValueError, match="not a multiple"):
        attention_pair_bias(t["s"][:5], t["q"][:5], t["k"][:5], t["v"][:5], t["z"], **kw)
    with pytest.raises(ValueError, match="mask batch"):
        attention_pair_bias(*[t[n] for n in POS], mask=mask[:1].expand(5, -1), **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p) for p in GOLD])
def test_gpu_matches_reference(path, dtype):
    from geometric_nn_ops_b200 import _lib
    g = dict(np.load(path))
    _lib.load().tri_reset_launch_count()
    prev = torch.backends.cuda.matmul.fp32_precision
    torch.backends.cuda.matmul.fp32_precision = "ieee"
    try:
        out, pz, grads = _run(g, dtype, "cuda")
    finally:
        torch.backends.cuda.matmul.fp32_precision = prev
    torch.cuda.synchronize()
    self_attention = g["in_q"].shape[2] == g["in_k"].shape[2] and g["inf"] < 0
    assert (_lib.launch_count() > 0) == self_attention      # the softmax core ran on this library's kernels
    # fp32: exact-fp32 kernels / torch fp32; bf16: inputs rounded to bf16 against the fp64 result on unrounded inputs
    tol = 2e-5 if dtype == torch.float32 else 6e-2
    assert _rel(out, g["out"]) < tol
    for name, val in grads.items():
        assert _rel(val, g["grad_" + name]) < (tol if dtype == torch.float32 else 1.5e-1), (name, _rel(val, g["grad_" + name]))

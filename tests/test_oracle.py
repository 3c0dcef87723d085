"""The numpy oracle against fixtures produced by the reference itself (CPU only)."""

import glob
import os

import numpy as np
import pytest

from oracle import triangle_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")
ATTN = sorted(glob.glob(os.path.join(GOLD, "attn_*.npz")))
TRIMUL = sorted(glob.glob(os.path.join(GOLD, "trimul_*.npz")))


def _close(a, b, tol=1e-11):
    scale = max(np.abs(b).max(), 1.0)
    assert a.shape == b.shape
    assert np.abs(a - b).max() <= tol * scale, np.abs(a - b).max()


def test_fixtures_present():
    assert len(ATTN) >= 5 and len(TRIMUL) >= 5


@pytest.mark.parametrize("path", ATTN, ids=[os.path.basename(p) for p in ATTN])
def test_attention_oracle_matches_reference(path):
    g = dict(np.load(path))
    scale = None if g["scale"] < 0 else float(g["scale"])
    args = (g["q"], g["k"], g["v"], g.get("bias"), g.get("mask"), scale)
    _close(orc.triangle_attention_fwd(*args), g["out"])
    dq, dk, dv, db = orc.triangle_attention_bwd(*args, g["d_out"])
    _close(dq, g["grad_q"])
    _close(dk, g["grad_k"])
    _close(dv, g["grad_v"])
    if "bias" in g:
        _close(db, g["grad_bias"])
    else:
        assert db is None


@pytest.mark.parametrize("path", TRIMUL, ids=[os.path.basename(p) for p in TRIMUL])
def test_trimul_oracle_matches_reference(path):
    g = dict(np.load(path))
    w = {k[2:]: v for k, v in g.items() if k.startswith("w_")}
    direction = str(g["direction"])
    _close(orc.trimul_fwd(g["x"], direction, g.get("mask"), **w), g["out"])
    grads = orc.trimul_bwd(g["x"], direction, g.get("mask"), g["d_out"], **w)
    assert set(grads) == {"x", *w}
    for name, val in grads.items():
        _close(val, g["grad_" + name], tol=1e-10)


def test_mask_bias_sign_and_value():
    m = np.array([True, False])
    b = orc.masked_key_bias(m, np.float32)
    assert b[0] == 0 and not np.signbit(b[0]) and b[1] == np.float32(-1e9)
    assert orc.mask_val(np.float64) == 1e18 and orc.mask_val(np.float16) == 65504 / 2


def test_bad_direction():
    with pytest.raises(ValueError, match="direction must be one of"):
        orc.trimul_fwd(np.zeros((2, 2, 4)), "sideways", None, p_in_weight=np.zeros((4, 4)))


# ---- the torch restatement that bench.py times on the host cores, against the same fixtures ---------------------
def _t64(a):
    import torch
    return None if a is None else torch.from_numpy(np.asarray(a)).double() if np.asarray(a).dtype != bool else torch.from_numpy(a)


@pytest.mark.parametrize("path", ATTN, ids=[os.path.basename(p) for p in ATTN])
def test_torch_restatement_attention_matches_reference(path):
    from oracle import torch_reference as tr
    g = dict(np.load(path))
    scale = None if g["scale"] < 0 else float(g["scale"])
    q, k, v, d_out = (_t64(g[n]) for n in ("q", "k", "v", "d_out"))
    bias, mask = _t64(g.get("bias")), _t64(g.get("mask"))
    for chunk in (None, 2):     # whole problem, and row blocks with the bias gradient summed over blocks
        out, dq, dk, dv, db = tr.attention_fwd_bwd(q, k, v, bias, mask, scale, d_out, row_chunk=chunk)
        _close(out.numpy(), g["out"])
        _close(dq.numpy(), g["grad_q"])
        _close(dk.numpy(), g["grad_k"])
        _close(dv.numpy(), g["grad_v"])
        if bias is not None:
            _close(db.numpy(), g["grad_bias"])


@pytest.mark.parametrize("path", TRIMUL, ids=[os.path.basename(p) for p in TRIMUL])
def test_torch_restatement_trimul_matches_reference(path):
    from oracle import torch_reference as tr
    g = dict(np.load(path))
    w = {k[2:]: _t64(v) for k, v in g.items() if k.startswith("w_")}
    out, grads = tr.trimul_fwd_bwd(_t64(g["x"]), str(g["direction"]), _t64(g.get("mask")), w, _t64(g["d_out"]))
    _close(out.numpy(), g["out"])
    for name, val in grads.items():
        _close(val.numpy(), g["grad_" + name], tol=1e-10)

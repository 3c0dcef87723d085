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

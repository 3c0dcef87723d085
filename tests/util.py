"""Seeded input builders and oracle comparison helpers shared by the tests.

Inputs are drawn on the CPU in fp32 from a seeded generator, rounded to the test dtype,
and then handed both to the CUDA library (as torch tensors) and to the numpy oracle (as
float64 arrays of the SAME rounded values), following the reference's protocol
(testutil/triangle_attention.py:81-108, testutil/trimul.py:207-231).
"""

import contextlib

import numpy as np
import torch

from oracle import triangle_oracle as orc

# (cos_min, rel_fro_max) against the fp64 oracle: the reference's own tables
# (testutil/metrics.py:96-108), applied to the forward and to every gradient.
TRIMUL_TOL = {
    (torch.float32, "ieee"): (1.0 - 1e-6, 1.5e-3),
    (torch.float32, "tf32"): (1.0 - 1e-6, 2e-3),
    (torch.float16, "ieee"): (1.0 - 1e-6, 2e-3),
    (torch.bfloat16, "ieee"): (1.0 - 1e-4, 1.5e-2),
}
ATTN_TOL = {
    (torch.float32, "ieee"): (1.0 - 1e-5, 1.5e-3),
    (torch.float32, "tf32"): (1.0 - 1e-5, 2e-3),
    (torch.float16, "ieee"): (1.0 - 1e-4, 2e-2),
    (torch.bfloat16, "ieee"): (1.0 - 1e-4, 5e-2),
}
# Tighter bound this build holds exact-fp32 results to (the reference's table allows 1.5e-3).
IEEE_REL_FRO = 1e-5
# max|a-b| / max|b| bounds stated for this build.
MAX_ABS_REL = {"ieee32": 1e-4, "tf32": 5e-3, torch.bfloat16: 2e-2, torch.float16: 5e-3}


@contextlib.contextmanager
def matmul_precision(precision):
    matmul = torch.backends.cuda.matmul
    prev = matmul.fp32_precision
    matmul.fp32_precision = precision
    try:
        yield
    finally:
        matmul.fp32_precision = prev


def f64(t):
    return None if t is None else t.detach().double().cpu().numpy()


def attn_inputs(B, S, N, H, D, dtype, *, seed=0, with_bias=True, with_mask=True, keep=0.75, bias_scale=1.0,
                device="cuda"):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    t = {"q": rn(B, S, N, H, D), "k": rn(B, S, N, H, D), "v": rn(B, S, N, H, D)}
    t["bias"] = rn(B, 1, H, N, N) * bias_scale if with_bias else None
    mask = None
    if with_mask:
        mask = torch.rand(B, S, 1, 1, N, generator=g) < keep
        mask[..., 0] = True
    d_out = rn(B, S, N, H, D)
    t = {k: (None if v is None else v.to(dtype).to(device)) for k, v in t.items()}
    return t, (None if mask is None else mask.to(device)), d_out.to(dtype).to(device)


def trimul_inputs(B, N, C, Ch, dtype, *, seed=0, biases=False, with_mask=True, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc  # noqa: E731
    x = rn(B, N, N, C)
    mask = (torch.rand(B, N, N, generator=g) < 0.9).float() if with_mask else None
    w = {
        "norm_in_weight": 1 + rn(C, sc=0.02), "norm_in_bias": rn(C, sc=0.02),
        "p_in_weight": rn(2 * Ch, C, sc=C ** -0.5), "g_in_weight": rn(2 * Ch, C, sc=C ** -0.5),
        "norm_out_weight": 1 + rn(Ch, sc=0.02), "norm_out_bias": rn(Ch, sc=0.02),
        "p_out_weight": rn(C, Ch, sc=Ch ** -0.5), "g_out_weight": rn(C, C, sc=C ** -0.5),
    }
    if biases:
        w |= {"p_in_bias": rn(2 * Ch, sc=0.05), "g_in_bias": rn(2 * Ch, sc=0.05),
              "p_out_bias": rn(C, sc=0.05), "g_out_bias": rn(C, sc=0.05)}
    d_out = rn(B, N, N, C)
    cv = lambda t: None if t is None else t.to(dtype).to(device)  # noqa: E731
    return cv(x), cv(mask), {k: cv(v) for k, v in w.items()}, cv(d_out)


def check_close(name, got, want, cos_min, fro_max, max_abs_rel=None):
    got = f64(got) if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{name}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{name}: non-finite values"
    c, f = orc.cos(got, want), orc.rel_fro(got, want)
    assert c >= cos_min, f"{name}: cos {c:.8f} < {cos_min}"
    assert f <= fro_max, f"{name}: rel-fro {f:.3e} > {fro_max:.1e}"
    if max_abs_rel is not None:
        m = orc.max_abs_rel(got, want)
        assert m <= max_abs_rel, f"{name}: max-abs/max|ref| {m:.3e} > {max_abs_rel:.1e}"
    return c, f


def attn_fwd_bwd(fn, t, mask, scale, d_out):
    leaves = {k: v.detach().clone().requires_grad_() for k, v in t.items() if v is not None}
    out = fn(leaves["q"], leaves["k"], leaves["v"], leaves.get("bias"), mask, scale)
    grads = torch.autograd.grad(out, list(leaves.values()), grad_outputs=d_out)
    return out, dict(zip(leaves, grads))


def attn_oracle(t, mask, scale, d_out):
    a = (f64(t["q"]), f64(t["k"]), f64(t["v"]), f64(t["bias"]), None if mask is None else mask.cpu().numpy(), scale)
    out = orc.triangle_attention_fwd(*a)
    dq, dk, dv, db = orc.triangle_attention_bwd(*a, f64(d_out))
    return out, {"q": dq, "k": dk, "v": dv, "bias": db}


def trimul_fwd_bwd(fn, x, mask, w, direction, d_out):
    xl = x.detach().clone().requires_grad_()
    wl = {k: v.detach().clone().requires_grad_() for k, v in w.items()}
    out = fn(xl, direction, mask, **wl)
    grads = torch.autograd.grad(out, [xl, *wl.values()], grad_outputs=d_out)
    return out, dict(zip(["x", *wl], grads))


def trimul_oracle(x, mask, w, direction, d_out):
    wn = {k: f64(v) for k, v in w.items()}
    out = orc.trimul_fwd(f64(x), direction, f64(mask), **wn)
    grads = orc.trimul_bwd(f64(x), direction, f64(mask), f64(d_out), **wn)
    return out, grads

"""CPU oracle for the two triangle ops: TEST INFRASTRUCTURE, not a product path.

A numpy restatement of the reference's pure-torch algorithms, used only as the
checker in ``tests/``, in ``__graft_entry__.smoke()`` and as the timed CPU
baseline of ``bench.py``.  The library itself never imports this module; the
product path is the CUDA extension and fails loudly when that is missing.

Parity status: PINNED.  ``tests/test_oracle.py`` checks every function here
against fixtures in ``tests/golden/`` that were produced by running the
reference's own code (``geometric_nn_ops_torch.triangle._reference``) in fp64,
forward and ``torch.autograd`` backward; ``tests/golden/make_golden.py`` is the
generating script.

Reference functions restated (paths inside the reference project):

* ``mask_val`` / ``masked_key_bias``   geometric_nn_ops_torch/triangle/_masking.py:13-42
* ``triangle_attention_fwd``           geometric_nn_ops_torch/triangle/_reference/triangle_attention.py:11-44
* ``trimul_fwd``                       geometric_nn_ops_torch/triangle/_reference/trimul.py:57-97
  (combine step: ``_combine_projections`` :44-54)

The backward functions have no hand-written counterpart in the reference (it
differentiates the forward with autograd); they are the analytic gradients of
the same forward and are pinned against autograd outputs in the fixtures.

Layouts are the reference's: q/k/v ``[B, N_seq, N_res, H, D]``, bias
``[B, 1, H, N_res, N_res]`` (batch may be 1), mask bool ``[B, N_seq, 1, 1, N_res]``;
x ``[*, N, N, C]``, pair mask ``[*, N, N]``.
"""

from __future__ import annotations

import numpy as np

DIRECTIONS = ("outgoing", "incoming")


# --------------------------------------------------------------------------- #
# masking helpers (_masking.py:13-42)
# --------------------------------------------------------------------------- #
def mask_val(dtype) -> float:
    """Distance a masked key's logit is pushed down, per accumulate dtype."""
    dtype = np.dtype(dtype) if not isinstance(dtype, str) else dtype
    if dtype == np.float64:
        return 1e18
    if dtype == np.float32 or dtype == "bfloat16":
        return 1e9
    if dtype == np.float16:
        return float(np.finfo(np.float16).max) / 2
    raise ValueError(f"Unsupported dtype {dtype}")


def masked_key_bias(mask: np.ndarray, dtype) -> np.ndarray:
    """bool mask -> additive bias: +0.0 where kept, -mask_val where masked.

    Spelled ``val * (float32(mask) - 1)`` exactly as the reference does, so that
    kept keys get +0.0 (not -0.0) and the product is formed in fp32.
    """
    return np.float32(mask_val(dtype)) * (mask.astype(np.float32) - np.float32(1))


# --------------------------------------------------------------------------- #
# triangle attention
# --------------------------------------------------------------------------- #
def _attn_probs(q, k, bias, mask, scale, acc):
    d = q.shape[-1]
    if scale is None:
        scale = d ** -0.5
    qs = np.swapaxes(q, -2, -3).astype(acc)  # [B, S, H, N, D]
    ks = np.swapaxes(k, -2, -3).astype(acc)
    logits = np.matmul(qs * acc(scale), np.swapaxes(ks, -1, -2))  # [B,S,H,N,N]
    if bias is not None:
        if bias.ndim == 4:
            bias = bias[:, None]
        logits = logits + bias.astype(acc)
    if mask is not None:
        logits = logits + masked_key_bias(mask, acc).astype(acc)
    logits = logits - logits.max(axis=-1, keepdims=True)
    p = np.exp(logits)
    p /= p.sum(axis=-1, keepdims=True)
    return p, scale


def triangle_attention_fwd(q, k, v, bias=None, mask=None, scale=None, acc=np.float64):
    """``O = softmax_j(scale q.k + bias + maskbias) V``; returns ``[B,S,N,H,D]`` in ``acc``."""
    p, _ = _attn_probs(q, k, bias, mask, scale, acc)
    vs = np.swapaxes(v, -2, -3).astype(acc)
    o = np.matmul(p, vs)  # [B,S,H,N,D]
    return np.swapaxes(o, -2, -3)


def triangle_attention_bwd(q, k, v, bias, mask, scale, d_out, acc=np.float64):
    """Analytic gradients of :func:`triangle_attention_fwd`.

    Returns ``(dq, dk, dv, dbias)``; ``dbias`` has the shape of ``bias``
    (summed over the row axis and over a broadcast batch), or ``None``.
    """
    p, scale = _attn_probs(q, k, bias, mask, scale, acc)
    qs = np.swapaxes(q, -2, -3).astype(acc)
    ks = np.swapaxes(k, -2, -3).astype(acc)
    vs = np.swapaxes(v, -2, -3).astype(acc)
    do = np.swapaxes(d_out, -2, -3).astype(acc)  # [B,S,H,N,D]
    dv = np.matmul(np.swapaxes(p, -1, -2), do)
    dp = np.matmul(do, np.swapaxes(vs, -1, -2))
    ds = p * (dp - (dp * p).sum(axis=-1, keepdims=True))
    dq = np.matmul(ds, ks) * acc(scale)
    dk = np.matmul(np.swapaxes(ds, -1, -2), qs) * acc(scale)
    dbias = None
    if bias is not None:
        dbias = ds.sum(axis=1, keepdims=True)  # over rows -> [B,1,H,N,N]
        b5 = bias if bias.ndim == 5 else bias[:, None]
        if b5.shape[0] == 1 and dbias.shape[0] != 1:
            dbias = dbias.sum(axis=0, keepdims=True)
        dbias = dbias.reshape(bias.shape)
    sw = lambda t: np.swapaxes(t, -2, -3)  # noqa: E731
    return sw(dq), sw(dk), sw(dv), dbias


# --------------------------------------------------------------------------- #
# triangle multiplicative update
# --------------------------------------------------------------------------- #
def _check_direction(direction: str) -> bool:
    if direction not in DIRECTIONS:
        raise ValueError(f"direction must be one of {DIRECTIONS}, got {direction!r}")
    return direction == "outgoing"


def _sigmoid(t):
    return 1.0 / (1.0 + np.exp(-t))


def _layer_norm(t, w, b, eps):
    mu = t.mean(axis=-1, keepdims=True)
    var = ((t - mu) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    hat = (t - mu) * rstd
    out = hat
    if w is not None:
        out = out * w
    if b is not None:
        out = out + b
    return out, hat, rstd


def _layer_norm_bwd(d_out, hat, rstd, w):
    dhat = d_out * w if w is not None else d_out
    m1 = dhat.mean(axis=-1, keepdims=True)
    m2 = (dhat * hat).mean(axis=-1, keepdims=True)
    d_in = rstd * (dhat - m1 - hat * m2)
    lead = tuple(range(d_out.ndim - 1))
    return d_in, (d_out * hat).sum(axis=lead), d_out.sum(axis=lead)


def _linear(t, w, b):
    y = np.matmul(t, w.T)
    return y if b is None else y + b


def _cm(t):
    """[*, r, s, c] -> channel-major [*, c, r, s] (contiguous, so matmul goes to BLAS)."""
    return np.ascontiguousarray(np.moveaxis(t, -1, -3))


def _pm(t):
    """channel-major [*, c, r, s] -> [*, r, s, c]."""
    return np.moveaxis(t, -3, -1)


def _T(t):
    return np.swapaxes(t, -1, -2)


def _combine(a, b, outgoing):
    """t[i,j,c] = sum_k a[i,k,c] b[j,k,c] (outgoing) or sum_k a[k,i,c] b[k,j,c] (incoming)."""
    a, b = _cm(a), _cm(b)
    return _pm(np.matmul(a, _T(b)) if outgoing else np.matmul(_T(a), b))


def trimul_fwd(
    x, direction="outgoing", mask=None, *, eps=1e-5,
    norm_in_weight=None, norm_in_bias=None, p_in_weight=None, p_in_bias=None,
    g_in_weight=None, g_in_bias=None, norm_out_weight=None, norm_out_bias=None,
    p_out_weight=None, p_out_bias=None, g_out_weight=None, g_out_bias=None,
    acc=np.float64, _cache=None,
):
    """LN -> p_in * sigmoid(g_in) * mask -> per-channel contraction -> LN -> p_out * sigmoid(g_out)."""
    outgoing = _check_direction(direction)
    cv = lambda t: None if t is None else np.asarray(t).astype(acc)  # noqa: E731
    x = cv(x)
    ch = p_in_weight.shape[0] // 2
    z, zhat, rstd_in = _layer_norm(x, cv(norm_in_weight), cv(norm_in_bias), eps)
    pp = _linear(z, cv(p_in_weight), cv(p_in_bias))
    gg = _sigmoid(_linear(z, cv(g_in_weight), cv(g_in_bias)))
    ab = pp * gg
    if mask is not None:
        ab = ab * cv(mask)[..., None]
    a, b = ab[..., :ch], ab[..., ch:]
    t = _combine(a, b, outgoing)
    u, that, rstd_out = _layer_norm(t, cv(norm_out_weight), cv(norm_out_bias), eps)
    y = _linear(u, cv(p_out_weight), cv(p_out_bias))
    go = _sigmoid(_linear(z, cv(g_out_weight), cv(g_out_bias)))
    if _cache is not None:
        _cache.update(z=z, zhat=zhat, rstd_in=rstd_in, pp=pp, gg=gg, a=a, b=b,
                      u=u, that=that, rstd_out=rstd_out, y=y, go=go)
    return y * go


def trimul_bwd(x, direction, mask, d_out, *, eps=1e-5, acc=np.float64, **weights):
    """Analytic gradients of :func:`trimul_fwd` wrt ``x`` and every weight given.

    Returns a dict keyed ``"x"`` plus the names of the weights that are not None.
    """
    outgoing = _check_direction(direction)
    cv = lambda t: None if t is None else np.asarray(t).astype(acc)  # noqa: E731
    w = {name: cv(val) for name, val in weights.items()}
    c = {}
    trimul_fwd(x, direction, mask, eps=eps, acc=acc, _cache=c, **weights)
    d_out = cv(d_out)
    lead = tuple(range(d_out.ndim - 1))
    flat = lambda t: t.reshape(-1, t.shape[-1])  # noqa: E731
    grads = {}

    dy = d_out * c["go"]
    dgo = d_out * c["y"] * c["go"] * (1.0 - c["go"])
    grads["p_out_weight"] = flat(dy).T @ flat(c["u"])
    grads["p_out_bias"] = dy.sum(axis=lead)
    grads["g_out_weight"] = flat(dgo).T @ flat(c["z"])
    grads["g_out_bias"] = dgo.sum(axis=lead)
    du = np.matmul(dy, w["p_out_weight"])
    dt, grads["norm_out_weight"], grads["norm_out_bias"] = _layer_norm_bwd(
        du, c["that"], c["rstd_out"], w.get("norm_out_weight"))
    a, b = c["a"], c["b"]
    a_c, b_c, dt_c = _cm(a), _cm(b), _cm(dt)
    if outgoing:   # t = a b^T
        da, db = _pm(np.matmul(dt_c, b_c)), _pm(np.matmul(_T(dt_c), a_c))
    else:          # t = a^T b
        da, db = _pm(np.matmul(b_c, _T(dt_c))), _pm(np.matmul(a_c, dt_c))
    dab = np.concatenate([da, db], axis=-1)
    if mask is not None:
        dab = dab * cv(mask)[..., None]
    dp = dab * c["gg"]
    dg = dab * c["pp"] * c["gg"] * (1.0 - c["gg"])
    grads["p_in_weight"] = flat(dp).T @ flat(c["z"])
    grads["p_in_bias"] = dp.sum(axis=lead)
    grads["g_in_weight"] = flat(dg).T @ flat(c["z"])
    grads["g_in_bias"] = dg.sum(axis=lead)
    dz = (np.matmul(dp, w["p_in_weight"]) + np.matmul(dg, w["g_in_weight"])
          + np.matmul(dgo, w["g_out_weight"]))
    grads["x"], grads["norm_in_weight"], grads["norm_in_bias"] = _layer_norm_bwd(
        dz, c["zhat"], c["rstd_in"], w.get("norm_in_weight"))
    return {k: v for k, v in grads.items() if k == "x" or weights.get(k) is not None}


# --------------------------------------------------------------------------- #
# metrics shared by the parity tests (same definitions as the reference's
# testutil/metrics.py:26-47: flattened cosine similarity, relative Frobenius)
# --------------------------------------------------------------------------- #
def cos(a, b) -> float:
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / max(na * nb, 1e-300))


def rel_fro(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm((a - b).ravel()) / max(np.linalg.norm(b.ravel()), 1e-30))


def max_abs_rel(a, b) -> float:
    """max|a-b| / max|b| : the relative max-error figure used for gradients."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))

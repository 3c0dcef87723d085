"""The reference's pure-torch CPU path, restated: TEST INFRASTRUCTURE and timed CPU baseline, not a product path.

``bench.py --impl reference`` and the ``cpu_baseline`` leg time these functions on the host cores; the tests
hold them to the golden fixtures (outputs of the reference's own code) in fp64.  The library never imports
this module.

Parity status: PINNED (``tests/test_oracle.py::test_torch_restatement_*`` against ``tests/golden/*.npz``).

What is restated (paths inside the reference project), op for op and in the same dtype at every step, so that
a bf16 run rounds where the reference's does:

* ``cpu_triangle_attention``  geometric_nn_ops_torch/triangle/_reference/triangle_attention.py:11-44
  (logits and softmax in fp32 -- fp64 for fp64 inputs --, additive key-mask term from _masking.py:13-42,
  result cast back to q's dtype)
* ``cpu_trimul``              geometric_nn_ops_torch/triangle/_reference/trimul.py:57-97 (LayerNorm, the two
  input projections multiplied in x's dtype, mask, per-channel contraction :44-54, LayerNorm, gated output)

The reference differentiates both with autograd; so does ``fwd_bwd`` here.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

_SENTINEL = {torch.float64: 1e18, torch.float32: 1e9, torch.bfloat16: 1e9}


def _key_mask_term(mask: torch.Tensor, acc: torch.dtype) -> torch.Tensor:
    """+0.0 on kept keys, -sentinel on masked ones, formed in fp32 as ``sentinel * (mask - 1)``."""
    sentinel = torch.finfo(torch.float16).max / 2 if acc == torch.float16 else _SENTINEL[acc]
    return (sentinel * (mask.float() - 1)).to(acc)


def cpu_triangle_attention(q, k, v, bias=None, mask=None, scale=None):
    """``[B, N_seq, N_res, H, D]`` in, same shape and dtype out; bias ``[B, 1, H, N, N]`` (or 4-D), mask bool."""
    acc = torch.float64 if q.dtype == torch.float64 else torch.float32
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    qh, kh, vh = (t.transpose(2, 3).to(acc) for t in (q, k, v))          # heads before residues
    logits = torch.matmul(qh * scale, kh.transpose(-1, -2))               # [B, S, H, N, N]
    if bias is not None:
        logits = logits + (bias.unsqueeze(1) if bias.dim() == 4 else bias).to(acc)
    if mask is not None:
        logits = logits + _key_mask_term(mask, acc)
    out = torch.matmul(torch.softmax(logits, dim=-1), vh)
    return out.transpose(2, 3).to(q.dtype)


def cpu_trimul(x, direction="outgoing", mask=None, *, eps=1e-5, norm_in_weight=None, norm_in_bias=None,
               p_in_weight=None, p_in_bias=None, g_in_weight=None, g_in_bias=None, norm_out_weight=None,
               norm_out_bias=None, p_out_weight=None, p_out_bias=None, g_out_weight=None, g_out_bias=None):
    """``x`` ``[*, N, N, C]``, ``mask`` ``[*, N, N]``; every op runs in x's dtype like the reference's torch path."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be one of ('outgoing', 'incoming'), got {direction!r}")
    hidden = p_in_weight.shape[0] // 2
    z = F.layer_norm(x, x.shape[-1:], norm_in_weight, norm_in_bias, eps)
    gated = F.linear(z, p_in_weight, p_in_bias) * F.linear(z, g_in_weight, g_in_bias).sigmoid()
    if mask is not None:
        gated = gated * mask[..., None]
    a = gated[..., :hidden].movedim(-1, -3)     # channel planes [*, C, N, N]
    b = gated[..., hidden:].movedim(-1, -3)
    if direction == "outgoing":                  # t[i, j] = sum_k a[i, k] b[j, k]
        t = torch.matmul(a, b.transpose(-1, -2))
    else:                                        # t[i, j] = sum_k a[k, i] b[k, j]
        t = torch.matmul(a.transpose(-1, -2), b)
    t = F.layer_norm(t.movedim(-3, -1), (hidden,), norm_out_weight, norm_out_bias, eps)
    return F.linear(t, p_out_weight, p_out_bias) * F.linear(z, g_out_weight, g_out_bias).sigmoid()


def attention_fwd_bwd(q, k, v, bias, mask, scale, d_out, row_chunk=None):
    """Forward and autograd backward of :func:`cpu_triangle_attention`.

    Rows are independent (they share only the bias), so with ``row_chunk`` the rows are processed in blocks and
    the bias gradient is summed over the blocks: the same arithmetic, with the fp32 logits of one block
    (``row_chunk * H * N * N`` floats) alive at a time instead of all ``N_seq`` rows (7 GB at N=768).
    Returns ``(out, dq, dk, dv, dbias)``.
    """
    S = q.shape[1]
    step = S if row_chunk is None else row_chunk
    outs, dqs, dks, dvs, dbias = [], [], [], [], None
    for r0 in range(0, S, step):
        sl = slice(r0, min(S, r0 + step))
        leaves = [t[:, sl].detach().requires_grad_() for t in (q, k, v)]
        b = None if bias is None else bias.detach().requires_grad_()
        o = cpu_triangle_attention(*leaves, b, None if mask is None else mask[:, sl], scale)
        grads = torch.autograd.grad(o, leaves + ([] if b is None else [b]), grad_outputs=d_out[:, sl])
        outs.append(o.detach())
        dqs.append(grads[0]); dks.append(grads[1]); dvs.append(grads[2])
        if b is not None:
            part = grads[3].to(torch.float64 if b.dtype == torch.float64 else torch.float32)
            dbias = part if dbias is None else dbias + part
    cat = lambda ts: torch.cat(ts, dim=1)  # noqa: E731
    return cat(outs), cat(dqs), cat(dks), cat(dvs), (None if dbias is None else dbias.to(bias.dtype))


def trimul_fwd_bwd(x, direction, mask, weights, d_out):
    """Forward and autograd backward of :func:`cpu_trimul`; returns ``(out, {"x": dx, weight name: grad, ...})``."""
    xl = x.detach().requires_grad_()
    wl = {n: t.detach().requires_grad_() for n, t in weights.items()}
    out = cpu_trimul(xl, direction, mask, **wl)
    grads = torch.autograd.grad(out, [xl, *wl.values()], grad_outputs=d_out)
    return out.detach(), dict(zip(["x", *wl], grads))

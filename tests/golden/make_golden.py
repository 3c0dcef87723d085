"""Generate the golden fixtures in this folder by running the reference itself.

Run once, in a container that has the reference checked out, as

    python tests/golden/make_golden.py /path/to/reference

It imports ``geometric_nn_ops_torch.triangle._reference`` from that checkout,
runs the reference's pure-torch forward in fp64 on small seeded inputs, takes
every gradient with ``torch.autograd.grad`` and writes inputs and results to
``*.npz`` files beside this script.  The tests only read the ``.npz`` files, so
they run where the reference is absent.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def attention_case(name, B, S, N, H, D, *, bias_batch=None, with_bias=True, with_mask=True,
                   full_mask_row=False, scale=None, seed=0, ref=None):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)  # noqa: E731
    q, k, v = rn(B, S, N, H, D), rn(B, S, N, H, D), rn(B, S, N, H, D)
    bias = rn(bias_batch or B, 1, H, N, N) if with_bias else None
    mask = None
    if with_mask:
        mask = torch.rand(B, S, 1, 1, N, generator=g) < 0.75
        mask[..., 0] = True
        if full_mask_row:
            mask[0, 1] = False
    d_out = rn(B, S, N, H, D)
    leaves = {n: t.double().requires_grad_() for n, t in
              dict(q=q, k=k, v=v, bias=bias).items() if t is not None}
    out = ref(leaves["q"], leaves["k"], leaves["v"], leaves.get("bias"), mask, scale)
    grads = torch.autograd.grad(out, list(leaves.values()), grad_outputs=d_out.double())
    rec = dict(q=_np(q), k=_np(k), v=_np(v), d_out=_np(d_out), out=_np(out),
               scale=np.array(-1.0 if scale is None else scale))
    if bias is not None:
        rec["bias"] = _np(bias)
    if mask is not None:
        rec["mask"] = _np(mask)
    for n, gr in zip(leaves, grads):
        rec["grad_" + n] = _np(gr)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print("wrote", name, {k_: v_.shape for k_, v_ in rec.items()})


def trimul_case(name, lead, N, C, Ch, direction, *, biases=False, with_mask=True, seed=0, ref=None):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g, dtype=torch.float32) * sc  # noqa: E731
    x = rn(*lead, N, N, C)
    mask = (torch.rand(*lead, N, N, generator=g) < 0.9).float() if with_mask else None
    w = {
        "norm_in_weight": 1 + rn(C, sc=0.02), "norm_in_bias": rn(C, sc=0.02),
        "p_in_weight": rn(2 * Ch, C, sc=C ** -0.5), "g_in_weight": rn(2 * Ch, C, sc=C ** -0.5),
        "norm_out_weight": 1 + rn(Ch, sc=0.02), "norm_out_bias": rn(Ch, sc=0.02),
        "p_out_weight": rn(C, Ch, sc=Ch ** -0.5), "g_out_weight": rn(C, C, sc=C ** -0.5),
    }
    if biases:
        w |= {"p_in_bias": rn(2 * Ch, sc=0.05), "g_in_bias": rn(2 * Ch, sc=0.05),
              "p_out_bias": rn(C, sc=0.05), "g_out_bias": rn(C, sc=0.05)}
    d_out = rn(*lead, N, N, C)
    xd = x.double().requires_grad_()
    wd = {n: t.double().requires_grad_() for n, t in w.items()}
    out = ref(xd, direction, None if mask is None else mask.double(), **wd)
    grads = torch.autograd.grad(out, [xd, *wd.values()], grad_outputs=d_out.double())
    rec = dict(x=_np(x), d_out=_np(d_out), out=_np(out), grad_x=_np(grads[0]),
               direction=np.array(direction))
    if mask is not None:
        rec["mask"] = _np(mask)
    for (n, t), gr in zip(w.items(), grads[1:]):
        rec["w_" + n] = _np(t)
        rec["grad_" + n] = _np(gr)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print("wrote", name, {k_: v_.shape for k_, v_ in rec.items()})


def pair_bias_case(name, B, M, H, U, V, DH, Zc, *, mask_batch="B", biases=False, inf=None, seed=0, ref=None):
    """attention_pair_bias on pre-projected q, k, v (reference: _reference/attention_pair_bias.py:26-89)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, sc=1.0: torch.randn(*s, generator=g, dtype=torch.float32) * sc  # noqa: E731
    D = H * DH
    t = dict(s=rn(B * M, U, D), q=rn(B * M, H, U, DH), k=rn(B * M, H, V, DH), v=rn(B * M, H, V, DH), z=rn(B, U, V, Zc),
             proj_g_weight=rn(D, D, sc=D ** -0.5), proj_o_weight=rn(D, D, sc=D ** -0.5),
             proj_z_weight=rn(H, Zc, sc=Zc ** -0.5), ln_z_weight=1 + rn(Zc, sc=0.05))
    if biases:
        t |= dict(proj_g_bias=rn(D, sc=0.05), proj_o_bias=rn(D, sc=0.05))
    mask = None
    if mask_batch is not None:
        mask = (torch.rand(B if mask_batch == "B" else B * M, V, generator=g) < 0.8).float()
        mask[:, 0] = 1.0
    d_out = rn(B * M, U, D)
    leaves = {n: x.double().requires_grad_() for n, x in t.items()}
    pos = [leaves[n] for n in ("s", "q", "k", "v", "z")]
    kw = {n: x for n, x in leaves.items() if n not in ("s", "q", "k", "v", "z")}
    out, pz = ref(*pos, mask=None if mask is None else mask.double(), inf=inf, return_z_proj=True, **kw)
    grads = torch.autograd.grad(out, list(leaves.values()), grad_outputs=d_out.double())
    rec = {"in_" + n: _np(x) for n, x in t.items()}
    rec |= dict(d_out=_np(d_out), out=_np(out), proj_z=_np(pz), M=np.array(M), inf=np.array(-1.0 if inf is None else inf))
    if mask is not None:
        rec["mask"] = _np(mask)
    for n, gr in zip(leaves, grads):
        rec["grad_" + n] = _np(gr)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print("wrote", name, {k_: v_.shape for k_, v_ in rec.items()})


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <checkout of the reference project>")
    sys.path.insert(0, sys.argv[1])
    from geometric_nn_ops_torch.triangle._reference.triangle_attention import (
        triangle_attention_torch,
    )
    from geometric_nn_ops_torch.triangle._reference.trimul import trimul_torch

    from geometric_nn_ops_torch.triangle._reference.attention_pair_bias import (
        attention_pair_bias_torch,
    )

    a, t = triangle_attention_torch, trimul_torch
    pair_bias_case("apb_self", 2, 3, 2, 16, 16, 8, 12, ref=attention_pair_bias_torch)
    pair_bias_case("apb_self_bias_maskbm", 1, 2, 4, 24, 24, 16, 8, mask_batch="BM", biases=True, seed=1,
                   ref=attention_pair_bias_torch)
    pair_bias_case("apb_cross_inf", 2, 1, 2, 6, 10, 8, 8, inf=1e6, seed=2, ref=attention_pair_bias_torch)
    pair_bias_case("apb_nomask", 1, 2, 2, 8, 8, 32, 16, mask_batch=None, seed=3, ref=attention_pair_bias_torch)
    attention_case("attn_small", 2, 5, 12, 2, 8, ref=a)
    attention_case("attn_bias_bcast", 2, 3, 9, 3, 16, bias_batch=1, scale=0.3, seed=1, ref=a)
    attention_case("attn_nobias_nomask", 1, 4, 17, 2, 32, with_bias=False, with_mask=False, seed=2, ref=a)
    attention_case("attn_full_mask_row", 1, 3, 20, 2, 8, full_mask_row=True, seed=3, ref=a)
    attention_case("attn_d32", 1, 3, 40, 2, 32, seed=4, ref=a)
    trimul_case("trimul_out_small", (1,), 10, 16, 8, "outgoing", ref=t)
    trimul_case("trimul_in_small", (1,), 10, 16, 8, "incoming", seed=1, ref=t)
    trimul_case("trimul_out_bias", (2,), 7, 32, 32, "outgoing", biases=True, seed=2, ref=t)
    trimul_case("trimul_in_bias_nomask", (2,), 9, 24, 16, "incoming", biases=True, with_mask=False, seed=3, ref=t)
    trimul_case("trimul_out_c64", (1,), 12, 64, 48, "outgoing", seed=4, ref=t)


if __name__ == "__main__":
    main()

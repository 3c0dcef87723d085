"""The pair stack (BASELINE config 4 at a reduced size) against the CPU oracle composition."""

import numpy as np
import pytest
import torch


def _oracle_weights(blocks):
    f64 = lambda t: t.double().numpy()  # noqa: E731
    return [{k: {m: f64(v) for m, v in getattr(b, k).items()} for k in ("trimul_out", "trimul_in", "attn_start", "attn_end")}
            for b in blocks]


@pytest.mark.gpu
@pytest.mark.parametrize("n,tail", [(64, 8), (128, 16)])
def test_two_blocks_against_oracle(n, tail):
    from geometric_nn_ops_b200 import pairstack
    from oracle import pairstack_oracle as po
    z, mask = pairstack.make_inputs(n, masked_tail=tail, seed=n)
    blocks = [pairstack.make_block_weights(s) for s in (0, 1)]
    got = pairstack.pair_stack(z.cuda(), mask.cuda(), [b.to("cuda") for b in blocks])
    want = po.pair_stack(z.double().numpy(), mask.double().numpy(), _oracle_weights(blocks))
    g = got.double().cpu().numpy()
    assert np.isfinite(g).all()
    rel = np.linalg.norm(g - want) / np.linalg.norm(want)
    assert rel < 1.5e-2, rel
    # the masked tail rows of the attention updates are uniform averages, not garbage: compare them on their own
    rel_tail = np.linalg.norm(g[:, -tail:] - want[:, -tail:]) / np.linalg.norm(want[:, -tail:])
    assert rel_tail < 1.5e-2, rel_tail


def test_flop_count_matches_the_stated_figures():
    from geometric_nn_ops_b200 import pairstack
    per_block = pairstack.stack_flops(1024, 1)
    assert abs(per_block - (2 * 481.0e9 + 2 * 549.8e9 + 208e9)) / per_block < 0.01


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("shape", [(1, 24, 40, 4), (2, 16, 16, 8), (1, 128, 128, 4)], ids=str)
def test_fused_projection_against_torch_fp32(shape, dtype):
    """LayerNorm + q/k/v/bias projection kernel against the same composition in fp32 torch on the rounded inputs."""
    from geometric_nn_ops_b200.triangle import attention_input_projection
    B, R, N, H = shape
    D = 128 // H
    g = torch.Generator().manual_seed(R + N)
    z = (torch.randn(B, R, N, 128, generator=g) * 2 + 0.5).to(dtype).cuda()
    w_qkv = (torch.randn(3 * H * D, 128, generator=g) * 128 ** -0.5).to(dtype).cuda()
    w_bias = (torch.randn(H, 128, generator=g) * 128 ** -0.5).to(dtype).cuda()
    ln_w = (1 + 0.1 * torch.randn(128, generator=g)).to(dtype).cuda()
    ln_b = (0.1 * torch.randn(128, generator=g)).to(dtype).cuda()
    for lw, lb in ((None, None), (ln_w, ln_b)):
        with torch.no_grad():
            q, k, v, bias = attention_input_projection(z, w_qkv, w_bias, H, lw, lb)
        assert q.shape == (B, R, N, H, D) and bias.shape == (B, H, R, N)
        zn = torch.nn.functional.layer_norm(z.float(), (128,), None if lw is None else lw.float(), None if lb is None else lb.float())
        zn = zn.to(dtype).float()                      # the kernel stores zn in the input dtype before the GEMM
        ref = (zn @ w_qkv.float().t()).view(B, R, N, 3, H, D)
        for got, want in ((q, ref[:, :, :, 0]), (k, ref[:, :, :, 1]), (v, ref[:, :, :, 2]),
                          (bias, (zn @ w_bias.float().t()).permute(0, 3, 1, 2))):
            rel = (got.float() - want).norm() / want.norm()
            assert rel < (6e-3 if dtype == torch.bfloat16 else 1e-3), rel
    with pytest.raises(RuntimeError, match="forward only"):
        attention_input_projection(z.requires_grad_(), w_qkv, w_bias, H)


def test_glue_on_cpu_with_the_ops_replaced_by_the_torch_restatement(monkeypatch):
    """The stack's own glue -- LayerNorm, projections, residual adds, and the ending-node attention on transposed
    *views* of the projections -- on the CPU in fp64, with the two CUDA ops swapped for the torch restatement of the
    reference, against the numpy composition: an index or transposition error in the glue shows up here without a GPU."""
    from geometric_nn_ops_b200 import pairstack
    from oracle import pairstack_oracle as po
    from oracle import torch_reference as tr

    monkeypatch.setattr(pairstack, "triangle_attention",
                        lambda q, k, v, bias, mask: tr.cpu_triangle_attention(q, k, v, bias, mask))
    monkeypatch.setattr(pairstack, "triangle_multiplicative_update",
                        lambda x, direction, mask, **w: tr.cpu_trimul(x, direction, mask, **w))
    n, tail = 24, 4
    z, mask = pairstack.make_inputs(n, masked_tail=tail, dtype=torch.float64, seed=3)
    blocks = [pairstack.make_block_weights(s, dtype=torch.float64) for s in (0, 1)]
    got = pairstack.pair_stack(z, mask, blocks).numpy()
    want = po.pair_stack(z.numpy(), mask.numpy(), _oracle_weights(blocks))
    assert np.isfinite(got).all()
    # the last `tail` rows of the ending-node problem are fully masked: uniform averages in both
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 1e-9, rel

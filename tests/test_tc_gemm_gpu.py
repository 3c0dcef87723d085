"""The tcgen05 batched GEMM against an fp64 matmul of the same (rounded) inputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [  # batch, M, N, K
    (1, 128, 128, 64), (1, 128, 256, 128), (3, 256, 512, 192), (2, 200, 136, 72), (4, 768, 768, 768),
    (1, 64, 40, 24),
]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True), (False, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=str)
@pytest.mark.parametrize("case", CASES, ids=str)
def test_bgemm(case, dtype, a_mn, b_mn):
    from geometric_nn_ops_b200.gemm import bgemm
    batch, M, N, K = case
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(batch, M, K, generator=g).to(dtype).cuda()
    b = torch.randn(batch, N, K, generator=g).to(dtype).cuda()
    want = torch.matmul(a.double(), b.double().transpose(1, 2))
    a_in = a.transpose(1, 2).contiguous() if a_mn else a
    b_in = b.transpose(1, 2).contiguous() if b_mn else b
    got32 = bgemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32, check=True)
    rel = ((got32.double() - want).norm() / want.norm()).item()
    assert rel < (1e-3 if dtype == torch.float32 else 1e-5), rel   # tf32 drops 13 mantissa bits; 16-bit products are exact
    got = bgemm(a_in, b_in, a_mn_major=a_mn, b_mn_major=b_mn, check=True)
    assert got.dtype == dtype
    assert torch.equal(got, got32.to(dtype))

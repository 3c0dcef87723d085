"""tri_permute_runs (the packing / unpacking copy of the row <-> channel exchanges) against torch's permute."""
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dims,run", [((2, 4, 1), 48 * 40), ((4, 2, 16), 24 * 40), ((2, 16, 4), 8), ((3, 5, 7), 1024 + 8)])
def test_permute_runs_matches_torch(dims, run):
    from geometric_nn_ops_b200.sharded import _permute_runs
    g = torch.Generator().manual_seed(sum(dims) + run)
    t = torch.randn(*dims, run, generator=g).to(torch.bfloat16).cuda()
    for perm in itertools.permutations(range(3)):
        got = _permute_runs(t, dims, perm, run)
        want = t.permute(*perm, 3).contiguous()
        assert got.shape == want.shape
        assert torch.equal(got, want), (dims, perm)


def test_permute_runs_rejects_misaligned_runs():
    from geometric_nn_ops_b200.sharded import _permute_runs
    t = torch.zeros(2, 2, 2, 4, dtype=torch.bfloat16, device="cuda")   # 8-byte runs
    with pytest.raises(RuntimeError, match="16"):
        _permute_runs(t, (2, 2, 2), (1, 0, 2), 4)

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


def test_scatter_runs_index_math_with_local_buffers():
    """tri_scatter_runs with every 'peer' buffer on this GPU: the rows->channels and channels->rows placements of
    two emulated ranks must reproduce what the all-to-all route computes."""
    import ctypes
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    world, L, cs, R, N = 2, 2, 4, 3, 8
    Ch = world * cs
    g = torch.Generator().manual_seed(3)
    full = torch.randn(L, Ch, world * R, N, generator=g).to(torch.bfloat16).cuda()      # all channels, all rows
    bufs = [torch.zeros(L, cs, world * R, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for me in range(world):   # rank `me` holds rows [me*R, (me+1)*R) of every channel
        mine = full[:, :, me * R:(me + 1) * R].contiguous()
        d = _lib.TriScatterDesc()
        d.dims[:] = (L, world, cs)
        d.dst_stride[:] = (cs * world, 0, world)
        d.dst_base_run = me
        d.run_bytes = R * N * 2
        d.peer_dim, d.n_peers = 1, world
        _lib.check(lib.tri_scatter_runs(ctypes.byref(d), ctypes.c_void_p(mine.data_ptr()), ptrs, stream), "scatter")
    torch.cuda.synchronize()
    for w in range(world):    # rank w must now hold its cs channels over all rows
        assert torch.equal(bufs[w], full[:, w * cs:(w + 1) * cs])
    # and back: channels -> rows
    outs = [torch.zeros(L, Ch, R, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    optrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in outs])
    for me in range(world):
        d = _lib.TriScatterDesc()
        d.dims[:] = (L, cs, world)
        d.dst_stride[:] = (world * cs, 1, 0)
        d.dst_base_run = me * cs
        d.run_bytes = R * N * 2
        d.peer_dim, d.n_peers = 2, world
        _lib.check(lib.tri_scatter_runs(ctypes.byref(d), ctypes.c_void_p(bufs[me].data_ptr()), optrs, stream), "scatter")
    torch.cuda.synchronize()
    for w in range(world):
        assert torch.equal(outs[w], full[:, :, w * R:(w + 1) * R])

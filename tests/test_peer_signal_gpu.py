"""Arrival flags of the peer-store exchange on one GPU: the copy kernel raises its flag, the wait kernel sees it, and a
wait for a flag that nobody raises runs out after its limit and reports which peer was missing (the GPU stays usable:
the wait is bounded by design, nothing here hangs or faults)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _signal(flags, state, rank, n_peers):
    from geometric_nn_ops_b200 import _lib
    ptrs = (ctypes.c_void_p * n_peers)(*[flags.data_ptr()] * n_peers)
    sig = _lib.TriPeerSignal()
    sig.flag_ptrs = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
    sig.state, sig.rank, sig.n_peers = state.data_ptr(), rank, n_peers
    return sig, ptrs   # keep the pointer array alive


def test_copy_raises_the_flag_and_the_wait_passes():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    sig, keep = _signal(flags, state, 0, 1)
    src = torch.arange(3 * 4 * 64, dtype=torch.float32, device="cuda").reshape(3, 1, 4, 64)
    dst = torch.zeros(4, 3, 64, dtype=torch.float32, device="cuda")          # dst[i2][i0] = src[i0][0][i2]
    d = _lib.TriScatterDesc()
    d.dims[:] = (3, 1, 4)
    d.dst_stride[:] = (1, 0, 3)
    d.dst_base_run, d.run_bytes, d.peer_dim, d.n_peers = 0, 64 * 4, 1, 1
    dptr = (ctypes.c_void_p * 1)(dst.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for epoch in (1, 2, 3):
        dst.zero_()
        _lib.check(lib.tri_scatter_runs_signal(ctypes.byref(d), ctypes.c_void_p(src.data_ptr()), dptr, ctypes.byref(sig),
                                               stream), "tri_scatter_runs_signal")
        _lib.check(lib.tri_peer_wait(ctypes.byref(sig), 0, stream), "tri_peer_wait")
        torch.cuda.synchronize()
        assert torch.equal(dst, src[:, 0].transpose(0, 1))
        assert flags[0].item() == epoch and state.tolist() == [epoch, epoch, 0, 0]


def test_a_wait_nobody_answers_runs_out_and_reports_the_peer():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    flags[0] = 1                                   # peer 0 has arrived, peer 1 never does
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    sig, keep = _signal(flags, state, 0, 2)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.tri_peer_wait(ctypes.byref(sig), 4_000_000, stream), "tri_peer_wait")   # ~2 ms of SM clocks
    torch.cuda.synchronize()
    assert state.tolist() == [0, 1, 0, 101]
    # the context is intact: the next kernel runs normally
    assert (torch.ones(8, device="cuda") * 2).sum().item() == 16.0


def test_bad_descriptors_are_refused():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    sig = _lib.TriPeerSignal()
    assert lib.tri_peer_wait(ctypes.byref(sig), 0, None) == -1
    assert lib.tri_scatter_runs_signal(None, None, None, None, None) == -1

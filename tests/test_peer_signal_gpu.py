"""Arrival flags of the peer-store exchange on one GPU: a barrier among "peers" that all map to this GPU passes and
advances its number, and a wait for a flag that nobody raises runs out after its limit and reports which peer was
missing (the GPU stays usable: the wait is bounded by design, nothing here hangs or faults)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _signal(flag_arrays, state, rank):
    from geometric_nn_ops_b200 import _lib
    n = len(flag_arrays)
    ptrs = (ctypes.c_void_p * n)(*[f.data_ptr() for f in flag_arrays])
    sig = _lib.TriPeerSignal()
    sig.flag_ptrs = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
    sig.state, sig.rank, sig.n_peers = state.data_ptr(), rank, n
    return sig, ptrs   # keep the pointer array alive


def test_a_barrier_with_itself_passes_and_counts():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    sig, keep = _signal([flags], state, 0)       # a world of one: this rank raises its own slot and waits for it
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for epoch in (1, 2, 3):
        _lib.check(lib.tri_peer_barrier(ctypes.byref(sig), 0, stream), "tri_peer_barrier")
        torch.cuda.synchronize()
        assert flags[0].item() == epoch and state.tolist() == [epoch, 0, 0, 0]


def test_a_wait_nobody_answers_runs_out_and_reports_the_peer():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    mine = torch.zeros(16, dtype=torch.int32, device="cuda")      # this rank's flags: slot 1 is never raised
    theirs = torch.zeros(16, dtype=torch.int32, device="cuda")    # stands for the silent peer's array
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    sig, keep = _signal([mine, theirs], state, 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.tri_peer_barrier(ctypes.byref(sig), 4_000_000, stream), "tri_peer_barrier")   # ~2 ms of SM clocks
    torch.cuda.synchronize()
    assert state.tolist() == [1, 0, 0, 101]                       # peer 1 was missing
    assert mine[0].item() == 1 and theirs[0].item() == 1          # this rank did raise its flag on both
    # the context is intact: the next kernel runs normally
    assert (torch.ones(8, device="cuda") * 2).sum().item() == 16.0


def test_bad_descriptors_are_refused():
    from geometric_nn_ops_b200 import _lib
    lib = _lib.load()
    sig = _lib.TriPeerSignal()
    assert lib.tri_peer_barrier(ctypes.byref(sig), 0, None) == -1

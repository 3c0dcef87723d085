"""Row-sharded (multi-GPU) forms of the two triangle ops: one process per GPU over NVLink.

The pair representation ``[B, N, N, C]`` is sharded over its first pair axis: rank ``r`` of ``P`` holds rows
``[r*N/P, (r+1)*N/P)``.  The reference is single-device; these wrappers are new.

* Triangle attention around the starting node attends along the second axis for a fixed row, so it is
  local; only the pair bias has to be whole on every rank and its gradient (a sum over rows) is
  all-reduced.  The ending-node variant is the same op on the transposed pair tensor:
  :func:`all_to_all_transpose` does that transpose with one all-to-all.
* The triangle multiplicative update is pixel-wise except for the contraction, and the contraction is
  independent per channel.  So the projected operands go from row shards to channel shards with one
  all-to-all, each rank contracts its ``C/P`` channels over the full ``N x N`` planes (either direction, it
  is only an operand-major flag), and the result returns to row shards with a second all-to-all.  Per
  rank that moves ``3/P`` of a pair-sized tensor per forward, against ``(P-1)/P`` for all-gathering ``b``.
  Weight gradients are partial sums per rank and are all-reduced.

The row <-> channel exchange is not an NCCL all-to-all: each rank writes every run straight into its final place in
the destination GPU's buffer (symmetric memory over NVLink), one pass over the data instead of pack + all-to-all +
unpack, and a one-block kernel with arrival flags and a bounded wait orders it (``tri_peer_barrier``).  The writes
are done by a copy kernel (``tri_scatter_runs``) or, on two GPUs, by strided two-dimensional copies on the copy
engines (``tri_scatter_runs_dma``: no SM is used, the step's other kernels keep the GPU; with more destinations the
copies of an exchange, which run one after the other, cost more latency than they free).
``TRI_B200_EXCHANGE=peer_kernel`` / ``peer_dma`` force one or the other, ``peer_allreduce`` uses the copy kernel and a
one-element all-reduce as the barrier,
``fused`` lets the gate-in GEMM's epilogue store a and b into the peers' buffers, ``nccl`` (or a CPU / gloo group)
selects the all-to-all route.
Kernels and copies only ever *write* to a peer; every load, and every tensor handed to NCCL, is in this GPU's memory.
"""

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib, _precision
from .gemm import bgemm
from .triangle._triattn import triangle_attention
from .triangle._trimul import _DTYPES, _aligned, is_outgoing


# Optional timing of the exchanges (bench.py turns it on for one eager step): name -> list of (start, end) events.
TIMERS = None


class _timed:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if TIMERS is not None:
            self.beg = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.beg.record()
        return self

    def __exit__(self, *exc):
        if TIMERS is not None:
            self.end.record()
            TIMERS.setdefault(self.name, []).append((self.beg, self.end))


def timing_summary():
    """{name: (calls, total_ms)} of the exchanges recorded since ``TIMERS`` was set to a dict."""
    torch.cuda.synchronize()
    return {k: (len(v), sum(b.elapsed_time(e) for b, e in v)) for k, v in (TIMERS or {}).items()}


def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


def shard_rows(n, rank, world):
    """Row range ``[i0, i1)`` of rank ``rank`` when ``n`` rows are split evenly over ``world`` ranks."""
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by the number of ranks {world}")
    r = n // world
    return rank * r, (rank + 1) * r


# ---------------------------------------------------------------------------------------------------
# exchanges (plain torch + one collective each; differentiable where a caller needs it)
# ---------------------------------------------------------------------------------------------------
def _permute_runs(t, dims, perm, run):
    """``t`` viewed as ``[*dims, run]`` -> a new contiguous tensor ``[dims[perm[0]], dims[perm[1]], dims[perm[2]], run]``.

    On CUDA this is one launch of the library's run-copy kernel (HBM-bound); torch's ``permute().contiguous()``
    reached a quarter of that on these shapes.  CPU tensors (the gloo tests) take the torch route.
    """
    out_dims = [dims[p] for p in perm]
    if not t.is_cuda:
        return t.reshape(*dims, run).permute(*perm, 3).contiguous()
    t = t.contiguous()
    out = torch.empty(*out_dims, run, dtype=t.dtype, device=t.device)
    lib = _lib.load()
    d = (ctypes.c_int64 * 3)(*dims)
    pm = (ctypes.c_int32 * 3)(*perm)
    stream = ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
    _lib.check(lib.tri_permute_runs(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.byref(d),
                                    ctypes.byref(pm), run * t.element_size(), stream), "tri_permute_runs")
    return out


# Peer-store exchange: with symmetric memory (every rank's receive buffer mapped into every other rank's address
# space) the all-to-all and both layout changes become ONE copy kernel per rank that stores each run straight into
# its place in the destination GPU's buffer over NVLink.  "Every rank has written" is ordered before "any rank reads"
# by arrival flags, not by a collective: a one-block kernel queued behind the copy kernel stores this rank's barrier
# number into a flag slot on every peer and then waits (bounded, about a second) until all peers' slots here have
# reached the same number.  No host round trip, nothing for NCCL to launch, and a captured graph replays as is.
# TRI_B200_EXCHANGE=peer_allreduce keeps the former barrier, a one-element all-reduce.
#
# Buffer reuse: a peer may overwrite a buffer only after this rank has finished reading it.  Each (call site, size)
# owns TWO buffers used alternately.  A peer's copy kernel of exchange k+2 (the next one into the same buffer) is
# queued behind its wait of exchange k+1, which completes only when this rank's copy kernel of k+1 has run, and that
# one is queued on this rank's stream behind whatever read exchange k.  So two calls in a row with the same tag
# are safe as long as the readers run on the stream the exchange was issued on.
_PEER = {}            # (tag, bytes, device, group, parity) -> _PeerBuffer
_PEER_TURN = {}       # (tag, bytes, device, group) -> which of the two buffers the next exchange uses
_PEER_STATE = {}      # (group, device) -> bool: every rank can take the peer-store route
_FLAG_BYTES = 256


class _PeerBuffer:
    """One symmetric allocation: the receive buffer followed by this rank's 16 arrival flags, plus the peers' views."""

    def __init__(self, nbytes, device, group):
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        data = (nbytes + 255) // 256 * 256
        self.buf = symm_mem.empty(data + _FLAG_BYTES, dtype=torch.uint8, device=device)
        self.buf[data:].zero_()
        hdl = symm_mem.rendezvous(self.buf, pg.group_name)
        world = hdl.world_size
        self.ptrs = (ctypes.c_void_p * world)(*[int(p) for p in hdl.buffer_ptrs])
        self.flag_ptrs = (ctypes.c_void_p * world)(*[int(p) + data for p in hdl.buffer_ptrs])
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        self.sig = _lib.TriPeerSignal()
        self.sig.flag_ptrs = ctypes.cast(self.flag_ptrs, ctypes.POINTER(ctypes.c_void_p))
        self.sig.state = self.state.data_ptr()
        self.sig.rank, self.sig.n_peers = dist.get_rank(group), world
        self.token = torch.zeros(1, dtype=torch.float32, device=device)    # for the all-reduce form of the barrier
        # nobody may raise a flag here before it has been zeroed
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


def peer_exchange_enabled(device, group=None):
    """True when the exchanges can use peer stores: CUDA, NCCL, symmetric memory; TRI_B200_EXCHANGE=nccl turns it off.

    The first call for a (group, device) tries a small symmetric allocation and lets the ranks agree on the outcome
    (a MIN all-reduce), so that either every rank takes the peer-store route or every rank takes the all-to-all.
    """
    key = (id(group), device.index)
    if key not in _PEER_STATE:
        ok = (os.environ.get("TRI_B200_EXCHANGE", "peer") in ("peer", "peer_kernel", "peer_dma", "peer_allreduce", "fused") and device.type == "cuda"
              and dist.get_backend(group) == "nccl")
        if ok:
            try:
                _peer_buffer("probe", 4096, device, group)
                good = 1.0
            except Exception as exc:   # no symmetric memory on this system: use the collective route
                print(f"[sharded] peer-store exchange unavailable ({exc!r}); using all-to-all", flush=True)
                good = 0.0
            flag = torch.tensor([good], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            ok = bool(flag.item() > 0.5)
        _PEER_STATE[key] = ok
    return _PEER_STATE[key]


def exchange_route(device, group=None):
    """Name of the route the row <-> channel exchanges take for this (group, device): for logs and benchmarks."""
    if not peer_exchange_enabled(device, group):
        return "nccl all_to_all"
    mode = os.environ.get("TRI_B200_EXCHANGE", "peer")
    world = _world(group)[0]
    moved = "copy-engine peer copies" if _use_copy_engines(world) else "peer stores"
    return {"peer": moved + " + arrival flags", "peer_kernel": moved + " + arrival flags",
            "peer_dma": moved + " + arrival flags", "peer_allreduce": "peer stores + all-reduce barrier",
            "fused": "gate-in epilogue peer stores + all-reduce barrier"}[mode]


def check_exchange_status():
    """Read the status word of every exchange buffer (synchronises) and raise if a barrier wait ever ran out: a peer
    that did not arrive within the limit means the data read after that barrier cannot be trusted."""
    torch.cuda.synchronize()
    for key, pb in _PEER.items():
        status = int(pb.state[3].item())
        if status != 0:
            raise RuntimeError(f"peer exchange {key[0]!r}: rank {status - 100} did not arrive within the wait limit")


def _peer_buffer(tag, nbytes, device, group):
    base = (tag, nbytes, device.index, id(group))
    turn = _PEER_TURN.get(base, 0)
    _PEER_TURN[base] = turn ^ 1
    key = base + (turn,)
    if key not in _PEER:
        _PEER[key] = _PeerBuffer(nbytes, device, group)
    return _PEER[key]


def _peer_barrier(pb, tag, group, stream):
    """Order "every rank's stores have landed" before this rank's readers (queued next on ``stream``)."""
    with _timed(tag + ".barrier"):
        if os.environ.get("TRI_B200_EXCHANGE", "peer") in ("peer", "peer_kernel", "peer_dma"):
            _lib.check(_lib.load().tri_peer_barrier(ctypes.byref(pb.sig), 0, stream), "tri_peer_barrier")
            if os.environ.get("TRI_B200_CHECK") == "1" and not torch.cuda.is_current_stream_capturing():
                status = int(pb.state[3].item())
                if status != 0:
                    raise RuntimeError(f"peer exchange {tag!r}: rank {status - 100} did not arrive within the wait limit")
        else:
            dist.all_reduce(pb.token, group=group)


def _use_copy_engines(world):
    """The default route's choice between the copy engines and the copy kernel.  The copies of one exchange run one
    after the other on the stream; with one remote destination that costs nothing and frees the SMs (2 GPUs: 4.75
    against 4.93 ms per bench step), with seven it lengthens every exchange (8 GPUs: 1.72 against 1.55 ms; spread over
    four streams, 2.09)."""
    mode = os.environ.get("TRI_B200_EXCHANGE", "peer")
    return mode == "peer_dma" or (mode == "peer" and world == 2)


def _peer_scatter(t, dims, dst_stride, base_run, peer_dim, run, out_shape, tag, group, persist):
    world, _ = _world(group)
    t = t.contiguous()
    nbytes = t.numel() * t.element_size()
    pb = _peer_buffer(tag, nbytes, t.device, group)
    d = _lib.TriScatterDesc()
    d.dims[:] = dims
    d.dst_stride[:] = dst_stride
    d.dst_base_run = base_run
    d.run_bytes = run * t.element_size()
    d.peer_dim = peer_dim
    d.n_peers = world
    stream = ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
    lib = _lib.load()
    with _timed(tag + ".peer_store"):
        rc = _lib.ERR_UNSUPPORTED
        if _use_copy_engines(world):                                  # strided copies on the copy engines: no SM used
            rc = lib.tri_scatter_runs_dma(ctypes.byref(d), ctypes.c_void_p(t.data_ptr()), pb.ptrs, stream)
            if rc not in (0, _lib.ERR_UNSUPPORTED):
                _lib.check(rc, "tri_scatter_runs_dma")
        if rc != 0:                                                   # the copy kernel
            _lib.check(lib.tri_scatter_runs(ctypes.byref(d), ctypes.c_void_p(t.data_ptr()), pb.ptrs, stream), "tri_scatter_runs")
    _peer_barrier(pb, tag, group, stream)
    # The buffer is rewritten two exchanges with this tag from now.  Results the caller keeps beyond that (tensors
    # saved for the backward) get a private copy.
    out = pb.buf.view(t.dtype)[: t.numel()].view(out_shape)
    return out.clone() if persist else out


def rows_to_channels(t, group=None, tag="rows_to_channels", persist=True):
    """``[L, Ch, R, N]`` (all channels, this rank's R rows) -> ``[L, Ch/P, P*R, N]`` (this rank's channels, all rows)."""
    world, me = _world(group)
    L, Ch, R, N = t.shape
    if Ch % world != 0:
        raise ValueError(f"{Ch} channels are not divisible by {world} ranks")
    cs = Ch // world
    if world > 1 and peer_exchange_enabled(t.device, group):
        # run (l, w, c) of the source -> GPU w, run ((l*cs + c)*world + me) of its [L, cs, world, R*N] buffer
        return _peer_scatter(t, (L, world, cs), (cs * world, 0, world), me, 1, R * N, (L, cs, world * R, N), tag, group, persist)
    with _timed("rows_to_channels.pack"):
        send = _permute_runs(t, (L, world, 1), (1, 0, 2), cs * R * N)       # [world, L, cs*R*N]
        recv = torch.empty_like(send)
    with _timed("rows_to_channels.all_to_all"):
        dist.all_to_all_single(recv, send, group=group)
    with _timed("rows_to_channels.unpack"):
        return _permute_runs(recv, (world, L, cs), (1, 2, 0), R * N).reshape(L, cs, world * R, N)


def channels_to_rows(t, group=None, tag="channels_to_rows", persist=True):
    """Inverse of :func:`rows_to_channels`: ``[L, Ch/P, N_rows, N]`` -> ``[L, Ch, N_rows/P, N]``."""
    world, me = _world(group)
    L, cs, rows, N = t.shape
    if rows % world != 0:
        raise ValueError(f"{rows} rows are not divisible by {world} ranks")
    R = rows // world
    if world > 1 and peer_exchange_enabled(t.device, group):
        # run (l, c, w) of the source -> GPU w, run ((l*world + me)*cs + c) of its [L, world, cs, R*N] buffer
        return _peer_scatter(t, (L, cs, world), (world * cs, 1, 0), me * cs, 2, R * N, (L, world * cs, R, N), tag, group, persist)
    with _timed("channels_to_rows.pack"):
        send = _permute_runs(t, (L, cs, world), (2, 0, 1), R * N)           # [world, L, cs, R*N]
        recv = torch.empty_like(send)
    with _timed("channels_to_rows.all_to_all"):
        dist.all_to_all_single(recv, send, group=group)
    with _timed("channels_to_rows.unpack"):
        return _permute_runs(recv, (world, L, 1), (1, 0, 2), cs * R * N).reshape(L, world * cs, R, N)


class _Transpose(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _transpose_impl(x, group)

    @staticmethod
    def backward(ctx, g):
        return _transpose_impl(g.contiguous(), ctx.group), None


def _transpose_impl(x, group):
    world, _ = _world(group)
    B, R, N = x.shape[0], x.shape[1], x.shape[2]
    tail = x.shape[3:]
    if N != R * world:
        raise ValueError(f"expected [B, N/P, N, ...] with N = {R * world}, got {tuple(x.shape)}")
    # chunk s of the column axis goes to rank s
    send = x.reshape(B, R, world, R, *tail).movedim(2, 0).contiguous()    # [P, B, R(i), R(j), ...]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[s] = x[i in shard s, j in my shard]  ->  out[j, i]
    return recv.movedim(0, 1).reshape(B, world * R, R, *tail).transpose(1, 2).contiguous()


def all_to_all_transpose(x, group=None):
    """Transpose the two pair axes of a row-sharded tensor ``[B, N/P, N, ...]``: the result is the shard
    ``[B, N/P, N, ...]`` of ``x^T``.  One all-to-all; differentiable (it is its own inverse)."""
    return _Transpose.apply(x, group)


# Gradients that are sums over ranks (the pair bias, every weight) each cost one small all-reduce; a training step that
# runs several sharded ops pays that latency several times.  Inside `deferred_grad_sync()` the ops hand back their
# rank-local sums and register the tensors; leaving the context (or `flush()`) adds them over ranks IN PLACE with one
# all-reduce per dtype.  Until then the registered gradients hold this rank's partial sums only.
_DEFERRED = []


class deferred_grad_sync:
    def __init__(self, group=None):
        self.group, self.items = group, []

    def __enter__(self):
        _DEFERRED.append(self)
        return self

    def __exit__(self, exc_type, exc, tb):
        _DEFERRED.remove(self)
        if exc_type is None:
            self.flush()
        return False

    def add(self, t):
        self.items.append(t)

    def flush(self):
        by_dtype = {}
        for t in self.items:
            by_dtype.setdefault(t.dtype, []).append(t)
        self.items = []
        for tensors in by_dtype.values():
            with _timed("grads.all_reduce"):
                if len(tensors) == 1 and tensors[0].is_contiguous():
                    dist.all_reduce(tensors[0], op=dist.ReduceOp.SUM, group=self.group)
                    continue
                flat = torch.cat([t.reshape(-1) for t in tensors])
                dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
                off = 0
                for t in tensors:
                    t.copy_(flat[off:off + t.numel()].view(t.shape))
                    off += t.numel()


def _sum_over_ranks(tensors, group, name):
    """All-reduce ``tensors`` now, or register them with the enclosing `deferred_grad_sync`."""
    if _DEFERRED:
        for t in tensors:
            _DEFERRED[-1].add(t)
        return
    with _timed(name):
        for t in tensors:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)


class _SumGradOverRanks(torch.autograd.Function):
    """Identity whose gradient is all-reduced: for tensors replicated on every rank (the pair bias)."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return t.view_as(t)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        _sum_over_ranks([g], ctx.group, "bias_grad.all_reduce")
        return g, None


def sharded_triangle_attention(q, k, v, bias=None, mask=None, scale=None, group=None):
    """Triangle attention on this rank's rows.  ``q, k, v``: ``[B, N/P, N, H, D]``; ``bias``: the whole
    ``[B, 1, H, N, N]`` on every rank (its gradient is summed over ranks); ``mask``: this rank's rows."""
    if bias is not None and bias.requires_grad:
        bias = _SumGradOverRanks.apply(bias, group)
    return triangle_attention(q, k, v, bias, mask, scale)


# ---------------------------------------------------------------------------------------------------
# triangle multiplicative update
# ---------------------------------------------------------------------------------------------------
def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _phase(lib, desc, phase, bufs, device):
    ws_bytes = lib.tri_mul_shard_ws_bytes(ctypes.byref(desc), phase)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    with torch.cuda.device(device):
        _lib.check(lib.tri_mul_shard_phase(ctypes.byref(desc), phase, ctypes.byref(bufs), _ptr(ws), ws_bytes, stream),
                   "tri_mul_shard_phase")
        _lib.check_device_status(ws, stream)


class _ShardedTriMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, outgoing, eps, group, *weights):
        lib = _lib.load()
        if not x.is_cuda:
            raise RuntimeError("sharded trimul needs CUDA tensors: there is no CPU implementation")
        named = dict(zip(_lib.WEIGHT_NAMES, weights))
        B, R, N, C = x.shape
        xc = _aligned(x)
        mc = None if mask is None else _aligned(mask.to(x.dtype).broadcast_to(x.shape[:-1]))
        wc = {n: (None if t is None else _aligned(t.detach().to(x.dtype))) for n, t in named.items()}
        Ch = wc["p_in_weight"].shape[0] // 2
        d = _lib.TriMulShardDesc()
        d.B, d.rows, d.N, d.C, d.Ch = B, R, N, C, Ch
        d.dtype = _DTYPES[x.dtype]
        precision = _precision.matmul_precision(fp32_operands=x.dtype == torch.float32)
        d.precision = _lib.PREC_TF32 if precision == _precision.TF32 else _lib.PREC_IEEE
        d.eps = eps
        nbytes = lib.tri_mul_shard_saved_bytes(ctypes.byref(d))
        if nbytes == 0:
            raise RuntimeError("sharded trimul: " + lib.tri_last_error().decode())
        saved = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        w = _lib.TriMulWeights()
        for n, t in wc.items():
            setattr(w, _lib.abi_field(n), None if t is None else t.data_ptr())

        ab = torch.empty(2, B, Ch, R, N, dtype=x.dtype, device=x.device)
        bufs = _lib.TriMulShardBufs()
        bufs.x, bufs.mask, bufs.w, bufs.saved = xc.data_ptr(), None if mc is None else mc.data_ptr(), ctypes.pointer(w), saved.data_ptr()
        # the prepared weights travel from phase to phase (and to the backward) instead of being rebuilt in each
        prep = torch.empty(lib.tri_mul_shard_prep_bytes(ctypes.byref(d)), dtype=torch.uint8, device=x.device)
        bufs.prep, bufs.prep_ready = prep.data_ptr(), 0
        world, me = _world(group)
        # one set of exchange buffers per direction: an outgoing and an incoming update may run side by side on two streams
        tag = "out." if outgoing else "in."
        if world > 1 and peer_exchange_enabled(x.device, group) and os.environ.get("TRI_B200_EXCHANGE") == "fused":
            # compute and exchange in one kernel: the gate-in epilogue stores a and b straight into the channel
            # owners' buffers; the one-element all-reduce orders "all ranks have stored" before "anyone reads".
            # Opt-in: at 2 GPUs it measured 6.1 ms per step against 5.95 ms for GEMM + copy kernel (32-byte
            # remote stores from the epilogue use NVLink less well than the copy kernel's long runs).
            pb = _peer_buffer(tag + "fwd.ab", 2 * B * Ch * R * N * xc.element_size(), x.device, group)
            bufs.peer_ab = ctypes.cast(pb.ptrs, ctypes.POINTER(ctypes.c_void_p))
            bufs.peer_world, bufs.peer_rank = world, me
            with _timed(tag + "fwd.ab.gemm_with_peer_store"):
                _phase(lib, d, _lib.PHASE_PROJECT, bufs, x.device)
            with _timed(tag + "fwd.ab.barrier"):
                dist.all_reduce(pb.token, group=group)
            bufs.peer_ab, bufs.peer_world = None, 0
            bufs.prep_ready = 1
            ab_ch = pb.buf.view(xc.dtype)[: 2 * B * Ch * R * N].view(2 * B, Ch // world, N, N).clone()   # saved for the backward
        else:
            bufs.a_cm, bufs.b_cm = ab[0].data_ptr(), ab[1].data_ptr()
            _phase(lib, d, _lib.PHASE_PROJECT, bufs, x.device)
            bufs.prep_ready = 1
            ab_ch = rows_to_channels(ab.reshape(2 * B, Ch, R, N), group, tag=tag + "fwd.ab")      # [2B, Cs, N, N]
        cs = ab_ch.shape[1]
        a_ch = ab_ch[:B].reshape(B * cs, N, N)
        b_ch = ab_ch[B:].reshape(B * cs, N, N)
        inc = not outgoing
        t_ch = bgemm(a_ch, b_ch, a_mn_major=inc, b_mn_major=inc)              # [B*Cs, N, N]
        t_loc = channels_to_rows(t_ch.reshape(B, cs, N, N), group, tag=tag + "fwd.t")            # [B, Ch, R, N]
        out = torch.empty_like(xc)
        bufs.t_cm, bufs.out = t_loc.data_ptr(), out.data_ptr()
        _phase(lib, d, _lib.PHASE_OUTPUT, bufs, x.device)

        ctx.save_for_backward(xc, mc, saved, a_ch, b_ch, t_loc, prep, *[t for t in wc.values() if t is not None])
        ctx.present = [t is not None for t in wc.values()]
        ctx.desc, ctx.group, ctx.outgoing = d, group, outgoing
        ctx.weight_dtypes = [None if t is None else t.dtype for t in weights]
        return out

    @staticmethod
    def backward(ctx, d_out):
        lib = _lib.load()
        xc, mc, saved, a_ch, b_ch, t_loc, prep, *present_w = ctx.saved_tensors
        it = iter(present_w)
        wc = {n: (next(it) if has else None) for n, has in zip(_lib.WEIGHT_NAMES, ctx.present)}
        d, group = ctx.desc, ctx.group
        B, R, N, Ch = d.B, d.rows, d.N, d.Ch
        dev = xc.device
        w = _lib.TriMulWeights()
        g = _lib.TriMulWeightGrads()
        names = [n for n, t in wc.items() if t is not None]
        sizes = [wc[n].numel() for n in names]
        flat = torch.zeros(sum(sizes), dtype=torch.float32, device=dev)        # one buffer -> one all-reduce
        grads, off = {}, 0
        for n, sz in zip(names, sizes):
            grads[n] = flat[off:off + sz].view(wc[n].shape)
            off += sz
        for n, t in wc.items():
            setattr(w, _lib.abi_field(n), None if t is None else t.data_ptr())
            if t is not None:
                setattr(g, _lib.abi_field(n), grads[n].data_ptr())
        dc = _aligned(d_out.to(xc.dtype))
        dt_loc = torch.empty_like(t_loc)
        bufs = _lib.TriMulShardBufs()
        bufs.x, bufs.mask, bufs.w, bufs.saved = xc.data_ptr(), None if mc is None else mc.data_ptr(), ctypes.pointer(w), saved.data_ptr()
        bufs.g = ctypes.pointer(g)
        bufs.prep, bufs.prep_ready = prep.data_ptr(), 1
        bufs.d_out, bufs.t_cm, bufs.dt_cm = dc.data_ptr(), t_loc.data_ptr(), dt_loc.data_ptr()
        _phase(lib, d, _lib.PHASE_OUTPUT_BWD, bufs, dev)
        tag = "out." if ctx.outgoing else "in."
        dt_ch = rows_to_channels(dt_loc, group, tag=tag + "bwd.dt", persist=False)
        cs = dt_ch.shape[1]
        dt_ch = dt_ch.reshape(B * cs, N, N)
        if ctx.outgoing:   # da[i,k] = sum_j dt[i,j] b[j,k];  db[j,k] = sum_i dt[i,j] a[i,k]
            da = bgemm(dt_ch, b_ch, a_mn_major=False, b_mn_major=True)
            db = bgemm(dt_ch, a_ch, a_mn_major=True, b_mn_major=True)
        else:              # da[k,i] = sum_j b[k,j] dt[i,j];  db[k,j] = sum_i a[k,i] dt[i,j]
            da = bgemm(b_ch, dt_ch, a_mn_major=False, b_mn_major=False)
            db = bgemm(a_ch, dt_ch, a_mn_major=False, b_mn_major=True)
        dab = channels_to_rows(torch.stack([da.reshape(B, cs, N, N), db.reshape(B, cs, N, N)]).reshape(2 * B, cs, N, N),
                               group, tag=tag + "bwd.dab", persist=False).reshape(2, B, Ch, R, N)
        dx = torch.empty_like(xc)
        bufs.a_cm, bufs.b_cm, bufs.dx = dab[0].data_ptr(), dab[1].data_ptr(), dx.data_ptr()
        _phase(lib, d, _lib.PHASE_PROJECT_BWD, bufs, dev)
        out = [dx if ctx.needs_input_grad[0] else None, None, None, None, None]
        if _DEFERRED:
            # the caller sums over ranks later, in one call for the whole step: hand back this rank's partial sums in
            # the weights' dtype (one cast of the flat buffer) and register them
            lows = {}
            for dt in {d_ for d_ in ctx.weight_dtypes if d_ is not None}:
                lows[dt] = flat.to(dt)
                _DEFERRED[-1].add(lows[dt])
            off = 0
            views = {}
            for n, sz in zip(names, sizes):
                views[n] = off
                off += sz
            for i, (n, dt) in enumerate(zip(_lib.WEIGHT_NAMES, ctx.weight_dtypes)):
                if n in grads and ctx.needs_input_grad[5 + i]:
                    out.append(lows[dt][views[n]:views[n] + wc[n].numel()].view(wc[n].shape))
                else:
                    out.append(None)
            return tuple(out)
        with _timed("weight_grads.all_reduce"):
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        for i, (n, dt) in enumerate(zip(_lib.WEIGHT_NAMES, ctx.weight_dtypes)):
            out.append(grads[n].to(dt) if n in grads and ctx.needs_input_grad[5 + i] else None)
        return tuple(out)


def sharded_triangle_multiplicative_update(x, direction="outgoing", mask=None, *, eps=1e-5, group=None,
                                           norm_in_weight=None, norm_in_bias=None, p_in_weight=None, p_in_bias=None,
                                           g_in_weight=None, g_in_bias=None, norm_out_weight=None,
                                           norm_out_bias=None, p_out_weight=None, p_out_bias=None,
                                           g_out_weight=None, g_out_bias=None):
    """Triangle multiplicative update on a row shard.  ``x``: ``[B, N/P, N, C]`` (this rank's rows of the pair
    tensor), ``mask``: ``[B, N/P, N]``; weights replicated.  Returns this rank's rows of the result; weight
    gradients come back already summed over ranks.  Needs C = C_hidden = 128 (the tensor-core kernels)."""
    outgoing = is_outgoing(direction)
    world, _ = _world(group)
    if x.dim() != 4 or x.shape[2] != x.shape[1] * world:
        raise ValueError(f"x must be [B, N/P, N, C] with P = {world}, got {tuple(x.shape)}")
    return _ShardedTriMul.apply(x, mask, outgoing, float(eps), group, norm_in_weight, norm_in_bias, p_in_weight,
                                p_in_bias, g_in_weight, g_in_bias, norm_out_weight, norm_out_bias, p_out_weight,
                                p_out_bias, g_out_weight, g_out_bias)


# ---------------------------------------------------------------------------------------------------
# benchmark step (used by bench.py --gpus N)
# ---------------------------------------------------------------------------------------------------
_SIDE_STREAMS = {}


def make_bench_step(n, rank, world, host_inputs):
    """One forward+backward of the three ops on this rank's row shard of the N-sized problem.

    The three ops of the step are independent of one another, so each runs on its own stream: the attention needs no
    exchange and its kernels fill the gaps the two multiplicative updates' exchanges leave, and one update's copy
    kernels run beside the other's GEMMs (TRI_B200_OVERLAP=0 puts everything back on one stream).  Every gradient
    that is a sum over ranks (pair bias, weights) is added in ONE all-reduce at the end of the step.
    """
    i0, i1 = shard_rows(n, rank, world)
    t, w = host_inputs(n, 0, torch)                  # same seed everywhere: weights and bias are replicated
    for name in ("q", "k", "v", "d_o", "key_mask", "x", "d_out", "pair_mask"):
        t[name] = t[name][:, i0:i1].contiguous()
    overlap = os.environ.get("TRI_B200_OVERLAP", "1") == "1"

    def step(td, wd):
        main = torch.cuda.current_stream()
        if overlap:
            streams = _SIDE_STREAMS.setdefault(main.device.index, [torch.cuda.Stream() for _ in range(3)])
        else:
            streams = [main, main, main]
        res = [None, None, None]

        def attention():
            q, k, v, bias = (td[m].detach().requires_grad_() for m in ("q", "k", "v", "bias"))
            o = sharded_triangle_attention(q, k, v, bias, td["key_mask"], q.shape[-1] ** -0.5)
            return [o, *torch.autograd.grad(o, [q, k, v, bias], grad_outputs=td["d_o"])]

        def update(direction):
            x = td["x"].detach().requires_grad_()
            wl = {m: p.detach().requires_grad_() for m, p in wd.items()}
            out = sharded_triangle_multiplicative_update(x, direction, td["pair_mask"], **wl)
            return [out, *torch.autograd.grad(out, [x, *wl.values()], grad_outputs=td["d_out"])]

        with deferred_grad_sync():
            for i, (st, fn) in enumerate(zip(streams, (attention, lambda: update("outgoing"), lambda: update("incoming")))):
                st.wait_stream(main)
                with torch.cuda.stream(st):
                    res[i] = fn()
            for st in streams:
                main.wait_stream(st)
            out = res[0] + res[1] + res[2]
            if overlap:
                for r_ in out:
                    r_.record_stream(main)      # allocated on a side stream, used (summed, copied out) on this one
        return out

    return step, t, w

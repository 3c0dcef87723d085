"""Row-sharded ops on 2+ GPUs (NCCL) against the single-GPU ops on the same inputs."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import util

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()


def _worker(rank, world, port, ret, exchange):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TRI_B200_CHECK="1", TRI_B200_EXCHANGE=exchange,
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    verdict = "ok"
    try:
        # Phase 1: everything that contains a collective, in the same order on every rank and with no assertion in
        # between, so that a wrong value on one rank can never make it leave the sequence while its peer waits
        # inside a collective.  Phase 2 compares locally.  Phase 3 agrees on the outcome before the group goes down.
        results = _run_collectives(rank, world)
        torch.cuda.synchronize()
        problems = _compare(results)
        if problems:
            verdict = "; ".join(problems)
    except Exception as exc:   # an exception in phase 1 (a failed launch) still reaches the agreement below
        import traceback
        verdict = traceback.format_exc() + repr(exc)
    try:
        flag = torch.tensor([1.0 if verdict == "ok" else 0.0], device=f"cuda:{rank}")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() < 0.5 and verdict == "ok":
            verdict = "ok here, a peer failed"
    except Exception as exc:
        verdict += f" (agreement failed: {exc!r})"
    ret[rank] = verdict
    dist.destroy_process_group()


def _run_collectives(rank, world):
    from geometric_nn_ops_b200 import sharded
    from geometric_nn_ops_b200.triangle import triangle_attention, trimul_b200

    dev = f"cuda:{rank}"
    N = 32 * world
    i0, i1 = sharded.shard_rows(N, rank, world)
    res = []   # (name, sharded result, single-GPU result, bound or None for exact equality)
    for direction in ("outgoing", "incoming"):
        x, mask, w, d_out = util.trimul_inputs(1, N, 128, 128, torch.bfloat16, seed=3, biases=True, device=dev)
        out, grads = util.trimul_fwd_bwd(trimul_b200, x, mask, w, direction, d_out)
        fn = lambda xx, dd, mm, **ww: sharded.sharded_triangle_multiplicative_update(xx, dd, mm, **ww)  # noqa: E731
        out_s, grads_s = util.trimul_fwd_bwd(fn, x[:, i0:i1].contiguous(), mask[:, i0:i1].contiguous(), w, direction,
                                             d_out[:, i0:i1].contiguous())
        res.append((direction + " out", out_s, out[:, i0:i1], 1e-3))
        res.append((direction + " dx", grads_s["x"], grads["x"][:, i0:i1], 2e-2))
        for name in w:
            res.append((direction + " d" + name, grads_s[name], grads[name], 3e-2))

    t, key_mask, d_o = util.attn_inputs(1, N, N, 4, 32, torch.bfloat16, seed=4, device=dev)
    out, grads = util.attn_fwd_bwd(triangle_attention, t, key_mask, None, d_o)
    loc = {k: (v[:, i0:i1].contiguous() if k != "bias" else v) for k, v in t.items()}
    out_s, grads_s = util.attn_fwd_bwd(sharded.sharded_triangle_attention, loc, key_mask[:, i0:i1].contiguous(), None,
                                       d_o[:, i0:i1].contiguous())
    res.append(("attention out", out_s, out[:, i0:i1], None))
    for name in ("q", "k", "v"):
        res.append(("attention d" + name, grads_s[name], grads[name][:, i0:i1], None))
    res.append(("attention dbias", grads_s["bias"], grads["bias"], 2e-2))   # summed over ranks in a different order

    pair = torch.randn(1, N, N, 16, generator=torch.Generator().manual_seed(5)).to(dev)
    res.append(("transpose", sharded.all_to_all_transpose(pair[:, i0:i1].contiguous()), pair.transpose(1, 2)[:, i0:i1], None))
    return res


def _compare(results):
    problems = []
    for name, got, want, bound in results:
        if bound is None:
            if not torch.equal(got, want):
                problems.append(f"{name}: not bit-identical (rel {_rel(got, want):.3e})")
        elif not _rel(got, want) < bound:
            problems.append(f"{name}: rel {_rel(got, want):.3e} >= {bound}")
    return problems


# the four exchange routes: strided peer copies on the copy engines (default), peer stores from a copy kernel, NCCL
# all-to-all, and the gate-in GEMM's epilogue storing into the peers' buffers
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("exchange", ["peer", "peer_kernel", "nccl", "fused"])
def test_sharded_matches_single_gpu(exchange):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:          # never leave a child behind: pytest would block on it at exit
        p.terminate()
    for p in stuck:
        p.join(30)
        if p.is_alive():
            p.kill()
            p.join(10)
    assert not stuck, f"{len(stuck)} rank(s) did not finish within the limit and were terminated"
    assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)

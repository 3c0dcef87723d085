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
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TRI_B200_CHECK="1", TRI_B200_EXCHANGE=exchange)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        _check(rank, world)
        ret[rank] = "ok"
    except Exception as exc:
        import traceback
        ret[rank] = traceback.format_exc() + repr(exc)
    finally:
        dist.destroy_process_group()


def _check(rank, world):
    from geometric_nn_ops_b200 import sharded
    from geometric_nn_ops_b200.triangle import triangle_attention, trimul_b200

    dev = f"cuda:{rank}"
    N = 32 * world
    i0, i1 = sharded.shard_rows(N, rank, world)
    for direction in ("outgoing", "incoming"):
        x, mask, w, d_out = util.trimul_inputs(1, N, 128, 128, torch.bfloat16, seed=3, biases=True, device=dev)
        out, grads = util.trimul_fwd_bwd(trimul_b200, x, mask, w, direction, d_out)
        fn = lambda xx, dd, mm, **ww: sharded.sharded_triangle_multiplicative_update(xx, dd, mm, **ww)  # noqa: E731
        out_s, grads_s = util.trimul_fwd_bwd(fn, x[:, i0:i1].contiguous(), mask[:, i0:i1].contiguous(), w, direction,
                                             d_out[:, i0:i1].contiguous())
        assert _rel(out_s, out[:, i0:i1]) < 1e-3, (direction, "out", _rel(out_s, out[:, i0:i1]))
        assert _rel(grads_s["x"], grads["x"][:, i0:i1]) < 2e-2, (direction, "dx")
        for name in w:
            assert _rel(grads_s[name], grads[name]) < 3e-2, (direction, name, _rel(grads_s[name], grads[name]))

    t, key_mask, d_o = util.attn_inputs(1, N, N, 4, 32, torch.bfloat16, seed=4, device=dev)
    out, grads = util.attn_fwd_bwd(triangle_attention, t, key_mask, None, d_o)
    loc = {k: (v[:, i0:i1].contiguous() if k != "bias" else v) for k, v in t.items()}
    out_s, grads_s = util.attn_fwd_bwd(sharded.sharded_triangle_attention, loc, key_mask[:, i0:i1].contiguous(), None,
                                       d_o[:, i0:i1].contiguous())
    assert torch.equal(out_s, out[:, i0:i1])
    for name in ("q", "k", "v"):
        assert torch.equal(grads_s[name], grads[name][:, i0:i1]), name
    assert _rel(grads_s["bias"], grads["bias"]) < 2e-2          # summed over ranks in a different order

    pair = torch.randn(1, N, N, 16, generator=torch.Generator().manual_seed(5)).to(dev)
    assert torch.equal(sharded.all_to_all_transpose(pair[:, i0:i1].contiguous()), pair.transpose(1, 2)[:, i0:i1])


# the three exchange routes: peer stores from a copy kernel (default), NCCL all-to-all, and the gate-in GEMM's
# epilogue storing into the peers' buffers
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("exchange", ["peer", "nccl", "fused"])
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
        assert not p.is_alive(), "rank did not finish"
    assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)

"""Host logic of the row-sharded wrappers on two gloo ranks (CPU): the exchanges and the row partition."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        globals()[fn_name](rank, world)
        ret[rank] = "ok"
    except Exception as exc:  # report instead of hanging the other rank
        ret[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


def _run(fn_name, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive(), "rank did not finish"
    assert dict(ret) == {r: "ok" for r in range(world)}, dict(ret)


def _full(shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def check_channel_exchange(rank, world):
    from geometric_nn_ops_b200 import sharded
    L, Ch, N = 3, 8, 6
    R, cs = N // world, Ch // world
    full = _full((L, Ch, N, N))                       # the same on every rank
    i0, i1 = sharded.shard_rows(N, rank, world)
    mine = full[:, :, i0:i1].contiguous()             # all channels, my rows
    got = sharded.rows_to_channels(mine)
    assert torch.equal(got, full[:, rank * cs:(rank + 1) * cs])   # my channels, all rows
    back = sharded.channels_to_rows(got)
    assert torch.equal(back, mine)


def check_transpose(rank, world):
    from geometric_nn_ops_b200 import sharded
    B, N, C = 2, 8, 5
    full = _full((B, N, N, C), seed=1)
    i0, i1 = sharded.shard_rows(N, rank, world)
    x = full[:, i0:i1].clone().requires_grad_()
    y = sharded.all_to_all_transpose(x)
    assert torch.equal(y, full.transpose(1, 2)[:, i0:i1])
    # gradient: the transpose of the upstream gradient's shard
    gfull = _full((B, N, N, C), seed=2)
    y.backward(gfull[:, i0:i1])
    assert torch.equal(x.grad, gfull.transpose(1, 2)[:, i0:i1])
    assert torch.equal(sharded.all_to_all_transpose(sharded.all_to_all_transpose(x.detach())), x.detach())


def check_replicated_grad(rank, world):
    from geometric_nn_ops_b200 import sharded
    bias = torch.ones(4, requires_grad=True)
    out = sharded._SumGradOverRanks.apply(bias, None) * float(rank + 1)
    out.sum().backward()
    assert torch.equal(bias.grad, torch.full((4,), float(sum(range(1, world + 1)))))


def check_deferred_grad_sync(rank, world):
    """Inside the context the gradients are this rank's partial sums; leaving it adds them over ranks in place, one
    all-reduce per dtype, through the tensors autograd handed back."""
    from geometric_nn_ops_b200 import sharded
    a = torch.ones(4, requires_grad=True)
    b = torch.ones(2, 3, requires_grad=True)
    c = torch.ones(5, dtype=torch.float64, requires_grad=True)
    with sharded.deferred_grad_sync() as sync:
        outs = [sharded._SumGradOverRanks.apply(t, None) * float(rank + 1) for t in (a, b, c)]
        ga, gb, gc = torch.autograd.grad([o.sum() for o in outs], [a, b, c])
        assert torch.equal(ga, torch.full((4,), float(rank + 1)))          # not summed yet
        assert len(sync.items) == 3
    total = float(sum(range(1, world + 1)))
    assert torch.equal(ga, torch.full((4,), total)) and torch.equal(gb, torch.full((2, 3), total))
    assert torch.equal(gc, torch.full((5,), total, dtype=torch.float64))
    # outside a context the sum happens at once
    (g2,) = torch.autograd.grad((sharded._SumGradOverRanks.apply(a, None) * float(rank + 1)).sum(), [a])
    assert torch.equal(g2, torch.full((4,), total))


def check_pair_block_glue(rank, world):
    """The sharded branch of the pair stack's block (bias all-gather, the two all-to-all transposes around the
    ending-node attention) against the single-process branch, in fp64, with the two CUDA ops replaced by the torch
    restatement of the reference (the sharded multiplicative update by gather + whole-tensor op + slice)."""
    from geometric_nn_ops_b200 import pairstack, sharded
    from oracle import torch_reference as tr

    n = 8 * world
    z, mask = pairstack.make_inputs(n, masked_tail=3, dtype=torch.float64, seed=5)
    w = pairstack.make_block_weights(7, dtype=torch.float64)
    i0, i1 = sharded.shard_rows(n, rank, world)

    def gathered_trimul(x, direction, m, group=None, **weights):
        xs = [torch.empty_like(x) for _ in range(world)]
        ms = [torch.empty_like(m) for _ in range(world)]
        dist.all_gather(xs, x.contiguous(), group=group)
        dist.all_gather(ms, m.contiguous(), group=group)
        return tr.cpu_trimul(torch.cat(xs, 1), direction, torch.cat(ms, 1), **weights)[:, i0:i1]

    pairstack.triangle_attention = lambda q, k, v, bias, m: tr.cpu_triangle_attention(q, k, v, bias, m)
    pairstack.triangle_multiplicative_update = lambda x, direction, m, **weights: tr.cpu_trimul(x, direction, m, **weights)
    sharded.sharded_triangle_multiplicative_update = gathered_trimul
    whole = pairstack.pair_block(z, mask, w)
    mine = pairstack.pair_block(z[:, i0:i1].contiguous(), mask[:, i0:i1].contiguous(), w, group=dist.group.WORLD)
    err = float((mine - whole[:, i0:i1]).norm() / whole[:, i0:i1].norm())
    assert err < 1e-12, err


@pytest.mark.parametrize("fn", ["check_channel_exchange", "check_transpose", "check_replicated_grad",
                                "check_deferred_grad_sync", "check_pair_block_glue"])
def test_two_ranks(fn):
    _run(fn)


def test_shard_rows_rejects_uneven_split():
    from geometric_nn_ops_b200 import sharded
    assert sharded.shard_rows(768, 3, 8) == (288, 384)
    with pytest.raises(ValueError, match="not divisible"):
        sharded.shard_rows(10, 0, 4)


def test_default_route_uses_copy_engines_on_two_gpus_only(monkeypatch):
    """The default peer route moves the slabs with copy-engine copies on 2 GPUs and with the copy kernel beyond (the
    measured crossover); the two forcing values override that."""
    from geometric_nn_ops_b200 import sharded

    monkeypatch.delenv("TRI_B200_EXCHANGE", raising=False)
    assert sharded._use_copy_engines(2)
    assert not sharded._use_copy_engines(4) and not sharded._use_copy_engines(8)
    monkeypatch.setenv("TRI_B200_EXCHANGE", "peer_kernel")
    assert not sharded._use_copy_engines(2)
    monkeypatch.setenv("TRI_B200_EXCHANGE", "peer_dma")
    assert sharded._use_copy_engines(2) and sharded._use_copy_engines(8)
    monkeypatch.setenv("TRI_B200_EXCHANGE", "nccl")
    assert not sharded._use_copy_engines(2)

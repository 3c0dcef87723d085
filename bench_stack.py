"""``bench.py --workload stack``: the 4-block pair stack, bf16 inference, on 1..8 GPUs (rows sharded).

BASELINE configuration: B=1, N=1024, c_z=128, four blocks with weights from seeds 0..3, z ~ N(0, 1), the last 64
residues masked out.  Before timing, the same code runs a reduced size (N=128 per 8 ranks or fewer) and is
checked against the CPU oracle composition (oracle/pairstack_oracle.py); a mismatch ends the run non-zero.
Prints one JSON line with the whole-stack time, TFLOP/s over the algorithmic forward FLOPs, and the split of
the time between the ops.
"""

import json
import os
import sys

import torch

from geometric_nn_ops_b200 import _lib, pairstack, sharded

N_STACK, N_BLOCKS, N_CHECK = 1024, 4, 128


def _shard(t, rank, world):
    i0, i1 = sharded.shard_rows(t.shape[1], rank, world)
    return t[:, i0:i1].contiguous()


def _parity(rank, world, group, dist):
    """Reduced-size run against the oracle (computed on every rank: a second of numpy at N=128)."""
    import numpy as np

    from oracle import pairstack_oracle as po
    n = N_CHECK
    z, mask = pairstack.make_inputs(n, masked_tail=8, seed=7)
    blocks = [pairstack.make_block_weights(s) for s in range(2)]
    got = pairstack.pair_stack(_shard(z, rank, world).cuda(), _shard(mask, rank, world).cuda(),
                               [b.to("cuda") for b in blocks], group)
    f64 = lambda t: t.double().numpy()  # noqa: E731
    ref = po.pair_stack(f64(z), f64(mask), [{k: {m: f64(v) for m, v in getattr(b, k).items()} for k in
                                             ("trimul_out", "trimul_in", "attn_start", "attn_end")} for b in blocks])
    i0, i1 = sharded.shard_rows(n, rank, world)
    a, b = got.double().cpu().numpy(), ref[:, i0:i1]
    err = torch.tensor([float(np.linalg.norm(a - b) / np.linalg.norm(b))], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
    # two blocks of bf16 ops with bf16 residual adds against fp64: the per-op bf16 bound of the reference's tables
    return {"against": f"cpu oracle composition, N={n}, 2 blocks", "metric": "rel-Frobenius, max over ranks",
            "max_rel_fro": {"z": err.item()}, "bound": 1.5e-2, "ok": err.item() <= 1.5e-2}


def main(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    n = args.n_res if args.n_res != 768 else N_STACK
    base = {"metric": f"pair stack ({N_BLOCKS} blocks) forward TFLOP/s, N={n}", "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{N_BLOCKS}-block pair stack (trimul out, trimul in, tri-attn start, tri-attn end; "
                                   f"residual adds), B=1, N={n}, c_z=128, H=4, D=32, bf16 inference",
                       "l2": "inputs larger than L2 (no flush)",
                       "parallelism": f"rows sharded over {world} GPU(s)" if world > 1 else "single GPU"}}
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(dict(base, impl="reference", unavailable="the reference has no pair-stack glue "
                                  "(its attention takes pre-projected tensors): no CPU arm for this workload")))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU path in the library)")
    torch.cuda.set_device(local)
    dist = group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    parity = None
    if not args.quick:
        parity = _parity(rank, world, group, dist)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps(dict(base, parity=parity, error="parity check failed: nothing was timed")), flush=True)
            sys.stdout.flush()
            os._exit(3)

    z, mask = pairstack.make_inputs(n)
    blocks = [pairstack.make_block_weights(s).to("cuda") for s in range(N_BLOCKS)]
    z_host, m_host = _shard(z, rank, world).pin_memory(), _shard(mask, rank, world).pin_memory()
    z_dev, m_dev = z_host.cuda(), m_host.cuda()
    for _ in range(args.warmup):
        out = pairstack.pair_stack(z_dev, m_dev, blocks, group)
    barrier()
    _lib.reset_launch_count()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    for _ in range(args.steps):
        out = pairstack.pair_stack(z_dev, m_dev, blocks, group)
    end.record()
    barrier()
    ms = beg.elapsed_time(end) / args.steps
    launches = _lib.launch_count()
    # end to end: the shard comes from pinned host memory and the result goes back, every step
    out_host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
    e_steps = max(2, min(args.steps, 5))
    barrier()
    beg.record()
    for _ in range(e_steps):
        z_dev.copy_(z_host, non_blocking=True)
        m_dev.copy_(m_host, non_blocking=True)
        out_host.copy_(pairstack.pair_stack(z_dev, m_dev, blocks, group), non_blocking=True)
    end.record()
    barrier()
    e2e_ms = beg.elapsed_time(end) / e_steps
    # per-kernel table from one more step
    _lib.profile_enable(True)
    pairstack.pair_stack(z_dev, m_dev, blocks, group)
    barrier()
    prof = _lib.profile_summary()
    _lib.profile_enable(False)
    t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        flops = pairstack.stack_flops(n, N_BLOCKS)
        kernels = {k: {"launches": v[0], "ms_per_step": v[1]} for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])}
        lib_ms = sum(v[1] for v in prof.values())
        print(json.dumps(dict(base, value=flops / (ms / 1e3) / 1e12, ms_per_step=ms,
                              e2e={"value": flops / (e2e_ms / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                                   "h2d_bytes_per_step": z_host.numel() * 2 + m_host.numel() * 2,
                                   "d2h_bytes_per_step": out_host.numel() * 2},
                              gpu_launches=launches, parity=parity, kernels=kernels,
                              time_in_library_kernels_ms=lib_ms, time_in_glue_and_exchanges_ms=ms - lib_ms)), flush=True)
    if dist is not None:
        try:
            dist.barrier()
        except Exception:
            pass
        sys.stdout.flush()
        os._exit(0)

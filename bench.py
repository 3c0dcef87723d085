"""Headline benchmark: triangle attention + triangle multiplicative update, forward+backward, N=768.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = triangle_attention fwd+bwd (B=1, N=768, H=4, D=32, bf16, pair bias + key mask) plus
triangle_multiplicative_update fwd+bwd in both directions (N=768, C=C_hidden=128, bf16), i.e. the
configuration the metric in BASELINE.json is quoted on.  Inputs are seeded synthetic tensors with the
shapes and distributions BASELINE.json lists.  Prints ONE JSON line (rank 0).

value      TFLOP/s over the timed steps with inputs resident in HBM (CUDA events, max over ranks).
e2e        the same metric through the public API with HOST (pinned) buffers: every step copies the
           inputs host->device and the results device->host inside the timed region.
roofline   the kernel with the largest share of the step, timed live with CUDA events on its stream
           (the library brackets each launch when profiling is on), against MEASURED_PEAKS.json.
parity     before anything is timed, the tensors the timed step produces are checked: on one GPU against the CPU
           oracle (attention: fp64 numpy on row and query slices; trimul: the torch restatement of the reference in
           fp32 on the same bf16-rounded inputs), on N GPUs every rank's shard against the single-GPU ops run on
           that rank.  A mismatch ends the run with a non-zero exit code.
cpu_baseline / --impl reference   the torch restatement of the reference's pure-torch CPU path (oracle/torch_reference.py),
           timed on this box's host cores with all of them, on the SAME configuration; `steps` is the number of
           steps actually run (bounded by a wall-clock budget).

--only attn|trimul restricts the step to one op (profiler captures); --workload stack runs the 4-block pair stack.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_RES, HEADS, HEAD_DIM, C_Z, C_HID = 768, 4, 32, 128, 128
CPU_SAMPLE_N = 192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def attn_flops(n, h=HEADS, d=HEAD_DIM, b=1):
    return 14.0 * b * n * h * n * n * d  # 4 fwd + 10 bwd per (row, head, query, key, d)


def trimul_flops(n, c=C_Z, ch=C_HID, b=1):
    m = b * n * n
    fwd = 2.0 * m * c * 4 * ch + 2.0 * m * c * c + 2.0 * m * ch * c + 2.0 * b * n ** 3 * ch
    return 3.0 * fwd  # backward = 2 x forward


def step_flops(n, only=None):
    return (attn_flops(n) if only != "trimul" else 0.0) + (2 * trimul_flops(n) if only != "attn" else 0.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.h)
                self.reasons |= {k for k, bit in names.items() if mask & bit}
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv is not None:
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.nv is not None:
            self.thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------
# synthetic inputs (host, fp32 draw -> bf16), BASELINE.json distributions
# ------------------------------------------------------------------------------------------------
def host_inputs(n, seed, torch, rows=None):
    """Inputs for one rank.  ``rows`` = (i0, i1) restricts the row axis (multi-GPU sharding)."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    rn = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(bf)  # noqa: E731
    i0, i1 = rows or (0, n)
    r = i1 - i0
    t = {
        "q": rn(1, r, n, HEADS, HEAD_DIM), "k": rn(1, r, n, HEADS, HEAD_DIM), "v": rn(1, r, n, HEADS, HEAD_DIM),
        "bias": rn(1, 1, HEADS, n, n), "d_o": rn(1, r, n, HEADS, HEAD_DIM),
        "x": rn(1, n, n, C_Z), "d_out": rn(1, n, n, C_Z),
        "pair_mask": (torch.rand(1, n, n, generator=g) < 0.9).to(bf),
    }
    key_mask = torch.rand(1, r, 1, 1, n, generator=g) < 0.95
    key_mask[..., 0] = True
    t["key_mask"] = key_mask
    w = {
        "norm_in_weight": 1 + rn(C_Z, sc=0.02).float(), "norm_in_bias": rn(C_Z, sc=0.02),
        "p_in_weight": rn(2 * C_HID, C_Z, sc=C_Z ** -0.5), "g_in_weight": rn(2 * C_HID, C_Z, sc=C_Z ** -0.5),
        "norm_out_weight": 1 + rn(C_HID, sc=0.02).float(), "norm_out_bias": rn(C_HID, sc=0.02),
        "p_out_weight": rn(C_Z, C_HID, sc=C_HID ** -0.5), "g_out_weight": rn(C_Z, C_Z, sc=C_Z ** -0.5),
    }
    w = {k: v.to(bf) for k, v in w.items()}
    return t, w


def one_step(t, w, torch, triangle_attention, trimul, only=None):
    """Forward+backward of the three ops through the public API; returns every result tensor."""
    res = []
    if only != "trimul":
        q, k, v, bias = (t[n].detach().requires_grad_() for n in ("q", "k", "v", "bias"))
        o = triangle_attention(q, k, v, bias, t["key_mask"], HEAD_DIM ** -0.5)
        res = [o, *torch.autograd.grad(o, [q, k, v, bias], grad_outputs=t["d_o"])]
    for direction in ("outgoing", "incoming") if only != "attn" else ():
        x = t["x"].detach().requires_grad_()
        wl = {n: p.detach().requires_grad_() for n, p in w.items()}
        out = trimul(x, direction, t["pair_mask"], **wl)
        res += [out, *torch.autograd.grad(out, [x, *wl.values()], grad_outputs=t["d_out"])]
    return res


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's pure-torch path (restated in oracle/torch_reference.py) on the host cores
# ------------------------------------------------------------------------------------------------
ATTN_ROW_CHUNK = 64   # rows per block on the CPU: the fp32 logits of one block are 0.6 GB at N=768


def cpu_step(t, w, tr, only=None):
    """One forward+backward of the three ops on the CPU, same inputs and dtype as the GPU step."""
    res = {}
    if only in (None, "attn"):
        res["attn"] = tr.attention_fwd_bwd(t["q"], t["k"], t["v"], t["bias"], t["key_mask"], HEAD_DIM ** -0.5, t["d_o"],
                                           row_chunk=ATTN_ROW_CHUNK)
    if only in (None, "trimul"):
        for direction in ("outgoing", "incoming"):
            res[direction] = tr.trimul_fwd_bwd(t["x"], direction, t["pair_mask"], w, t["d_out"])
    return res


def cpu_reference(n, steps, warmup, budget_s, only=None):
    """Time the CPU path at pair side ``n``: ``warmup`` untimed steps, then up to ``steps`` timed ones, stopping
    early once ``budget_s`` seconds of timed work have passed.  Returns (cpu_baseline dict, seconds per step,
    steps actually run)."""
    import torch

    from oracle import torch_reference as tr

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t, w = host_inputs(n, 0, torch)
    for _ in range(warmup):
        cpu_step(t, w, tr, only)
    done, t0 = 0, time.perf_counter()
    while done < steps:
        cpu_step(t, w, tr, only)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return {
        "value": step_flops(n, only) / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
        "sample": f"the whole step at N={n} in bf16 (torch {torch.__version__} CPU ops, {cores} threads; attention in "
                  f"blocks of {ATTN_ROW_CHUNK} rows), {dt:.2f} s per step, {done} timed step(s) after {warmup} warm-up",
    }, dt, done


# ------------------------------------------------------------------------------------------------
# parity of the timed tensors
# ------------------------------------------------------------------------------------------------
RESULT_NAMES = (["attn.out", "attn.dq", "attn.dk", "attn.dv", "attn.dbias"] +
                [f"{d}.{n}" for d in ("outgoing", "incoming") for n in
                 ("out", "dx", "d_norm_in_weight", "d_norm_in_bias", "d_p_in_weight", "d_g_in_weight", "d_norm_out_weight",
                  "d_norm_out_bias", "d_p_out_weight", "d_g_out_weight")])
# bf16 against a higher-precision result: the reference's own tables (testutil/metrics.py:96-108), rel-Frobenius
PARITY_FRO = {"attn": 5e-2, "outgoing": 1.5e-2, "incoming": 1.5e-2}


def _rel_fro(a, b):
    import numpy as np
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm((a - b).ravel()) / max(np.linalg.norm(b.ravel()), 1e-30))


def parity_single_gpu(res, host_t, host_w, torch, only=None):
    """Check the step's results (device tensors in RESULT_NAMES order) against the CPU oracle.

    Attention: fp64 numpy oracle on three 8-row slices (out, dq, dk, dv: rows are independent) and on a 16-query
    slice over all rows (the bias gradient of those queries, which is a sum over every row).  Trimul: the torch
    restatement of the reference in fp32 on the same bf16-rounded inputs, whole tensors, forward and every gradient.
    """
    import numpy as np

    from oracle import torch_reference as tr
    from oracle import triangle_oracle as orc

    f64 = lambda t: t.detach().double().cpu().numpy()  # noqa: E731
    got = dict(zip(names_for(only), res))
    report, worst = {}, 0.0
    if only in (None, "attn"):
        q, k, v, bias, d_o = (f64(host_t[m]) for m in ("q", "k", "v", "bias", "d_o"))
        mask = host_t["key_mask"].numpy()
        n_rows = q.shape[1]
        errs = {m: 0.0 for m in ("out", "dq", "dk", "dv")}
        for r0 in sorted({0, n_rows // 2 - 3, n_rows - 8}):
            sl = slice(r0, r0 + 8)
            o_ref = orc.triangle_attention_fwd(q[:, sl], k[:, sl], v[:, sl], bias, mask[:, sl], HEAD_DIM ** -0.5)
            g_ref = orc.triangle_attention_bwd(q[:, sl], k[:, sl], v[:, sl], bias, mask[:, sl], HEAD_DIM ** -0.5, d_o[:, sl])
            for m, ref in zip(("out", "dq", "dk", "dv"), (o_ref, *g_ref[:3])):
                errs[m] = max(errs[m], _rel_fro(f64(got["attn." + m][:, sl]), ref))
        qs = slice(q.shape[2] // 3, q.shape[2] // 3 + 16)
        db_ref = orc.triangle_attention_bwd(q[:, :, qs], k, v, bias[..., qs, :], mask, HEAD_DIM ** -0.5, d_o[:, :, qs])[3]
        errs["dbias"] = _rel_fro(f64(got["attn.dbias"][..., qs, :]), db_ref)
        for m, e in errs.items():
            report["attn." + m] = e
            worst = max(worst, e / PARITY_FRO["attn"])
    if only in (None, "trimul"):
        f32 = lambda d: {m: t.float() for m, t in d.items()}  # noqa: E731
        t32, w32 = f32({m: host_t[m] for m in ("x", "pair_mask", "d_out")}), f32(host_w)
        for direction in ("outgoing", "incoming"):
            o_ref, g_ref = tr.trimul_fwd_bwd(t32["x"], direction, t32["pair_mask"], w32, t32["d_out"])
            refs = {"out": o_ref, "dx": g_ref["x"], **{"d_" + m: g_ref[m] for m in host_w}}
            for m, ref in refs.items():
                e = _rel_fro(f64(got[f"{direction}.{m}"]), ref.double().numpy())
                report[f"{direction}.{m}"] = e
                worst = max(worst, e / PARITY_FRO[direction])
    return {"against": "cpu oracle (attention: fp64 numpy on row / query slices; trimul: fp32 torch restatement)",
            "metric": "rel-Frobenius", "bounds": PARITY_FRO, "max_rel_fro": report, "ok": worst <= 1.0}


def names_for(only):
    if only == "attn":
        return RESULT_NAMES[:5]
    if only == "trimul":
        return RESULT_NAMES[5:]
    return RESULT_NAMES


def parity_sharded(res, dev_t, dev_w, rank, world, torch, triangle_attention, trimul, dist, n):
    """Every rank runs the single-GPU ops on the WHOLE problem and compares its shard of each result (weight and
    bias gradients: the whole tensor, they come back summed over ranks).  Returns the worst rel-Frobenius per
    tensor over all ranks."""
    from geometric_nn_ops_b200 import sharded
    i0, i1 = sharded.shard_rows(n, rank, world)
    full_t, full_w = host_inputs(n, 0, torch)
    full_t = {m: t.cuda() for m, t in full_t.items()}
    ref = one_step(full_t, dev_w, torch, triangle_attention, trimul)
    errs = []
    for name, a, b in zip(RESULT_NAMES, res, ref):
        whole = name == "attn.dbias" or (".d_" in name)
        if not whole:
            b = b[:, i0:i1]
        a, b = a.detach(), b.detach()
        errs.append(float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)))
    e = torch.tensor(errs, device="cuda", dtype=torch.float64)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    errs = e.tolist()
    # same kernels on the same rows: attention is bit-identical, the rest agrees to the rounding of the split sums
    ok = True
    for name, err in zip(RESULT_NAMES, errs):
        op, m = name.split(".", 1)
        lim = 0.0 if (op == "attn" and m in ("out", "dq", "dk", "dv")) else (1e-3 if m == "out" else 3e-2)
        ok = ok and err <= lim
    return {"against": "single-GPU ops on the same rank, whole problem", "metric": "rel-Frobenius, max over ranks",
            "max_rel_fro": dict(zip(RESULT_NAMES, errs)), "ok": ok,
            "exchange": sharded.exchange_route(torch.device("cuda", torch.cuda.current_device()))}


def _finish(dist):
    """Leave a multi-rank run without tearing NCCL down: a captured graph still references the communicator,
    and destroying the process group under it has hung; the process is about to exit anyway."""
    try:
        dist.barrier()
    except Exception:
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--n-res", type=int, default=N_RES, help="pair side (default: the headline 768)")
    ap.add_argument("--graph", action="store_true", help="(default) replay the step from a CUDA graph")
    ap.add_argument("--eager", action="store_true", help="launch the timed steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--quick", action="store_true",
                    help="timed region only: no parity check, no end-to-end leg and no CPU baseline (for profiler captures)")
    ap.add_argument("--only", choices=["attn", "trimul"], default=None,
                    help="restrict the step to triangle attention or to the two multiplicative updates (single GPU)")
    ap.add_argument("--workload", choices=["ops", "stack"], default="ops",
                    help="ops: the headline step (default); stack: the 4-block pair stack, bf16 inference")
    ap.add_argument("--cpu-budget", type=float, default=150.0,
                    help="--impl reference: stop after this many seconds of timed CPU steps")
    args = ap.parse_args()
    if args.workload == "stack":
        import bench_stack
        return bench_stack.main(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n, only = args.n_res, args.only
    if only is not None and world > 1:
        raise SystemExit("--only is a single-GPU option")
    ops = {"attn": f"tri-attn fwd+bwd (B=1,N={n},H={HEADS},D={HEAD_DIM})",
           "trimul": f"trimul outgoing+incoming fwd+bwd (N={n},C={C_Z},Ch={C_HID})"}
    config = {"workload": " + ".join(ops[m] for m in ("attn", "trimul") if only in (None, m)) + ", bf16",
              "l2": "inputs larger than L2 (no flush)",
              "parallelism": f"rows sharded over {world} GPU(s)" if world > 1 else "single GPU"}
    what = {None: "tri-attn+trimul", "attn": "tri-attn", "trimul": "trimul"}[only]
    base = {"metric": f"{what} fwd+bwd TFLOP/s, N={n}", "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config}

    if args.impl == "reference":
        if rank != 0:
            return
        warm = min(args.warmup, 1)
        cpu, dt, done = cpu_reference(n, max(1, args.steps), warm, args.cpu_budget, only)
        line = dict(base, impl="reference", steps=done, warmup=warm, value=cpu["value"], ms_per_step=dt * 1e3,
                    cpu_baseline=cpu,
                    e2e={"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        # `config` stays the b200 arm's, key for key; what differs about this run is said here
        line["reference_run"] = {"where": "host cores", "steps_requested": args.steps, "warmup_requested": args.warmup,
                                 "note": "steps and warmup are what was run: a CPU step takes seconds and the run "
                                         "stops once --cpu-budget seconds of timed steps have passed"}
        print(json.dumps(line))
        return

    import torch

    from geometric_nn_ops_b200 import _lib
    from geometric_nn_ops_b200.triangle import triangle_attention, trimul_b200

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU path in the library)")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"   # keep stdout to the one JSON line
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world > 1:
        from geometric_nn_ops_b200 import sharded
        step_fn, host_t, host_w = sharded.make_bench_step(n, rank, world, host_inputs)
    else:
        host_t, host_w = host_inputs(n, 0, torch)
        step_fn = lambda t, w: one_step(t, w, torch, triangle_attention, trimul_b200, only)  # noqa: E731
    pin = lambda d: {k_: v_.pin_memory() for k_, v_ in d.items()}  # noqa: E731
    host_t, host_w = pin(host_t), pin(host_w)
    to_dev = lambda d: {k_: v_.cuda(non_blocking=True) for k_, v_ in d.items()}  # noqa: E731
    dev_t, dev_w = to_dev(host_t), to_dev(host_w)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity of the tensors about to be timed (the reference's benchmarks check before timing too,
    # benchmarks/bench_trimul_micro.py:67-69) ------------------------------------------------------------------
    parity = None
    if not args.quick:
        res = step_fn(dev_t, dev_w)
        torch.cuda.synchronize()
        if world > 1:
            sharded.check_exchange_status()      # no barrier wait may have run out
            parity = parity_sharded(res, dev_t, dev_w, rank, world, torch, triangle_attention, trimul_b200, dist, n)
        else:
            parity = parity_single_gpu(res, host_t, host_w, torch, only)
        del res
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps(dict(base, parity=parity, error="parity check failed: nothing was timed")), flush=True)
            if dist is not None:
                try:
                    dist.barrier()
                except Exception:
                    pass
            sys.stdout.flush()
            os._exit(3)

    for _ in range(args.warmup):
        step_fn(dev_t, dev_w)
    barrier()

    # ---- timed region: device-resident inputs -------------------------------------------------
    # A step is ~190 launches; on several GPUs each rank's shard is small enough for host launch latency to show,
    # and on one GPU the library's per-kernel event brackets would otherwise sit inside the timed region.  So
    # the whole step (kernels and exchanges) is captured once in a CUDA graph and replayed, and the kernel
    # table comes from one extra eager step outside the timed region (--eager times eager launches instead).
    graph = None
    if not args.eager:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_fn(dev_t, dev_w)
            torch.cuda.current_stream().wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step_fn(dev_t, dev_w)   # noqa: F841  (keeps the captured outputs alive)
            graph.replay()
            barrier()
        except Exception as exc:   # capture is an optimisation: fall back to eager launches
            print(f"[bench] CUDA graph capture failed, running eagerly: {exc!r}", file=sys.stderr)
            graph = None
            barrier()
    config["launch"] = "cuda graph replay" if graph is not None else "eager"
    _lib.reset_launch_count()
    if graph is None:
        _lib.profile_enable(True)
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        beg.record()
        for _ in range(args.steps):
            if graph is not None:
                graph.replay()
            else:
                step_fn(dev_t, dev_w)
        end.record()
        barrier()
    ms = beg.elapsed_time(end) / args.steps
    if world > 1:
        sharded.check_exchange_status()
    launches = _lib.launch_count()
    prof_steps = args.steps
    exchanges = None
    if graph is not None:   # launches and per-kernel times from one eager step outside the timed region
        _lib.reset_launch_count()
        _lib.profile_enable(True)
        if world > 1:
            from geometric_nn_ops_b200 import sharded as _sh
            _sh.TIMERS = {}
        step_fn(dev_t, dev_w)
        barrier()
        if world > 1:
            exchanges = {k_: {"calls": v_[0], "ms_per_step": v_[1]} for k_, v_ in _sh.timing_summary().items()}
            _sh.TIMERS = None
        launches = _lib.launch_count() * args.steps
        prof_steps = 1
    prof = _lib.profile_summary()
    _lib.profile_enable(False)

    # ---- e2e: host buffers, copies inside the timed region --------------------------------------
    # Every step copies all inputs from pinned host memory and all results back.  Three streams (copy-in,
    # compute, copy-out) and two sets of device input buffers let the PCIe transfers of neighbouring steps
    # overlap the kernels, as a server streaming independent requests would; one untimed step first
    # allocates the device and pinned result buffers.
    h2d = sum(v.numel() * v.element_size() for v in list(host_t.values()) + list(host_w.values()))
    e2e_steps = 2 if args.quick else max(3, min(args.steps, 8))
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_sets = [(to_dev(host_t), to_dev(host_w)) for _ in range(2)]
    res = step_fn(*dev_sets[0])
    out_host = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in res]
    d2h = sum(r.numel() * r.element_size() for r in out_host)
    del res
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    barrier()
    t_beg = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_beg.record(main)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    for k in range(e2e_steps):
        i = k & 1
        dt, dw = dev_sets[i]
        with torch.cuda.stream(s_in):
            if k >= 2:
                s_in.wait_event(ev_done[i])          # the step that last used this input set has run
            for name, src in host_t.items():
                dt[name].copy_(src, non_blocking=True)
            for name, src in host_w.items():
                dw[name].copy_(src, non_blocking=True)
            ev_in[i].record(s_in)
        main.wait_event(ev_in[i])
        res = step_fn(dt, dw)
        ev_done[i].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            for dst, src in zip(out_host, res):
                src.record_stream(s_out)
                dst.copy_(src, non_blocking=True)
    main.wait_stream(s_out)
    main.wait_stream(s_in)
    t_end.record(main)
    barrier()
    e2e_ms = t_beg.elapsed_time(t_end) / e2e_steps

    times = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    if rank != 0:
        _finish(dist)
        return

    flops = step_flops(n, only)
    pk, pk_kind = peaks()
    top = max(prof.items(), key=lambda kv: kv[1][1]) if prof else None
    roofline = None
    if top is not None:
        name, (cnt, tot_ms, kflops, kbytes) = top
        sec = tot_ms / 1e3
        tensor_bound = kflops > 0 and kflops / max(kbytes, 1.0) > pk["bf16_tflops"] * 1e12 / (pk["hbm_gbs"] * 1e9)
        extra = {}
        if tensor_bound:
            # the kernel is timed on its own by event brackets: the burst figure is the denominator
            ach, peak, unit = kflops / sec / 1e12, pk["bf16_tflops"], "TFLOP/s"
            extra = {"peak_sustained": pk["bf16_tflops_sustained"], "frac_of_sustained": ach / pk["bf16_tflops_sustained"]}
        else:
            ach, peak, unit = kbytes / sec / 1e9, pk["hbm_gbs"], "GB/s"
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "ncu_dram_traffic_n768_bf16.json")
        if world == 1 and n == N_RES and os.path.exists(tpath):
            with open(tpath) as f:
                traffic = json.load(f).get(name)
        roofline = {"kernel": name, "bound": "tensor" if tensor_bound else "hbm", "achieved": ach, "peak": peak,
                    "unit": unit, "frac": ach / peak, "traffic": traffic,
                    "traffic_source": "one ncu capture of this kernel at this size (profiles/ncu_dram_traffic_n768_bf16.json)"
                    if traffic is not None else None,
                    "peak_source": f"of {pk_kind} (burst)" if tensor_bound else f"of {pk_kind}",
                    "launches": cnt, "avg_launch_ms": tot_ms / cnt, "share_of_step": tot_ms / prof_steps / ms, **extra}
        if name.startswith("tc_attn_") and name != "tc_attn_delta":
            # The attention passes are dense contractions by their FLOPs, but what binds them is the exponential
            # (MUFU) pipe: one ex2 per (row, head, query, key) per pass, 16 per clock per SM.
            sm_mhz = clocks.summary().get("sm_mhz") or 1965
            exps = float(n) ** 3 * HEADS / world
            peak_exp = 16.0 * 148 * sm_mhz * 1e6
            roofline["binding_pipe"] = "exp (MUFU)"
            roofline["exp_pipe"] = {"exponentials_per_launch": exps, "achieved_per_s": exps / (sec / cnt),
                                    "peak_per_s": peak_exp, "frac": exps / (sec / cnt) / peak_exp}
    kernels = {k_: {"launches": v_[0], "ms_per_step": v_[1] / prof_steps} for k_, v_ in
               sorted(prof.items(), key=lambda kv: -kv[1][1])}
    cpu = None
    if world == 1 and not args.quick:
        cpu, _, _ = cpu_reference(n, 1, 0, 0.0, only)
    line = dict(base, value=flops / (ms / 1e3) / 1e12, ms_per_step=ms,
                pct_of_bf16_peak={"measured_burst": flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"] / world,
                                  "measured_sustained": flops / (ms / 1e3) / 1e12 / pk["bf16_tflops_sustained"] / world,
                                  "nominal_2250": flops / (ms / 1e3) / 1e12 / 2250.0 / world},
                e2e={"value": flops / (e2e_ms / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                     "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                gpu_launches=launches, path=_lib.last_path(), clocks=clocks.summary(), roofline=roofline,
                parity=parity, kernels=kernels, exchanges=exchanges, cpu_baseline=cpu)
    print(json.dumps(line), flush=True)
    if dist is not None:
        _finish(dist)


if __name__ == "__main__":
    main()

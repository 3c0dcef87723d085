"""Size sweeps of the two triangle ops and of a residual stack of multiplicative updates.

    python bench_sweep.py trimul    --sizes 256 384 512 768 --dtype bf16 [--biases] [--out FILE.csv]
    python bench_sweep.py attention --sizes 256 384 512 768 --dtype bf16 [--out FILE.csv]
    python bench_sweep.py stack     --sizes 256 512 768 --depth 48 --directions alternate [--out FILE.csv]

These stand where the reference has ``benchmarks/bench_trimul_micro.py`` (forward in training and inference mode
and backward per size and direction, each case checked against the fp64 reference before it is timed,
``:67-72, 148``) and ``benchmarks/bench_trimul_stack.py`` (a residual stack of depth D, inference and training
step, with peak allocated / reserved memory columns, ``:54-99``); the reference has no triangle-attention sweep,
``attention`` adds one.  Timing follows their convention: a warm-up window, then the median over a measurement
window, each repetition bracketed by CUDA events, with a buffer larger than L2 written between repetitions.
Before a case is timed its result is compared with the CPU oracle (``oracle/``, used here as the checker only:
the sweep refuses to time a case that fails); sizes above ``--check-max`` are checked on a
reduced problem of the same kind, because the fp64 oracle of a whole N=768 update takes a minute.
"""

import argparse
import csv
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _timed_ms(fn, warmup_ms, rep_ms):
    """Median device time of ``fn`` in ms (CUDA events), L2 flushed between repetitions."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn()
    torch.cuda.synchronize()
    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    beg.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    one = max(beg.elapsed_time(end), 1e-3)
    for _ in range(max(1, int(warmup_ms / one))):
        fn()
    times = []
    for _ in range(max(3, min(200, int(rep_ms / one)))):
        flush.zero_()
        beg.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(beg.elapsed_time(end))
    return statistics.median(times)


def _peak_memory_gib(fn):
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    fn()
    torch.cuda.synchronize()
    return torch.cuda.max_memory_allocated() / 2 ** 30, torch.cuda.max_memory_reserved() / 2 ** 30


def _oracle_modules():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from tests import util
    return util


def _check_trimul(op, n, c, dtype, direction, biases, util):
    x, mask, w, d_out = util.trimul_inputs(1, n, c, c, dtype, seed=3, biases=biases)
    out, grads = util.trimul_fwd_bwd(op, x, mask, w, direction, d_out)
    o_ref, g_ref = util.trimul_oracle(x, mask, w, direction, d_out)
    precision = "tf32" if dtype == torch.float32 and torch.backends.cuda.matmul.fp32_precision == "tf32" else "ieee"
    cos_min, fro = util.TRIMUL_TOL[dtype, precision]
    util.check_close("out", out, o_ref, cos_min, fro)
    for name, val in grads.items():
        util.check_close("grad_" + name, val, g_ref[name], cos_min, fro)


def sweep_trimul(args):
    from geometric_nn_ops_b200.triangle import trimul_b200
    util = _oracle_modules()
    dtype = DTYPES[args.dtype]
    rows = []
    for n in args.sizes:
        for direction in args.directions:
            _check_trimul(trimul_b200, min(n, args.check_max), args.channels, dtype, direction, args.biases, util)
            x, mask, w, d_out = util.trimul_inputs(1, n, args.channels, args.channels, dtype, seed=3, biases=args.biases)
            xl = x.clone().requires_grad_()
            wl = {k: v.clone().requires_grad_() for k, v in w.items()}
            leaves = [xl, *wl.values()]

            def fwd_infer():
                with torch.no_grad():
                    return trimul_b200(x, direction, mask, **w)

            def fwd_train():
                return trimul_b200(xl, direction, mask, **wl)

            out = fwd_train()

            def bwd():
                torch.autograd.grad(out, leaves, grad_outputs=d_out, retain_graph=True)

            m = float(n) * n
            flops = 2.0 * m * args.channels * 6 * args.channels + 2.0 * float(n) ** 3 * args.channels
            row = {"size": n, "direction": direction, "dtype": args.dtype,
                   "fwd_infer_ms": _timed_ms(fwd_infer, args.warmup, args.rep),
                   "fwd_train_ms": _timed_ms(fwd_train, args.warmup, args.rep),
                   "bwd_ms": _timed_ms(bwd, args.warmup, args.rep)}
            row["fwd_infer_tflops"] = flops / row["fwd_infer_ms"] / 1e9
            row["bwd_tflops"] = 2 * flops / row["bwd_ms"] / 1e9
            rows.append(row)
            print(row, flush=True)
            del out
    return rows


def sweep_attention(args):
    from geometric_nn_ops_b200.triangle import triangle_attention
    util = _oracle_modules()
    dtype = DTYPES[args.dtype]
    rows = []
    for n in args.sizes:
        # oracle check on a slice of rows of the full-size problem (rows are independent)
        t, mask, d_out = util.attn_inputs(1, 8, n, args.heads, args.head_dim, dtype, seed=5, keep=0.95)
        out, grads = util.attn_fwd_bwd(triangle_attention, t, mask, None, d_out)
        o_ref, g_ref = util.attn_oracle(t, mask, None, d_out)
        cos_min, fro = util.ATTN_TOL[dtype, "ieee" if dtype != torch.float32 else
                                     ("tf32" if torch.backends.cuda.matmul.fp32_precision == "tf32" else "ieee")]
        util.check_close("out", out, o_ref, cos_min, fro)
        for name, val in grads.items():
            util.check_close("grad_" + name, val, g_ref[name], cos_min, fro)
        t, mask, d_out = util.attn_inputs(1, n, n, args.heads, args.head_dim, dtype, seed=5, keep=0.95)
        leaves = {k: v.clone().requires_grad_() for k, v in t.items()}

        def fwd_infer():
            with torch.no_grad():
                return triangle_attention(t["q"], t["k"], t["v"], t["bias"], mask)

        def fwd_train():
            return triangle_attention(leaves["q"], leaves["k"], leaves["v"], leaves["bias"], mask)

        out = fwd_train()

        def bwd():
            torch.autograd.grad(out, list(leaves.values()), grad_outputs=d_out, retain_graph=True)

        pairs = float(n) * args.heads * n * n
        row = {"size": n, "heads": args.heads, "head_dim": args.head_dim, "dtype": args.dtype,
               "fwd_infer_ms": _timed_ms(fwd_infer, args.warmup, args.rep),
               "fwd_train_ms": _timed_ms(fwd_train, args.warmup, args.rep),
               "bwd_ms": _timed_ms(bwd, args.warmup, args.rep)}
        row["fwd_infer_tflops"] = 4.0 * pairs * args.head_dim / row["fwd_infer_ms"] / 1e9
        row["bwd_tflops"] = 10.0 * pairs * args.head_dim / row["bwd_ms"] / 1e9
        rows.append(row)
        print(row, flush=True)
        del out
    return rows


def sweep_stack(args):
    """Residual stack ``x = x + layer(x, mask)`` of ``depth`` multiplicative updates (the reference's stack
    convention, testutil/trimul.py:161-164): inference step, training step, peak memory of each."""
    from geometric_nn_ops_b200.triangle import trimul_b200
    util = _oracle_modules()
    dtype = DTYPES[args.dtype]
    rows = []
    for n in args.sizes:
        for direction in args.directions:
            dirs = [("outgoing", "incoming")[i % 2] if direction == "alternate" else direction for i in range(args.depth)]
            _check_trimul(trimul_b200, min(n, args.check_max), args.channels, dtype, dirs[0], args.biases, util)
            layers = [util.trimul_inputs(1, 8, args.channels, args.channels, dtype, seed=10 + i, biases=args.biases)[2]
                      for i in range(args.depth)]
            x, mask, _, d_out = util.trimul_inputs(1, n, args.channels, args.channels, dtype, seed=4)
            params = [p.requires_grad_() for w in layers for p in w.values()]
            xl = x.clone().requires_grad_()

            def run(x0):
                z = x0
                for w, d in zip(layers, dirs):
                    z = z + trimul_b200(z, d, mask, **w)
                return z

            def infer_step():
                with torch.no_grad():
                    return run(x)

            def train_step():
                torch.autograd.grad(run(xl), [xl, *params], grad_outputs=d_out)

            if not torch.isfinite(infer_step().float()).all():
                raise RuntimeError("non-finite output")
            row = {"depth": args.depth, "size": n, "direction": direction, "dtype": args.dtype}
            for name, step in (("infer_step", infer_step), ("train_step", train_step)):
                row[name + "_ms"] = _timed_ms(step, args.warmup, args.rep)
                row[name + "_alloc_gib"], row[name + "_reserved_gib"] = _peak_memory_gib(step)
            rows.append(row)
            print(row, flush=True)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["trimul", "attention", "stack"])
    ap.add_argument("--sizes", type=int, nargs="+", default=[256, 384, 512, 768], help="pair side N")
    ap.add_argument("--channels", type=int, default=128, help="c_z == c_hidden")
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=32)
    ap.add_argument("--directions", nargs="+", default=None, choices=["outgoing", "incoming", "alternate"])
    ap.add_argument("--dtype", default="bf16", choices=list(DTYPES))
    ap.add_argument("--biases", action="store_true", help="give the projections biases")
    ap.add_argument("--depth", type=int, default=48, help="stack: number of layers")
    ap.add_argument("--warmup", type=float, default=25.0, help="warm-up window (ms)")
    ap.add_argument("--rep", type=float, default=100.0, help="measurement window (ms)")
    ap.add_argument("--check-max", type=int, default=256, help="largest N whose whole result is compared with the fp64 oracle")
    ap.add_argument("--out", default=None, help="write the rows to this CSV file")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a GPU (there is no CPU path in the library)")
    if args.directions is None:
        args.directions = ["alternate"] if args.what == "stack" else ["outgoing", "incoming"]
    if args.what != "stack" and "alternate" in args.directions:
        raise SystemExit("'alternate' only means something for a stack")
    print(f"# device {torch.cuda.get_device_name(0)}, torch {torch.__version__}, dtype {args.dtype}, "
          f"fp32 matmul precision {torch.backends.cuda.matmul.fp32_precision}")
    rows = {"trimul": sweep_trimul, "attention": sweep_attention, "stack": sweep_stack}[args.what](args)
    if args.out and rows:
        with open(args.out, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0]))
            wr.writeheader()
            wr.writerows(rows)
    return rows


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Single-GPU Newton-Schulz microbenchmark.

Shapes 4096x4096, 1024x4096, 4096x14336, 14336x4096, 3072x8192, 8 matrices of
each, bf16, entries iid N(0,1).  Two schedules:

  classic   5 quintic iterations with (3.4445, -4.7750, 2.0315), direct form
            with the Gram matrix on the smaller dimension
  polar     the production schedule: Polar-Express coefficients, Gram form,
            restart at iteration 2, fp16 operands (``polar-bf16``: bf16 operands)

For every shape the script prints the time per batch of 8, dense-equivalent
TFLOP/s (every product counted as a full 2*m*k*n GEMM, the convention that
makes implementations comparable) and the orthogonality error
max|X X^T - I| next to that of an fp32 PyTorch run of the same schedule.

    python benchmarks/bench_ns.py                  # this package's kernels
    python benchmarks/bench_ns.py --impl reference # the reference from baseline/_ref
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPES = [(4096, 4096), (1024, 4096), (4096, 14336), (14336, 4096), (3072, 8192)]
CLASSIC = [(3.4445, -4.7750, 2.0315)] * 5


def dense_flops(m0: int, n0: int, schedule: str) -> float:
    m, n = min(m0, n0), max(m0, n0)
    if schedule == "classic":
        return 5.0 * (4.0 * m * m * n + 2.0 * m**3)
    return 28.0 * m**3 + 8.0 * m * m * n


def orth_err(O) -> float:
    import torch

    X = O.float()
    if X.shape[0] > X.shape[1]:
        X = X.T
    return (X @ X.T - torch.eye(X.shape[0], device=X.device)).abs().max().item()


def fp32_reference(G, schedule: str):
    sys.path.insert(0, ROOT) if ROOT not in sys.path else None
    import torch

    X = G.float()
    t = X.shape[0] > X.shape[1]
    if t:
        X = X.T
    X = X / (X.norm() + 1e-7)
    if schedule == "classic":
        for a, b, c in CLASSIC:
            A = X @ X.T
            X = a * X + (b * A + c * A @ A) @ X
    else:
        sys.path.insert(0, ROOT) if ROOT not in sys.path else None
        from dmuon_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFICIENTS, _gram_iteration

        _, X = _gram_iteration(X, list(POLAR_EXPRESS_COEFFICIENTS), [2])
    return X.T if t else X


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--schedules", default="classic,polar,polar-bf16")
    args = ap.parse_args()
    import torch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.impl == "ours":
        sys.path.insert(0, ROOT)
        from dmuon_b200.ops import gemm as G
        from dmuon_b200.ops import ns_sm100
        from dmuon_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFICIENTS

        def run(X, schedule):
            if schedule == "classic":
                return ns_sm100.newton_schulz_batched(X, CLASSIC, [], 1e-7, "direct", torch.bfloat16)
            cd = torch.bfloat16 if schedule == "polar-bf16" else torch.float16
            return ns_sm100.newton_schulz_batched(X, list(POLAR_EXPRESS_COEFFICIENTS), [2], 1e-7, "gram", cd)

        info = {"backend": "tcgen05 sm_100a kernels"}
    else:
        ref = os.path.join(ROOT, "baseline", "_ref")
        sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
        sys.path.insert(0, ref)
        import importlib

        import dmuon

        nsmod = importlib.import_module("dmuon.optim.newton_schulz")
        ns = dmuon.NewtonSchulz()          # production path: selects quack / cuBLAS per shape
        status = dmuon.get_backend_status() if hasattr(dmuon, "get_backend_status") else {}

        def run(X, schedule):
            outs = []
            for i in range(X.shape[0]):
                if schedule == "classic":
                    outs.append(nsmod.direct_newton_schulz(X[i], steps=5, coefficients=CLASSIC))
                else:
                    outs.append(ns.local(X[i], 5))
            return torch.stack(outs)

        info = {"backend": str(status)}

    rows = []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for schedule in args.schedules.split(","):
        if args.impl == "reference" and schedule == "polar-bf16":
            continue                                # the reference's Gram path is fp16 only
        for m0, n0 in SHAPES:
            torch.manual_seed(0)
            X = torch.randn(args.batch, m0, n0, device=dev).bfloat16()
            for _ in range(args.warmup):
                out = run(X, schedule)
            torch.cuda.synchronize()
            times = []
            for _ in range(args.iters):
                flush.zero_()                      # 256 MiB write: evicts the 126 MB L2
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                out = run(X, schedule)
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            ms = sorted(times)[len(times) // 2]
            err = max(orth_err(out[i]) for i in range(min(2, args.batch)))
            ref32 = fp32_reference(X[0], schedule)
            row = {
                "impl": args.impl, "schedule": schedule, "shape": [m0, n0], "batch": args.batch,
                "ms_per_batch": round(ms, 4),
                "dense_tflops": round(dense_flops(m0, n0, schedule) * args.batch / ms / 1e9, 1),
                "orth_err": round(err, 4), "orth_err_fp32": round(orth_err(ref32), 4),
                "max_abs_diff_vs_fp32": round((out[0].float() - ref32).abs().max().item(), 4),
            }
            rows.append(row)
            print(json.dumps(row), flush=True)
    if args.impl == "ours":
        G.check_status(dev)
    print(json.dumps({"impl": args.impl, "info": info, "rows": len(rows)}))


if __name__ == "__main__":
    main()

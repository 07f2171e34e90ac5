#!/usr/bin/env python
"""Symmetric products and Gram Newton-Schulz over the projection shapes of common LLMs.

    python benchmarks/bench_syrk.py summary                  # per shape: X X^T against cuBLAS, Gram NS end to end
    python benchmarks/bench_syrk.py detail --models 8B       # per shape: every product class of one iteration
    python benchmarks/bench_syrk.py                          # both

``summary`` times, for every (model, projection) shape with ``--batch`` matrices:

* the Gram product ``R = X X^T`` (``m x m`` output, ``K = n``) on this package's
  symmetric kernel (lower-triangle tiles computed, mirrored on store) against
  ``torch.bmm(X, X^T)`` (cuBLAS computes the full square);
* one production Newton-Schulz (Gram form, Polar-Express coefficients, restart at
  iteration 2, fp16 operands) on the kernels against the same schedule in PyTorch
  (library GEMMs, fp16).

``detail`` splits one iteration into its product classes -- Gram ``X X^T``
(symmetric, K = n), polynomial ``R R`` (symmetric, K = m, with and without a ``C``
operand) and apply ``Q X`` (dense) -- each against ``torch.bmm``.

Times are CUDA events after warm-up with a 256 MiB write between repetitions (the
126 MB L2 does not hold the operands of the previous one); TFLOP/s are
dense-equivalent (a symmetric product is counted as the full ``2 m m k``).  One JSON
line per row.  Counterpart of the reference's ``benchmarks/bench_syrk.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

#: (model, hidden, ffn, q heads, kv heads, head dim)
MODELS = {
    "1B": ("Llama-3.2-1B", 2048, 8192, 32, 8, 64),
    "3B": ("Llama-3.2-3B", 3072, 8192, 24, 8, 128),
    "8B": ("Llama-3.1-8B", 4096, 14336, 32, 8, 128),
    "70B": ("Llama-3.1-70B", 8192, 28672, 64, 8, 128),
}


def shapes_of(key: str) -> list[tuple[str, str, int, int]]:
    name, d, ffn, h, kv, hd = MODELS[key]
    return [
        (name, "q_proj", h * hd, d), (name, "k_proj", kv * hd, d), (name, "v_proj", kv * hd, d), (name, "o_proj", d, h * hd),
        (name, "gate_proj", ffn, d), (name, "up_proj", ffn, d), (name, "down_proj", d, ffn),
    ]


def unique_shapes(keys) -> list[tuple[str, str, int, int]]:
    seen, out = set(), []
    for k in keys:
        for model, proj, rows, cols in shapes_of(k):
            m, n = min(rows, cols), max(rows, cols)
            if (m, n) in seen:
                continue
            seen.add((m, n))
            out.append((model, proj, rows, cols))
    return out


class Timer:
    def __init__(self, torch, dev, iters: int, warmup: int):
        self.torch, self.iters, self.warmup = torch, iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self, fn) -> float:
        torch = self.torch
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return sorted(times)[len(times) // 2]


def batch_for(m: int, n: int, want: int) -> int:
    """Keep operands and outputs of one case within a few GB."""
    per = (m * n + m * m) * 2
    return max(1, min(want, int(3e9 // max(per, 1))))


def summary(args, torch, G, ns_sm100, timer) -> None:
    from dmuon_b200.optim.newton_schulz import POLAR_EXPRESS_COEFFICIENTS, _gram_iteration

    dev = torch.device("cuda", 0)
    coefs = list(POLAR_EXPRESS_COEFFICIENTS)
    for model, proj, rows, cols in unique_shapes(args.models):
        m, n = min(rows, cols), max(rows, cols)
        L = batch_for(m, n, args.batch)
        torch.manual_seed(0)
        X = (torch.randn(L, m, n, device=dev) * 0.05).to(torch.float16)
        R = torch.empty(L, m, m, device=dev, dtype=torch.float16)

        def ours():
            G.gemm(X, X, R, symmetric=True)

        def lib():
            torch.bmm(X, X.transpose(1, 2), out=R)

        t_ours, t_lib = timer(ours), timer(lib)
        flop = 2.0 * m * m * n * L

        Gm = torch.randn(L, rows, cols, device=dev).bfloat16()

        def ns_ours():
            return ns_sm100.newton_schulz_batched(Gm, coefs, [2], 1e-7, "gram", torch.float16)

        def ns_lib():
            outs = []
            for i in range(L):
                x = Gm[i].float()
                x = x.T if rows > cols else x
                x = (x / (x.norm() + 1e-7)).to(torch.float16)
                outs.append(_gram_iteration(x, coefs, [2])[1])
            return outs

        t_ns, t_ns_lib = timer(ns_ours), timer(ns_lib)
        print(json.dumps({
            "what": "summary", "model": model, "proj": proj, "shape": [rows, cols], "batch": L,
            "gram_ms": round(t_ours, 4), "gram_cublas_ms": round(t_lib, 4), "gram_speedup": round(t_lib / t_ours, 3),
            "gram_dense_tflops": round(flop / t_ours / 1e9, 1), "gram_cublas_tflops": round(flop / t_lib / 1e9, 1),
            "ns_ms": round(t_ns, 4), "ns_pytorch_ms": round(t_ns_lib, 4), "ns_speedup": round(t_ns_lib / t_ns, 3),
        }), flush=True)
        G.check_status(dev)


def detail(args, torch, G, timer) -> None:
    dev = torch.device("cuda", 0)
    for model, proj, rows, cols in unique_shapes(args.models):
        m, n = min(rows, cols), max(rows, cols)
        L = batch_for(m, n, args.batch)
        torch.manual_seed(0)
        X = (torch.randn(L, m, n, device=dev) * 0.05).to(torch.float16)
        S = (torch.randn(L, m, m, device=dev) * 0.05).to(torch.float16)
        S = ((S + S.transpose(1, 2)) * 0.5).contiguous()                  # symmetric operand, as R and P are
        C = S.clone()
        Rm = torch.empty(L, m, m, device=dev, dtype=torch.float16)
        Y = torch.empty(L, m, n, device=dev, dtype=torch.float16)
        cases = {
            "gram  X X^T      (sym, K=n)": (lambda: G.gemm(X, X, Rm, symmetric=True),
                                            lambda: torch.bmm(X, X.transpose(1, 2), out=Rm), 2.0 * m * m * n),
            "poly  R R        (sym, K=m)": (lambda: G.gemm(S, S, Rm, symmetric=True),
                                            lambda: torch.bmm(S, S, out=Rm), 2.0 * m * m * m),
            "poly  c R R + b R (sym, C) ": (lambda: G.gemm(S, S, Rm, C=C, beta=0.5, symmetric=True),
                                            lambda: torch.baddbmm(C, S, S, beta=0.5, out=Rm), 2.0 * m * m * m),
            "apply Q X        (dense, X read as stored)": (lambda: G.gemm(S, X, Y, b_mn=True),
                                            lambda: torch.bmm(S, X, out=Y), 2.0 * m * m * n),
        }
        for label, (ours, lib, flop1) in cases.items():
            t_ours, t_lib = timer(ours), timer(lib)
            flop = flop1 * L
            print(json.dumps({
                "what": "detail", "model": model, "proj": proj, "shape": [rows, cols], "batch": L, "op": label.strip(),
                "ms": round(t_ours, 4), "cublas_ms": round(t_lib, 4), "speedup": round(t_lib / t_ours, 3),
                "dense_tflops": round(flop / t_ours / 1e9, 1), "cublas_tflops": round(flop / t_lib / 1e9, 1),
            }), flush=True)
        G.check_status(dev)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("what", nargs="?", choices=("summary", "detail", "both"), default="both")
    ap.add_argument("--models", default="1B,3B,8B", help="comma-separated subset of " + ",".join(MODELS))
    ap.add_argument("--batch", type=int, default=8, help="matrices per launch (reduced for the largest shapes)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    args.models = [k.strip() for k in args.models.split(",") if k.strip()]
    for k in args.models:
        if k not in MODELS:
            raise SystemExit(f"unknown model {k!r}; choose from {', '.join(MODELS)}")

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench_syrk.py times CUDA kernels: no GPU visible")
    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import ns_sm100

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    timer = Timer(torch, dev, args.iters, args.warmup)
    if args.what in ("summary", "both"):
        summary(args, torch, G, ns_sm100, timer)
    if args.what in ("detail", "both"):
        detail(args, torch, G, timer)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

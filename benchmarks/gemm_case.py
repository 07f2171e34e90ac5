#!/usr/bin/env python
"""Run one configuration of the tcgen05 GEMM a few times (for timing or for an
``ncu`` capture of a small case).

    python benchmarks/gemm_case.py --m 4096 --n 4096 --k 4096 --batch 2 --b-mn
    python benchmarks/gemm_case.py --m 4096 --k 14336 --batch 2 --symmetric
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _sustain(run, seconds: float, flop_per_call: float) -> dict:
    """Back-to-back launches for about ``seconds``; device time from CUDA events
    around the whole train of launches, SM clock and power read through NVML
    while it runs (reading only)."""
    import statistics
    import threading
    import time

    import torch

    samples: list[tuple[int, float]] = []
    stop = threading.Event()

    def sampler():
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
            while not stop.is_set():
                samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                                pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0))
                time.sleep(0.05)
        except Exception:
            pass

    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run()
    torch.cuda.synchronize()
    t0 = time.time()
    run()
    torch.cuda.synchronize()
    per = max(time.time() - t0, 1e-5)
    calls = max(8, min(20000, int(seconds / per)))
    th = threading.Thread(target=sampler, daemon=True)
    th.start()
    a.record()
    for _ in range(calls):
        run()
    b.record()
    torch.cuda.synchronize()
    stop.set()
    th.join(timeout=1.0)
    ms = a.elapsed_time(b)
    tail = samples[len(samples) // 3:] or samples
    return {
        "calls": calls,
        "seconds": round(ms / 1e3, 3),
        "dense_tflops": round(flop_per_call * calls / ms / 1e9, 1),
        "sm_mhz_median": statistics.median(c for c, _ in tail) if tail else None,
        "power_w_median": round(statistics.median(w for _, w in tail), 1) if tail else None,
    }


def pull_linear_case(args) -> None:
    import torch

    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import pull_linear as PL

    dev = torch.device("cuda", 0)
    M, N, K = args.m, (args.n or args.m), args.k
    torch.manual_seed(0)
    x = (torch.randn(M, K, device=dev) * 0.05).bfloat16()
    w_owner = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    w_local = torch.zeros_like(w_owner)
    flag = torch.full((4,), 1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = []
    for it in range(args.warmup + args.iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        PL.pull_linear(x, w_local, w_owner.data_ptr(), pub_flag=flag[1:], pub_want=1)
        b.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            times.append(a.elapsed_time(b))
    G.check_status(dev)
    ms = sorted(times)[len(times) // 2]
    print(json.dumps({"case": "pull_linear (owner = second buffer on this GPU)", "tokens": M, "out": N, "in": K,
                      "ms": round(ms, 4), "dense_tflops": round(2.0 * M * N * K / ms / 1e9, 1),
                      "weight_mb": round(N * K * 2 / 1e6, 1)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--bn", type=int, default=256)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--symmetric", action="store_true")
    ap.add_argument("--fp16", action="store_true")
    ap.add_argument("--with-c", action="store_true")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--two-cta", action="store_true", help="CTA-pair kernel (cta_group::2, 256 x 256 tiles)")
    ap.add_argument("--quad", action="store_true",
                    help="CTA-quad kernel (two pairs per cluster share their A rows through distributed shared memory)")
    ap.add_argument("--sustain", type=float, default=0.0,
                    help="also run the product back to back for this many seconds and report the sustained rate "
                         "with the SM clock and power sampled meanwhile (the regime inside a training step)")
    ap.add_argument("--cublas", action="store_true", help="also time torch.bmm on the same operands")
    ap.add_argument("--pull-linear", action="store_true",
                    help="the fused publish + forward GEMM (Y = X W^T while W is fetched from its owner) on ONE "
                         "device: the owner's copy is a second buffer of this GPU; --m tokens, --n out, --k in")
    args = ap.parse_args()
    import torch
    if args.pull_linear:
        return pull_linear_case(args)

    from dmuon_b200.ops import gemm as G

    dev = torch.device("cuda", 0)
    dt = torch.float16 if args.fp16 else torch.bfloat16
    M, K, L = args.m, args.k, args.batch
    N = M if (args.symmetric or not args.n) else args.n
    torch.manual_seed(0)
    A = (torch.randn(L, K, M, device=dev) if args.a_mn else torch.randn(L, M, K, device=dev)).mul_(0.05).to(dt)
    if args.symmetric:
        B, b_mn = A, args.a_mn
    else:
        b_mn = args.b_mn
        B = (torch.randn(L, K, N, device=dev) if b_mn else torch.randn(L, N, K, device=dev)).mul_(0.05).to(dt)
    C = torch.randn(L, M, N, device=dev).to(dt) if args.with_c else None
    out = torch.empty(L, M, N, device=dev, dtype=dt)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def run():
        G.gemm(A, B, out, a_mn=args.a_mn, b_mn=b_mn, C=C, beta=0.5 if C is not None else 0.0,
               symmetric=args.symmetric, bn=args.bn, two_cta=2 if args.quad else args.two_cta)

    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    G.check_status(dev)
    ms = sorted(times)[len(times) // 2]
    rec = {"M": M, "N": N, "K": K, "batch": L, "bn": args.bn, "a_mn": args.a_mn, "b_mn": b_mn,
           "symmetric": args.symmetric, "kernel": "quad" if args.quad else ("pair" if args.two_cta else "single"),
           "ms": round(ms, 4), "dense_tflops": round(2.0 * M * N * K * L / ms / 1e9, 1)}
    if args.quad:
        rec["quad_clusters"] = G.quad_max_clusters()
    if args.sustain > 0:
        rec["sustained"] = _sustain(run, args.sustain, 2.0 * M * N * K * L)
    if args.cublas:
        Af = A.transpose(1, 2) if args.a_mn else A
        Bf = B if b_mn else B.transpose(1, 2)
        for _ in range(args.warmup):
            torch.bmm(Af, Bf)
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            torch.bmm(Af, Bf)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        rec["cublas_ms"] = round(sorted(ts)[len(ts) // 2], 4)
        rec["cublas_tflops"] = round(2.0 * M * N * K * L / rec["cublas_ms"] / 1e9, 1)
        if args.sustain > 0:
            rec["cublas_sustained"] = _sustain(lambda: torch.bmm(Af, Bf), args.sustain, 2.0 * M * N * K * L)
    print(json.dumps(rec))


if __name__ == "__main__":
    main()

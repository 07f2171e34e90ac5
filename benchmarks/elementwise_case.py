#!/usr/bin/env python
"""Time one of the HBM-bound kernels on a working set larger than L2 and report
the achieved bandwidth (algorithmic bytes / CUDA-event time) against the copy
bandwidth measured on this machine (MEASURED_PEAKS.json next to the repository
root when present, otherwise the value passed with --peak-gbs).

    python benchmarks/elementwise_case.py --op swiglu_fwd
    python benchmarks/elementwise_case.py --op xent --rows 2048
    python benchmarks/elementwise_case.py --op prologue

Ops: swiglu_fwd, swiglu_bwd, rope, xent, prologue, adamw, clip_sumsq, clip_scale,
cast, peer_prologue, peer_pull, tp_gather, tp_apply.  The peer and
tensor-parallel kernels run on ONE device here: the buffers of the "other
ranks" are other allocations of the same GPU, which exercises the same code
and gives the HBM-side rate (the NVLink-side rate is in bench_comm.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peak_gbs(default: float) -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "of measured"
    except Exception:
        return default, "of fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=("swiglu_fwd", "swiglu_bwd", "rope", "xent", "prologue", "adamw", "clip_sumsq", "clip_scale",
                             "cast", "peer_prologue", "peer_pull", "tp_gather", "tp_apply"))
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--peak-gbs", type=float, default=6650.0)
    args = ap.parse_args()

    import torch

    from dmuon_b200.ops import model_ops as MO
    from dmuon_b200.ops import multi_tensor as MT

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    R, C = args.rows, args.cols
    bf = torch.bfloat16

    if args.op in ("swiglu_fwd", "swiglu_bwd"):
        g = torch.randn(R, C, device=dev, dtype=bf)
        u = torch.randn(R, C, device=dev, dtype=bf)
        d = torch.randn(R, C, device=dev, dtype=bf)
        o1, o2 = torch.empty_like(g), torch.empty_like(g)
        lib = MO._lib()
        st = lambda: MO._stream(g)
        if args.op == "swiglu_fwd":
            run = lambda: lib.dmuon_swiglu_fwd(g.data_ptr(), u.data_ptr(), o1.data_ptr(), g.numel(), 0, 0, st())
            nbytes = 3 * g.numel() * 2
        else:
            run = lambda: lib.dmuon_swiglu_bwd(g.data_ptr(), u.data_ptr(), d.data_ptr(), o1.data_ptr(), o2.data_ptr(),
                                               g.numel(), 0, 0, st())
            nbytes = 5 * g.numel() * 2
    elif args.op == "rope":
        from dmuon_b200.models.llama import rope_tables

        hq, hk, hd = 32, 8, 128
        q = torch.randn(1, R, hq * hd, device=dev, dtype=bf)
        k = torch.randn(1, R, hk * hd, device=dev, dtype=bf)
        cos, sin = rope_tables(R, hd, 500000.0, dev)
        run = lambda: MO._rope_launch(q, k, cos, sin, hd, False)
        nbytes = 2 * (q.numel() + k.numel()) * 2 + 2 * cos.numel() * 4
    elif args.op == "xent":
        V = 128256
        rows = min(R, 2048)
        logits = torch.randn(rows, V, device=dev, dtype=bf)
        labels = torch.randint(0, V, (rows,), device=dev)
        run = lambda: MO.softmax_xent_(logits, labels, 1.0)
        nbytes = 2 * logits.numel() * 2           # read once from HBM, written once (second read served by L2)
    elif args.op == "prologue":
        L, m, n = 4, 4096, 14336
        grads = [torch.randn(m, n, device=dev, dtype=bf) for _ in range(L)]
        moms = [torch.zeros(m, n, device=dev) for _ in range(L)]
        xs = [torch.empty(m, n, device=dev) for _ in range(L)]
        sumsq = torch.zeros(L, device=dev)
        run = lambda: MT.muon_prologue(grads, moms, xs, list(range(L)), sumsq, 0.95, True)
        nbytes = L * m * n * (2 + 4 + 4 + 4)
    elif args.op == "adamw":
        L, numel = 2, 128256 * 4096 // 2
        ps = [torch.randn(numel, device=dev) for _ in range(L)]
        gs = [torch.randn(numel, device=dev) for _ in range(L)]
        ms = [torch.zeros(numel, device=dev) for _ in range(L)]
        vs = [torch.zeros(numel, device=dev) for _ in range(L)]
        run = lambda: MT.adamw(ps, gs, ms, vs, [1] * L, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
        nbytes = L * numel * 4 * 7
    elif args.op == "clip_scale":
        L, m, n = 4, 4096, 14336
        ts = [torch.randn(m, n, device=dev, dtype=bf) for _ in range(L)]
        coef = torch.full((L,), 0.999, device=dev)
        run = lambda: MT.clip_scale(ts, list(range(L)), coef)
        nbytes = L * m * n * 2 * 2
    elif args.op == "cast":
        L, m, n = 4, 4096, 14336
        srcs = [torch.randn(m, n, device=dev) for _ in range(L)]
        dsts = [torch.empty(m, n, device=dev, dtype=bf) for _ in range(L)]
        run = lambda: MT.cast(srcs, dsts)
        nbytes = L * m * n * (4 + 2)
    elif args.op == "peer_prologue":
        # reduce-to-owner fused with the prologue: 4 "ranks" whose gradient arenas are 4 local buffers
        from dmuon_b200.ops import peer as P

        W, L, m, n = 4, 2, 4096, 14336
        arenas = [torch.randn(L * m * n, device=dev, dtype=bf) for _ in range(W)]
        moms = [torch.zeros(m * n, device=dev) for _ in range(L)]
        xs = [torch.empty(m * n, device=dev, dtype=torch.float16) for _ in range(L)]
        sumsq = torch.zeros(L, device=dev)
        pre = torch.ones(L, device=dev)
        run = lambda: P.peer_prologue([a.data_ptr() for a in arenas], [i * m * n for i in range(L)], [m * n] * L, bf,
                                      moms, xs, list(range(L)), sumsq, scale=1.0 / W, mu=0.95, nesterov=True,
                                      xscale=pre)
        nbytes = L * m * n * (2 * W + 4 + 4 + 2)
    elif args.op == "peer_pull":
        from dmuon_b200.ops import peer as P

        n = 256 << 20
        src = torch.empty(n, dtype=torch.uint8, device=dev)
        dst = torch.empty(n, dtype=torch.uint8, device=dev)
        run = lambda: P.peer_pull([src.data_ptr()], [dst.data_ptr()], [n], [0], None, 0, None, dev)
        nbytes = 2 * n
    elif args.op in ("tp_gather", "tp_apply"):
        from dmuon_b200.ops import tp_peer as TP

        T, L, m, n = 2, 2, 4096, 14336
        if args.op == "tp_gather":
            # column shards (the strided case) of L full matrices, read in place, prologue in the same pass
            shards = [[torch.randn(m, n // T, device=dev, dtype=bf) for _ in range(T)] for _ in range(L)]
            moms = [torch.zeros(m, n, device=dev) for _ in range(L)]
            xs = [torch.empty(m, n, device=dev, dtype=torch.float16) for _ in range(L)]
            sumsq = torch.zeros(L, device=dev)
            jobs = [TP.ShardJob(i, shards[i][t].data_ptr(), m, n // T, t * (n // T), n) for i in range(L) for t in range(T)]
            run = lambda: TP.gather_prologue(jobs, bf, moms, xs, list(range(L)), sumsq, mu=0.95, nesterov=True)
            nbytes = L * m * n * (2 + 4 + 4 + 2)
        else:
            delta = [torch.randn(m, n, device=dev) for _ in range(L)]
            masters = [torch.randn(m, n // T, device=dev) for _ in range(L)]
            srcs = [d.data_ptr() + (n // T) * 4 for d in delta]           # the second rank's column slice
            run = lambda: TP.apply_delta(srcs, [n] * L, masters, [0.998] * L)
            nbytes = L * m * (n // T) * (4 + 4 + 4)
    else:
        L, m, n = 4, 4096, 14336
        ts = [torch.randn(m, n, device=dev, dtype=bf) for _ in range(L)]
        acc = torch.zeros(L, device=dev)
        run = lambda: MT.clip_sumsq(ts, list(range(L)), acc)
        nbytes = L * m * n * 2

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
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
    ms = sorted(times)[len(times) // 2]
    peak, label = peak_gbs(args.peak_gbs)
    gbs = nbytes / ms / 1e6
    print(json.dumps({"op": args.op, "ms": round(ms, 4), "algorithmic_gb": round(nbytes / 1e9, 3),
                      "achieved_gbs": round(gbs, 1), "peak_gbs": peak, "fraction": round(gbs / peak, 3), "of": label}))


if __name__ == "__main__":
    main()

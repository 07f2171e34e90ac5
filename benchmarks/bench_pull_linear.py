#!/usr/bin/env python
"""Fused owner-publish + linear on two GPUs against broadcast-then-GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29500 benchmarks/bench_pull_linear.py

Rank 0 owns W; rank 1 times, for Llama-3-8B layer shapes with 8192 tokens:
  fused      one kernel: pull W over NVLink (bulk copies through shared memory)
             while multiplying with the tiles that have arrived
  nccl+gemm  dist.broadcast(W) then F.linear (cuBLAS)
  gemm only  F.linear on a local W, and this package's kernel on a local W
and reports the fraction of the roofline max(FLOPs / measured GEMM peak,
bytes / 770 GB/s measured peer-copy bandwidth).  Device-timed with CUDA events,
L2 flushed between iterations, max over ranks.
"""
from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = [("q/o_proj", 4096, 4096), ("k/v_proj", 1024, 4096), ("gate/up_proj", 14336, 4096), ("down_proj", 4096, 14336)]
TOKENS = 8192
PEAK_TFLOPS = 1410.6      # measured sustained bf16 cuBLAS throughput on this pool
LINK_GBS = 770.0          # measured peer-copy bandwidth per direction


def main():
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    import torch.nn.functional as F

    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import pull_linear as PL

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    assert world >= 2, "run on two GPUs"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    group = dist.group.WORLD

    def timed(fn, iters=8, warmup=3):
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(iters):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        t = torch.tensor(sorted(times)[len(times) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for name, n, k in SHAPES:
        torch.manual_seed(0)
        x = (torch.randn(TOKENS, k, device=dev) * 0.05).bfloat16()
        w = symm_mem.empty(n * k, dtype=torch.bfloat16, device=dev)
        hdl = symm_mem.rendezvous(w, group.group_name)
        w2 = w.view(n, k)
        if rank == 0:
            w2.copy_((torch.randn(n, k, device=dev) * 0.05).bfloat16())
        flags = torch.ones(8, dtype=torch.int32, device=dev)
        owner_ptr = int(hdl.buffer_ptrs[0])
        y = torch.empty(TOKENS, n, device=dev, dtype=torch.bfloat16)
        dist.barrier()

        def fused():
            if rank == 0:
                PL.pull_linear(x, w2, None, out=y)
            else:
                PL.pull_linear(x, w2, owner_ptr, pub_flag=flags, pub_want=1, out=y)

        def nccl_gemm():
            dist.broadcast(w2, src=0)
            F.linear(x, w2)

        def gemm_cublas():
            F.linear(x, w2)

        def gemm_ours():
            PL.pull_linear(x, w2, None, out=y)

        t_fused, t_nccl, t_cublas, t_ours = timed(fused), timed(nccl_gemm), timed(gemm_cublas), timed(gemm_ours)
        if rank == 1:
            ref = F.linear(x.float(), w2.float())
            fused()
            torch.cuda.synchronize()
            err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)
        else:
            err = 0.0
        G.check_status(dev)
        flops = 2.0 * TOKENS * n * k
        roof_ms = max(flops / (PEAK_TFLOPS * 1e9), n * k * 2 / (LINK_GBS * 1e6))
        if rank == 1:
            print(json.dumps({
                "shape": name, "N": n, "K": k, "tokens": TOKENS,
                "fused_ms": round(t_fused, 4), "nccl_bcast_plus_cublas_ms": round(t_nccl, 4),
                "cublas_gemm_only_ms": round(t_cublas, 4), "our_gemm_only_ms": round(t_ours, 4),
                "roofline_ms": round(roof_ms, 4), "fused_fraction_of_roofline": round(roof_ms / t_fused, 3),
                "rel_err": err,
            }), flush=True)
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

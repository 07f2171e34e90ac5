#!/usr/bin/env python
"""Data-plane microbenchmark: how fast one owner's data reaches everybody
(publish) and everybody's data reaches one owner (reduce), per mechanism.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_comm.py
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_comm.py --sizes-mb 16.8,117.4

Sizes default to what one owner sends per layer of Llama-3-8B in bf16: packed
k+v (16.8 MB), q or o (33.6 MB), one MLP matrix (117.4 MB), and a whole
layer's span of one owner at 8 ranks (54.5 MB).

Publish, owner = rank 0, all other ranks end up with the bytes:
  nccl_broadcast      dist.broadcast (what the reference does per owner and layer)
  ce_pull             every reader copies from the owner's symmetric buffer with a copy engine
  sm_pull             every reader copies with a kernel that loads through the peer mapping
  multicast_store     the owner stores once through the NVSwitch multicast mapping (multimem.st)
Reduce, owner = rank 0 ends up with the sum:
  nccl_reduce         dist.reduce(SUM)
  ce_gather_sum       owner copies every peer's slice with copy engines, then one local sum kernel
  sm_peer_sum         owner's kernel loads every peer's slice through the peer mappings and sums
  multicast_reduce    owner reads its span once through the multicast mapping (multimem.ld_reduce)

Every number is device time (CUDA events on the timed rank's stream, ranks
aligned by a barrier first), median of ``--iters``, max over ranks.  GB/s is
payload bytes / time; ``of_link`` divides by the measured peer-copy rate of this
pool (770 GB/s per direction per GPU).  For publish with N readers the owner's
egress is (N-1) x payload unless the switch replicates; for reduce the owner's
ingress is (N-1) x payload unless the switch reduces.

Counterpart of the reference's ``benchmarks/bench_comm.py:36`` (all-gather vs
broadcast vs concurrent broadcasts through NCCL only).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 770.0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="16.8,33.6,54.5,117.4")
    ap.add_argument("--iters", type=int, default=9)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import peer as P

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    group = dist.group.WORLD
    sizes = [int(float(x) * 1e6) // 4096 * 4096 for x in args.sizes_mb.split(",")]
    nmax = max(sizes) // 2

    sym = symm_mem.empty(nmax, dtype=torch.bfloat16, device=dev)
    sym.normal_()
    flags = symm_mem.empty(64, dtype=torch.int32, device=dev)
    flags.zero_()
    torch.cuda.synchronize()
    hdl = symm_mem.rendezvous(sym, group.group_name)
    fh = symm_mem.rendezvous(flags, group.group_name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
    status = G.status_buffer(dev)
    local_buf = torch.empty(nmax, dtype=torch.bfloat16, device=dev)
    stage = torch.empty(max(world - 1, 1) * nmax, dtype=torch.bfloat16, device=dev)
    out32 = torch.empty(nmax, dtype=torch.float32, device=dev)
    del fh

    def timed(fn) -> float:
        """Median device ms of ``fn`` on this rank (0 when this rank does nothing), max over ranks."""
        ts = []
        for it in range(args.warmup + args.iters):
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                ts.append(a.elapsed_time(b))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows = []
    for nbytes in sizes:
        n = nbytes // 2
        view = sym[:n]
        rec = {"payload_mb": round(nbytes / 1e6, 1), "world": world}

        # ---------------- publish ----------------
        rec["nccl_broadcast_ms"] = timed(lambda: dist.broadcast(view, src=0))
        rec["ce_pull_ms"] = timed(lambda: P.copy_async(local_buf.data_ptr(), ptrs[0], nbytes, dev) if rank != 0 else None)
        rec["sm_pull_ms"] = timed(
            lambda: P.peer_pull([ptrs[0]], [local_buf.data_ptr()], [nbytes], [0], None, 0, status, dev) if rank != 0 else None)
        if mc:
            rec["multicast_store_ms"] = timed(
                lambda: P.multicast_broadcast([local_buf.data_ptr()], [mc], [nbytes], dev) if rank == 0 else None)
        # ---------------- reduce ----------------
        rec["nccl_reduce_ms"] = timed(lambda: dist.reduce(view, dst=0))

        def ce_gather_sum():
            if rank != 0:
                return
            k = 0
            for r in range(world):
                if r != rank:
                    P.copy_async(stage.data_ptr() + k * nbytes, ptrs[r], nbytes, dev)
                    k += 1
            bases = [ptrs[0]] + [stage.data_ptr() + i * nbytes for i in range(world - 1)]
            P.peer_prologue(bases, [0], [n], torch.bfloat16, [None], [out32[:n]], [0], None, scale=1.0 / world, mu=0.0,
                            nesterov=False, status=status)

        rec["ce_gather_sum_ms"] = timed(ce_gather_sum)
        rec["sm_peer_sum_ms"] = timed(
            lambda: P.peer_prologue(ptrs, [0], [n], torch.bfloat16, [None], [out32[:n]], [0], None, scale=1.0 / world,
                                    mu=0.0, nesterov=False, status=status) if rank == 0 else None)
        if mc:
            rec["multicast_reduce_ms"] = timed(
                lambda: P.multicast_reduce([mc], [local_buf.data_ptr()], [nbytes], torch.bfloat16, dev) if rank == 0 else None)
            rec["multicast_reduce_16cta_ms"] = timed(
                lambda: P.multicast_reduce([mc], [local_buf.data_ptr()], [nbytes], torch.bfloat16, dev,
                                           blocks_per_tensor=16) if rank == 0 else None)
        for k in [k for k in rec if k.endswith("_ms")]:
            ms = rec[k]
            rec[k] = round(ms, 4)
            if ms > 0:
                gbs = nbytes / ms / 1e6
                rec[k[:-3] + "_gbs"] = round(gbs, 1)
                rec[k[:-3] + "_of_link"] = round(gbs / LINK_GBS, 3)
        rows.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
    G.check_status(dev)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

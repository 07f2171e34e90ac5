#!/usr/bin/env python
"""Optimizer benchmark: where the time of ``Muon.step()`` goes.

    python benchmarks/bench_optimizer.py phase                       # 1 GPU
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_optimizer.py phase --model llama3-8b
    python benchmarks/bench_optimizer.py shapes                      # per-shape Newton-Schulz + update, 1 GPU

``phase`` trains a Llama-shaped decoder under FSDP2 + dedicated Muon and prints,
per step, the device time of forward+backward and of every phase of the
optimizer step (waiting for gradients, Muon, dedicated AdamW, publish, AdamW
on FSDP shards), taken from ``Muon(record_step_profile=True)`` /
``consume_last_step_profile()``; max over ranks.

``shapes`` times the batched update of one shape at a time (momentum, Nesterov,
norm, Newton-Schulz products, weight update) on synthetic gradients, for the
matrix shapes and per-owner batch sizes of Llama-3-8B on 1 and 8 GPUs, and
converts to executed TFLOP/s (symmetric products counted at the tiles computed).

Counterpart of the reference's ``benchmarks/bench_optimizer.py:65`` (phase
comparison and detailed step breakdown, host timers around synchronisations).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

MODELS = {
    "llama3-8b": dict(d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128, ffn_hidden=14336,
                      vocab_size=128256, seq=8192, mb=1),
    "llama3.2-3b": dict(d_model=3072, n_layers=28, n_heads=24, n_kv_heads=8, head_dim=128, ffn_hidden=8192,
                        vocab_size=128256, seq=4096, mb=2),
    "small": dict(d_model=1024, n_layers=4, n_heads=8, n_kv_heads=4, head_dim=128, ffn_hidden=4096,
                  vocab_size=32000, seq=1024, mb=2),
}


def phase(args) -> None:
    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    dims = dict(MODELS[args.model])
    seq, mb = dims.pop("seq"), dims.pop("mb")
    torch.manual_seed(42)
    with torch.device(dev):
        model = LlamaModel(LlamaConfig(rope_theta=500000.0, **dims))
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, compute_dtype=torch.bfloat16,
                          reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3, weight_decay=0.1, record_step_profile=True)
    gen = torch.Generator().manual_seed(7 + rank)
    batches = [torch.randint(0, dims["vocab_size"], (mb, seq + 1), generator=gen).to(dev) for _ in range(2)]
    rows = []
    for step in range(args.warmup + args.steps):
        b = batches[step % 2]
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        opt.zero_grad()
        model(b[:, :-1], labels=b[:, 1:]).backward()
        e1.record()
        opt.step()
        e2.record()
        torch.cuda.synchronize()
        prof = opt.consume_last_step_profile() or {}
        if step >= args.warmup:
            rows.append({"fwd_bwd_ms": e0.elapsed_time(e1), "optimizer_ms": e1.elapsed_time(e2), **prof})
    keys = sorted({k for r in rows for k in r})
    med = torch.tensor([statistics.median(r.get(k, 0.0) for r in rows) for k in keys], device=dev, dtype=torch.float64)
    dist.all_reduce(med, op=dist.ReduceOp.MAX)
    if rank == 0:
        out = {"bench": "optimizer_phase", "model": args.model, "world": world, "seq": seq, "micro_batch": mb,
               "steps": args.steps, "median_ms_max_over_ranks": {k: round(float(v), 3) for k, v in zip(keys, med.tolist())}}
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def ns_flops(m0: int, n0: int, n_coef: int = 5, restarts=(2,)) -> tuple[float, float]:
    """(dense-equivalent, executed) FLOPs of one Gram-form Newton-Schulz with the
    step-polynomial recurrence: per step P = cR^2+bR+aI, Q = PQ (not in the first
    step of a window), R = (RP)P (not before a restart or at the end); restarts add
    an apply and a Gram.  Symmetric m x m products execute 136/256 of their tiles."""
    m, n = min(m0, n0), max(m0, n0)
    mmm, mmn_sym, mmn = 0, 1, 1          # initial Gram (symmetric, K = n), final apply
    q_open = False
    for i in range(n_coef):
        if i in restarts and i != 0:
            mmn += 1
            mmn_sym += 1
            q_open = False
        mmm += 1                           # P
        if q_open:
            mmm += 1                       # Q = P Q
        q_open = True
        if i < n_coef - 1 and (i + 1) not in restarts:
            mmm += 2                       # R = (R P) P
    dense = 2.0 * (mmm * m**3 + (mmn_sym + mmn) * m * m * n)
    executed = 2.0 * (0.53125 * mmm * m**3 + (0.53125 * mmn_sym + mmn) * m * m * n)
    return dense, executed


def shapes(args) -> None:
    import torch

    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import ns_sm100
    from dmuon_b200.optim.muon import muon_update_scale
    from dmuon_b200.optim.newton_schulz import DEFAULT_COEFFICIENTS, DEFAULT_RESTART_ITERATIONS

    dev = torch.device("cuda", 0)
    # (rows, cols, matrices per owner at 8 GPUs, at 1 GPU) for Llama-3-8B
    cases = [(4096, 4096, 8, 64), (1024, 4096, 8, 64), (14336, 4096, 8, 64), (4096, 14336, 4, 32)]
    for rows, cols, l8, l1 in cases:
        for L in sorted({l8, min(l1, ns_sm100.max_batch(rows, cols))}):
            torch.manual_seed(0)
            grads = [torch.randn(rows, cols, device=dev, dtype=torch.bfloat16) * 0.01 for _ in range(L)]
            moms = [torch.zeros(rows, cols, device=dev) for _ in range(L)]
            masters = [torch.randn(rows, cols, device=dev) * 0.02 for _ in range(L)]
            pubs = [torch.empty(rows, cols, device=dev, dtype=torch.bfloat16) for _ in range(L)]

            def run():
                ns_sm100.muon_update_batched(
                    grads, moms, masters, mu=0.95, nesterov=True, coefs=DEFAULT_COEFFICIENTS,
                    restarts=DEFAULT_RESTART_ITERATIONS, formulation="gram", lr=0.02, weight_decay=0.1,
                    update_scale=muon_update_scale((rows, cols)), publish=pubs)

            for _ in range(2):
                run()
            torch.cuda.synchronize()
            ts = []
            for _ in range(args.steps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                run()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            G.check_status(dev)
            ms = statistics.median(ts)
            dense, executed = ns_flops(rows, cols)
            print(json.dumps({
                "bench": "optimizer_shapes", "rows": rows, "cols": cols, "batch": L, "ms": round(ms, 3),
                "ms_per_matrix": round(ms / L, 4), "dense_tflops": round(dense * L / ms / 1e9, 1),
                "executed_tflops": round(executed * L / ms / 1e9, 1), "gemm_cluster": G.cluster_mode(),
            }), flush=True)
            del grads, moms, masters, pubs
            ns_sm100.release_workspaces()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=("phase", "shapes"))
    ap.add_argument("--model", choices=tuple(MODELS), default="llama3-8b")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    (phase if args.what == "phase" else shapes)(args)


if __name__ == "__main__":
    main()

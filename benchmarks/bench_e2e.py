#!/usr/bin/env python
"""Dedicated ownership against the obvious alternative, on the same model and ranks.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_e2e.py
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_e2e.py --cpu --layers 2 --width 128

Three arms train the same decoder (``dmuon_b200.models``) on the same synthetic
batches:

``redundant``  plain FSDP2 for every parameter; before the update every rank
               all-gathers the full gradient of every matrix and runs the SAME
               Newton-Schulz iteration on it (N times the orthogonalisation work,
               one all-gather per matrix), then updates its own shard.  This is what
               Muon under FSDP2 looks like without ownership.
``owned``      ``dedicate_params`` + ``Muon``: every matrix has one owner; gradients
               are reduced to it, it orthogonalises once, the new weights are
               published before the next forward.
``adamw``      FSDP2 + fused AdamW, the usual yardstick ("Muon overhead").

All arms use this package's Newton-Schulz (``dmuon_b200.newton_schulz``: sm_100a
kernels on a GPU, PyTorch on CPU), so the difference between ``redundant`` and
``owned`` is the placement, not the kernel.  Times are CUDA events on the device
(wall clock on CPU), max over ranks, after warm-up; one JSON line per arm plus a
summary line.  Counterpart of the reference's ``benchmarks/bench_e2e.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def _pred(name, p):
    return "proj" in name and p.ndim == 2


def build_model(args, device):
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    cfg = LlamaConfig(vocab_size=args.vocab, d_model=args.width, n_layers=args.layers, n_heads=args.heads,
                      n_kv_heads=args.kv_heads or args.heads, head_dim=args.width // args.heads,
                      ffn_hidden=args.ffn or 4 * args.width, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(device):
        return cfg, LlamaModel(cfg)


def shard(model, mesh, on_gpu):
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16) if on_gpu else MixedPrecisionPolicy()
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp, reshard_after_forward=False)
    fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=False)


class RedundantMuon:
    """Muon for FSDP2-sharded matrices without ownership: every rank rebuilds the
    full gradient and orthogonalises it; AdamW for everything else."""

    def __init__(self, model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-3, ns_steps=5):
        import dmuon_b200 as dmuon

        self.ns = dmuon.newton_schulz
        self.lr, self.mu, self.wd, self.ns_steps = lr, momentum, weight_decay, ns_steps
        named = list(model.named_parameters())
        self.matrices = [p for n, p in named if _pred(n, p)]
        rest = [p for n, p in named if not _pred(n, p)]
        self.rest = torch.optim.AdamW(rest, lr=adamw_lr, weight_decay=0.01, fused=rest[0].is_cuda) if rest else None
        self.bufs: dict[int, torch.Tensor] = {}

    def zero_grad(self, set_to_none=True):
        for p in self.matrices:
            p.grad = None
        if self.rest is not None:
            self.rest.zero_grad(set_to_none=set_to_none)

    @torch.no_grad()
    def step(self):
        from torch.distributed.tensor import DTensor

        for p in self.matrices:
            if p.grad is None:
                continue
            g = p.grad
            full = g.full_tensor() if isinstance(g, DTensor) else g          # the all-gather every rank pays
            buf = self.bufs.get(id(p))
            if buf is None:
                buf = self.bufs[id(p)] = torch.zeros_like(full, dtype=torch.float32)
            buf.mul_(self.mu).add_(full.float())
            u = full.float().add(buf, alpha=self.mu)
            o = self.ns(u, steps=self.ns_steps)                              # ... and the work every rank repeats
            scale = 0.2 * max(u.shape) ** 0.5
            local = p._local_tensor if isinstance(p, DTensor) else p
            rows = local.shape[0]
            r0 = dist.get_rank(p.device_mesh.get_group()) * rows if isinstance(p, DTensor) else 0
            piece = o[r0 : r0 + rows]
            if piece.shape[0] < rows:                                        # padded last shard
                pad = torch.zeros(rows - piece.shape[0], *piece.shape[1:], dtype=piece.dtype, device=piece.device)
                piece = torch.cat((piece, pad))
            local.mul_(1.0 - self.lr * self.wd).add_(piece.to(local.dtype), alpha=-self.lr * scale)
        if self.rest is not None:
            self.rest.step()


def build_arm(arm, args, device, mesh):
    import dmuon_b200 as dmuon

    on_gpu = device.type == "cuda"
    cfg, model = build_model(args, device)
    if arm == "owned":
        dmuon.dedicate_params(model, mesh, _pred, compute_dtype=torch.bfloat16 if on_gpu else None,
                              reshard_after_forward=False)
        shard(model, mesh, on_gpu)
        opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-3, ns_steps=5,
                         first_step_progress_log=False)
    elif arm == "redundant":
        shard(model, mesh, on_gpu)
        opt = RedundantMuon(model)
    else:
        shard(model, mesh, on_gpu)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=on_gpu)
    return cfg, model, opt


def time_arm(arm, args, device, mesh, rank, world):
    on_gpu = device.type == "cuda"
    cfg, model, opt = build_arm(arm, args, device, mesh)
    gen = torch.Generator().manual_seed(11 + rank)
    pool = [torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=gen) for _ in range(4)]
    pool = [b.pin_memory() for b in pool] if on_gpu else pool

    def step(i):
        b = pool[i % len(pool)].to(device, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        loss = model(b[:, :-1], labels=b[:, 1:])
        loss.backward()
        opt.step()
        return loss

    for i in range(args.warmup):
        step(i)
    if on_gpu:
        torch.cuda.synchronize()
    dist.barrier()
    if on_gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for i in range(args.steps):
        loss = step(args.warmup + i)
    if on_gpu:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([ms, float(loss.detach())], dtype=torch.float64, device=device)
    worst = t.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    peak = torch.cuda.max_memory_allocated(device) / 2**30 if on_gpu else 0.0
    out = {"arm": arm, "ms_per_step": round(float(worst[0]), 3), "loss": round(float(t[1]) / world, 4),
           "peak_mem_gib": round(peak, 2), "ranks": world}
    del model, opt
    if on_gpu:
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(device)
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--arms", default="redundant,owned,adamw")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--ffn", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    from torch.distributed.device_mesh import init_device_mesh

    use_cuda = torch.cuda.is_available() and not args.cpu
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp",))

    results = {}
    for arm in [a.strip() for a in args.arms.split(",") if a.strip()]:
        if arm not in ("redundant", "owned", "adamw"):
            raise SystemExit(f"unknown arm {arm!r}")
        results[arm] = time_arm(arm, args, device, mesh, rank, world)
        if rank == 0:
            print(json.dumps(results[arm]), flush=True)
    if rank == 0:
        summary = {"summary": True, "ranks": world, "device": device.type}
        if "owned" in results and "redundant" in results:
            summary["owned_vs_redundant_speedup"] = round(results["redundant"]["ms_per_step"] / results["owned"]["ms_per_step"], 3)
        if "owned" in results and "adamw" in results:
            summary["owned_vs_adamw_step_ratio"] = round(results["owned"]["ms_per_step"] / results["adamw"]["ms_per_step"], 3)
        print(json.dumps(summary), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

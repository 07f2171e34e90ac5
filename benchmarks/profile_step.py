#!/usr/bin/env python
"""Capture a torch-profiler trace of a few training steps and summarise it.

    # one GPU, Llama-3.2-3B shapes
    python benchmarks/profile_step.py --model llama3.2-3b --steps 2
    # 8 GPUs, Llama-3-8B, one trace per rank under ./traces
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/profile_step.py --model llama3-8b
    # no GPU: the tiny decoder over gloo (checks the tool itself)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/profile_step.py --cpu --model tiny

Every rank trains the decoder of ``dmuon_b200.models`` with dedicated-ownership
Muon (or, with ``--optimizer adamw``, FSDP2 + fused AdamW) for ``--warmup`` steps,
then records ``--steps`` steps with ``torch.profiler`` (CPU + CUDA activities, no
shapes, no stacks: the overhead stays small), writes ``<out>/<tag>_rank<r>.trace.json``
(open it in Perfetto / chrome://tracing) and prints what ``benchmarks/analyze_trace.py``
finds in rank 0's trace: device time per kernel family, how much communication was
hidden behind compute, the longest device-idle gaps, the ``dmuon.*`` ranges.

Numbers printed under a profiler are for orientation, never benchmark values
(``bench.py`` times without one).  Counterpart of the reference's
``benchmarks/profile_llm_3b.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

MODELS = {
    # name: (vocab, width, layers, heads, kv heads, head dim, ffn, default batch, default sequence)
    "tiny": (1024, 256, 4, 4, 4, 64, 1024, 4, 128),
    "llama3.2-1b": (128256, 2048, 16, 32, 8, 64, 8192, 4, 4096),
    "llama3.2-3b": (128256, 3072, 28, 24, 8, 128, 8192, 2, 4096),
    "llama3-8b": (128256, 4096, 32, 32, 8, 128, 14336, 1, 8192),
}


def build(args, device, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    vocab, d, layers, heads, kv, hd, ffn, _b, _s = MODELS[args.model]
    cfg = LlamaConfig(vocab_size=vocab, d_model=d, n_layers=layers, n_heads=heads, n_kv_heads=kv, head_dim=hd,
                      ffn_hidden=ffn, rope_theta=500000.0)
    torch.manual_seed(0)
    with torch.device(device):
        model = LlamaModel(cfg)
    mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp",))
    on_gpu = device.type == "cuda"
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16) if on_gpu else MixedPrecisionPolicy()
    if args.optimizer == "muon":
        dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2,
                              compute_dtype=torch.bfloat16 if on_gpu else None,
                              reshard_after_forward=bool(args.reshard_after_forward))
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp, reshard_after_forward=bool(args.reshard_after_forward))
    fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=bool(args.reshard_after_forward))
    if args.optimizer == "muon":
        opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1, first_step_progress_log=False)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=on_gpu)
    return cfg, model, opt


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", choices=sorted(MODELS), default="llama3.2-3b")
    ap.add_argument("--optimizer", choices=("muon", "adamw"), default="muon")
    ap.add_argument("--batch", type=int, default=0, help="micro-batch per rank (0: the model's default)")
    ap.add_argument("--seq", type=int, default=0, help="sequence length (0: the model's default)")
    ap.add_argument("--steps", type=int, default=2, help="profiled steps")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reshard-after-forward", action="store_true")
    ap.add_argument("--cpu", action="store_true", help="gloo on CPU (tool check; use --model tiny)")
    ap.add_argument("--out", type=Path, default=Path("traces"))
    ap.add_argument("--tag", default="")
    ap.add_argument("--gap-us", type=float, default=200.0)
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available() and not args.cpu
    if "RANK" not in os.environ:
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    cfg, model, opt = build(args, device, world)
    batch = args.batch or MODELS[args.model][7]
    seq = args.seq or MODELS[args.model][8]
    gen = torch.Generator().manual_seed(7 + rank)
    ids = torch.randint(0, cfg.vocab_size, (batch, seq + 1), generator=gen)
    ids = ids.pin_memory() if use_cuda else ids

    def step():
        b = ids.to(device, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        loss = model(b[:, :-1], labels=b[:, 1:])
        loss.backward()
        opt.step()
        return loss

    for _ in range(args.warmup):
        step()
    if use_cuda:
        torch.cuda.synchronize()
    dist.barrier()

    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if use_cuda else [])
    with profile(activities=acts, record_shapes=False, with_stack=False) as prof:
        for _ in range(args.steps):
            loss = step()
        if use_cuda:
            torch.cuda.synchronize()
    args.out.mkdir(parents=True, exist_ok=True)
    tag = args.tag or f"{args.model}_{args.optimizer}_n{world}"
    path = args.out / f"{tag}_rank{rank}.trace.json"
    prof.export_chrome_trace(str(path))
    dist.barrier()
    if rank == 0:
        import analyze_trace

        summary = analyze_trace.analyze(analyze_trace.load_events(path), args.gap_us)
        summary["per_step_note"] = f"{args.steps} profiled steps; divide the totals by that"
        print(f"trace: {path}  (loss {float(loss.detach()):.4f})")
        print(analyze_trace.format_report(summary), end="")
        (args.out / f"{tag}_rank0.summary.json").write_text(json.dumps(summary, indent=2) + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

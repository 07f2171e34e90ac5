#!/usr/bin/env python
"""Data-parallel training with dedicated-ownership Muon: the smallest complete program.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basic_dp.py          # 4 GPUs, NCCL
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/basic_dp.py --cpu    # no GPU: gloo

What it shows, in the order a training script needs it:

1. ``dedicate_params`` BEFORE ``fully_shard``: every selected matrix gets one owner rank
   (balanced by optimizer cost); FSDP2 then only sees what is left.
2. ``Muon``: Newton-Schulz updates for the owned matrices, AdamW for everything else, one optimizer.
3. gradient clipping over the owned Muon gradients, a learning-rate schedule through ``param_groups``.
4. a checkpoint in the single-GPU layout (full tensors by parameter name) and a resume from it.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import dmuon_b200 as dmuon  # noqa: E402


class Block(nn.Module):
    def __init__(self, d: int, ff: int):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.gate_proj = nn.Linear(d, ff, bias=False)
        self.up_proj = nn.Linear(d, ff, bias=False)
        self.down_proj = nn.Linear(ff, d, bias=False)

    def forward(self, x):
        h = self.norm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Net(nn.Module):
    def __init__(self, vocab: int = 512, d: int = 256, ff: int = 1024, n_layers: int = 4):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(Block(d, ff) for _ in range(n_layers))
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids, labels):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x)
        return F.cross_entropy(self.head(x).flatten(0, 1).float(), labels.flatten())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="gloo on CPU instead of NCCL on GPUs")
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available() and not args.cpu
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp",))

    torch.manual_seed(0)                                    # identical initial weights on every rank
    model = Net().to(device)

    # 1. ownership: the 2-D projection matrices go to Muon, one owner each
    owners = dmuon.dedicate_params(
        model, mesh, lambda name, p: "proj" in name and p.ndim == 2,
        compute_dtype=torch.bfloat16 if use_cuda else None,   # forward/backward copies; masters stay fp32
        reshard_after_forward=False,                          # keep the published copy for backward ("Z2")
    )
    # the same compute dtype for what FSDP2 manages, so that activations and dedicated weights agree
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32) if use_cuda else MixedPrecisionPolicy()
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)               # embedding, head, norms: ordinary FSDP2
    if rank == 0:
        per_rank = [sum(1 for o in owners.values() if o == r) for r in range(world)]
        print(f"{len(owners)} dedicated matrices, owners per rank: {per_rank}")

    # 2. one optimizer for both kinds of parameters
    opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5, adamw_lr=1e-3)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: min(1.0, (s + 1) / 5))

    gen = torch.Generator().manual_seed(100 + rank)          # every rank trains on its own data:
    pool = [torch.randint(0, 512, (8, 65), generator=gen).to(device) for _ in range(4)]   # a tiny fixed set
    counter = [0]

    def batch():
        ids = pool[counter[0] % len(pool)]
        counter[0] += 1
        return ids[:, :-1], ids[:, 1:]

    def train_step():
        ids, labels = batch()
        loss = model(ids, labels)
        opt.zero_grad()
        loss.backward()
        dmuon.clip_grad_norm_(opt, 1.0)                       # 3. global norm of the owned Muon gradients
        opt.step()
        sched.step()
        return loss

    for step in range(args.steps):
        loss = train_step()
        if step % 5 == 0:
            lt = loss.detach().float().clone()
            dist.all_reduce(lt)
            if rank == 0:
                print(f"step {step:3d}  loss {float(lt) / world:.4f}  lr {opt.param_groups[0]['lr']:.4f}")

    # 4. checkpoint: plain {name: full tensor} dictionaries, identical to a single-GPU state_dict
    # (rank0_only=True, the default, keeps the data on rank 0 only: that is what one writes to disk;
    # here every rank keeps a copy because the resume below reads it on every rank)
    model_sd = dmuon.get_model_state_dict(model, rank0_only=False)
    optim_sd = dmuon.get_optimizer_state_dict(model, opt, rank0_only=False)
    if rank == 0:
        n_bytes = sum(t.numel() * t.element_size() for t in model_sd.values())
        print(f"checkpoint: {len(model_sd)} tensors, {n_bytes / 2**20:.1f} MiB; "
              f"optimizer sections {sorted(optim_sd)}")
    # resume (here: into the same objects) and keep training
    dmuon.set_model_state_dict(model, model_sd)
    dmuon.set_optimizer_state_dict(model, opt, optim_sd)
    loss = train_step()
    if rank == 0:
        print(f"after resume: loss {float(loss.detach()):.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

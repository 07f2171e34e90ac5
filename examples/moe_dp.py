#!/usr/bin/env python
"""Mixture of experts under dedicated ownership.

    DMUON_ZERO_FILL_MISSING_GRADS=1 torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/moe_dp.py
    DMUON_ZERO_FILL_MISSING_GRADS=1 torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/moe_dp.py --cpu

Every expert's three projection matrices are dedicated Muon matrices (one owner each, balanced over all ranks); the router,
embeddings and norms stay with FSDP2 and AdamW.  The hook boundary is the decoder layer, which every rank calls whichever
experts its tokens choose.  Because routing depends on the data, an expert can be idle on a rank in a step; the switch
above makes such an expert contribute zeros, so that all ranks send the same buffers (see
docs/guides/custom-hook-boundaries.md).  The program prints how the expert matrices are spread over the owners and the loss
as it falls.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import dmuon_b200 as dmuon  # noqa: E402
from dmuon_b200.models.moe import MoEConfig, MoEModel  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available() and not args.cpu
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    mesh = init_device_mesh(device.type, (world,), mesh_dim_names=("dp",))

    cfg = MoEConfig.tiny(n_experts=args.experts, top_k=args.top_k, balance_coef=0.01)
    torch.manual_seed(0)
    model = MoEModel(cfg).to(device)
    owners = dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2,
                                   compute_dtype=torch.bfloat16 if use_cuda else None, reshard_after_forward=False)
    # the same compute dtype for what FSDP2 manages, so that activations and dedicated weights agree
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32) if use_cuda else MixedPrecisionPolicy()
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=3e-3, first_step_progress_log=False)
    if rank == 0:
        per_owner = [0] * world
        for p, o in owners.items():
            per_owner[int(o)] += 1
        print(f"{len(owners)} dedicated matrices ({cfg.n_layers} layers x ({cfg.n_experts} experts x 3 + 4 attention)), "
              f"per owner: {per_owner}")

    gen = torch.Generator().manual_seed(100 + rank)
    pool = [torch.randint(0, cfg.vocab_size, (4, 33), generator=gen).to(device) for _ in range(4)]
    for step in range(args.steps):
        ids = pool[step % len(pool)]
        opt.zero_grad()
        loss = model(ids[:, :-1], labels=ids[:, 1:])
        loss.backward()
        dmuon.clip_grad_norm_(opt, 1.0)
        opt.step()
        if step % 5 == 0 or step == args.steps - 1:
            lt = loss.detach().float().clone()
            dist.all_reduce(lt)
            if rank == 0:
                print(f"step {step:3d}  loss {float(lt) / world:.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

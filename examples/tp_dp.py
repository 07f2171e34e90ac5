#!/usr/bin/env python
"""Tensor parallel x data parallel training with dedicated-ownership Muon.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/tp_dp.py            # 4 GPUs: DP 2 x TP 2
    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/tp_dp.py --cpu      # gloo, no GPU

The attention and MLP projections are sharded over the ``tp`` mesh dimension with PyTorch's DTensor plans
(column-parallel q/k/v/gate/up, row-parallel o/down).  ``dedicate_params`` recognises those DTensors by
itself: a sharded matrix gets a data-parallel owner (who receives the reduced gradient of its shard
column) AND a tensor-parallel owner inside that rank's TP group.  At optimizer time the TP owner gathers
the shards of the reduced gradient, orthogonalises the FULL matrix and scatters the pre-scaled update
back, so Newton-Schulz sees the same matrix it would see without tensor parallelism.

``--distributed-gram`` switches to the variant where the TP owner broadcasts the small Gram factors and
every TP rank applies them to its own shard (cheaper when the factors are much smaller than the matrix).
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
from torch.distributed.fsdp import fully_shard
from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import dmuon_b200 as dmuon  # noqa: E402


class Attention(nn.Module):
    def __init__(self, d: int, n_heads: int, n_kv_heads: int):
        super().__init__()
        self.hd = d // n_heads
        self.groups = n_heads // n_kv_heads
        self.q_proj = nn.Linear(d, n_heads * self.hd, bias=False)
        self.k_proj = nn.Linear(d, n_kv_heads * self.hd, bias=False)
        self.v_proj = nn.Linear(d, n_kv_heads * self.hd, bias=False)
        self.o_proj = nn.Linear(n_heads * self.hd, d, bias=False)

    def forward(self, x):
        b, s, _ = x.shape
        # -1 head counts: under tensor parallelism each rank sees its share of the heads
        q = self.q_proj(x).view(b, s, -1, self.hd).transpose(1, 2)
        k = self.k_proj(x).view(b, s, -1, self.hd).transpose(1, 2)
        v = self.v_proj(x).view(b, s, -1, self.hd).transpose(1, 2)
        k = k.repeat_interleave(self.groups, dim=1)
        v = v.repeat_interleave(self.groups, dim=1)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(y.transpose(1, 2).reshape(b, s, -1))


class MLP(nn.Module):
    def __init__(self, d: int, ff: int):
        super().__init__()
        self.gate_proj = nn.Linear(d, ff, bias=False)
        self.up_proj = nn.Linear(d, ff, bias=False)
        self.down_proj = nn.Linear(ff, d, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, d, ff, n_heads, n_kv_heads):
        super().__init__()
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.attn = Attention(d, n_heads, n_kv_heads)
        self.mlp = MLP(d, ff)

    def forward(self, x):
        x = x + self.attn(self.n1(x))
        return x + self.mlp(self.n2(x))


class Net(nn.Module):
    def __init__(self, vocab=512, d=256, ff=1024, n_layers=4, n_heads=4, n_kv_heads=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(Block(d, ff, n_heads, n_kv_heads) for _ in range(n_layers))
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids, labels):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x)
        return F.cross_entropy(self.head(x).flatten(0, 1).float(), labels.flatten())


TP_PLAN = {
    "attn.q_proj": ColwiseParallel(), "attn.k_proj": ColwiseParallel(), "attn.v_proj": ColwiseParallel(),
    "attn.o_proj": RowwiseParallel(),
    "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel(),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--distributed-gram", action="store_true")
    args = ap.parse_args()

    use_cuda = torch.cuda.is_available() and not args.cpu
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if world % args.tp:
        raise SystemExit(f"world size {world} is not a multiple of --tp {args.tp}")
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    mesh = init_device_mesh(device.type, (world // args.tp, args.tp), mesh_dim_names=("dp", "tp"))
    dp_mesh, tp_mesh = mesh["dp"], mesh["tp"]

    torch.manual_seed(0)
    model = Net().to(device)
    for layer in model.layers:                               # 1. tensor parallelism first
        parallelize_module(layer, tp_mesh, TP_PLAN)
    owners = dmuon.dedicate_params(                          # 2. then ownership over the data-parallel mesh
        model, dp_mesh, lambda name, p: "proj" in name and p.ndim == 2, reshard_after_forward=False,
    )
    for layer in model.layers:                               # 3. FSDP2 for the rest
        fully_shard(layer, mesh=dp_mesh)
    fully_shard(model, mesh=dp_mesh)
    opt = dmuon.Muon(model, lr=0.02, weight_decay=0.1, adamw_lr=1e-3, tp_distributed_gram=args.distributed_gram)

    if rank == 0:
        tp_owned = sum(1 for dp in dmuon.get_dedicated_params(model) if dp.tp_group is not None)
        print(f"mesh dp={world // args.tp} x tp={args.tp}: {len(owners)} dedicated matrices, {tp_owned} tensor-parallel")

    # ranks of one TP group must see the same batch; data-parallel ranks see different ones
    gen = torch.Generator().manual_seed(100 + dp_mesh.get_local_rank())
    pool = [torch.randint(0, 512, (8, 65), generator=gen).to(device) for _ in range(4)]
    for step in range(args.steps):
        ids = pool[step % len(pool)]
        loss = model(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        dmuon.clip_grad_norm_(opt, 1.0)
        opt.step()
        if step % 5 == 0:
            lt = loss.detach().float().clone()
            dist.all_reduce(lt)
            if rank == 0:
                print(f"step {step:3d}  loss {float(lt) / world:.4f}")
    sd = dmuon.get_model_state_dict(model)                   # full (unsharded) tensors on rank 0
    if rank == 0:
        w = sd["layers.0.attn.q_proj.weight"]
        print(f"checkpoint holds the full q_proj: {tuple(w.shape)}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

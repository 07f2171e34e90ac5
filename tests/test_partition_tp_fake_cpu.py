"""Partition of a 3-D job (replicate 2 x shard 4 x TP 2 = 16 ranks) checked in
ONE process with PyTorch's ``fake`` process-group backend: real DeviceMesh and
DTensor objects, no communication.  Pins tensor-parallel detection, the 2-D
owner coordinates and the per-owner balance of TP owners."""
import collections
import os
import tempfile

import torch
import torch.multiprocessing as mp
import torch.nn as nn


class Blk(nn.Module):
    def __init__(self):
        super().__init__()
        self.up_proj = nn.Linear(64, 256, bias=False)
        self.down_proj = nn.Linear(256, 64, bias=False)
        self.norm = nn.LayerNorm(64)


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList(Blk() for _ in range(8))
        self.head = nn.Linear(64, 8)


def _body(out_path: str, rank: int):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module
    from torch.testing._internal.distributed.fake_pg import FakeStore

    dist.init_process_group("fake", store=FakeStore(), rank=rank, world_size=16)
    from dmuon_b200.parallel.partition import compute_balanced_assignment
    from dmuon_b200.parallel.topology import get_tp_shard_dim, is_tp_sharded

    mesh = init_device_mesh("cpu", (2, 4, 2), mesh_dim_names=("replicate", "shard", "tp"))
    torch.manual_seed(0)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    pred = lambda n, p: "proj" in n                      # noqa: E731
    res = compute_balanced_assignment(model, mesh["shard"], pred, replicate_mesh=mesh["replicate"])
    dp = frozenset({"replicate", "shard"})
    named = [(n, p) for n, p in model.named_parameters() if pred(n, p)]
    owners = {n: res[p] for n, p in named}
    tp_owner = {n: res.tp_owners[p] for n, p in named}
    info = {
        "owners": owners,
        "tp_owner": tp_owner,
        "tp_flags": [is_tp_sharded(p, dp) for _, p in named],
        "norm_is_tp": is_tp_sharded(model.layers[0].norm.weight, dp),
        "dims": (get_tp_shard_dim(model.layers[0].up_proj.weight, dp), get_tp_shard_dim(model.layers[0].down_proj.weight, dp)),
    }
    torch.save(info, out_path)
    dist.destroy_process_group()


def _run(rank: int):
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "out.pt")
        ctx = mp.get_context("spawn")
        p = ctx.Process(target=_body, args=(path, rank), daemon=True)
        p.start()
        p.join(120)
        assert not p.is_alive() and p.exitcode == 0
        return torch.load(path, weights_only=False)


def test_three_dimensional_partition_on_a_fake_sixteen_rank_job():
    a = _run(rank=5)
    b = _run(rank=12)
    # the assignment is a pure function of the model and the mesh sizes: every rank computes the same one
    assert a["owners"] == b["owners"] and a["tp_owner"] == b["tp_owner"]
    assert all(a["tp_flags"]) and not a["norm_is_tp"]
    assert a["dims"] == (0, 1)                               # column-parallel shards rows, row-parallel shards columns
    owners = list(a["owners"].values())
    assert all(isinstance(o, tuple) and 0 <= o[0] < 4 and 0 <= o[1] < 2 for o in owners)
    load = collections.Counter(owners)
    assert len(load) == 8 and max(load.values()) - min(load.values()) <= 1     # 16 matrices over 8 owner slots
    # inside every data-parallel owner the two TP ranks share the full-matrix work
    per_owner = collections.defaultdict(list)
    for n, o in a["owners"].items():
        per_owner[o].append(a["tp_owner"][n])
    for o, tps in per_owner.items():
        assert all(t in (0, 1) for t in tps)
        if len(tps) >= 2:
            assert set(tps) == {0, 1}, (o, tps)

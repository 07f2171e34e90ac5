"""Tensor-parallel matrices under dedicated Muon on CPU (gloo, DP2 x TP2):
gather reduced shards to the TP owner, orthogonalise the full matrix, scatter
the update -- must equal single-process Muon on the unsharded model."""
import math

import pytest
import torch
import torch.nn as nn

from dist_utils import run_ranks

LR, MU, WD, ALR = 0.02, 0.95, 0.1, 1e-3


class Block(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.up_proj = nn.Linear(d, h, bias=False)
        self.down_proj = nn.Linear(h, d, bias=False)

    def forward(self, x):
        return x + self.down_proj(torch.nn.functional.gelu(self.up_proj(self.norm(x))))


class Net(nn.Module):
    def __init__(self, d=32, h=64, n=3):
        super().__init__()
        self.inp = nn.Linear(8, d)
        self.layers = nn.ModuleList(Block(d, h) for _ in range(n))
        self.head = nn.Linear(d, 4)

    def forward(self, x):
        x = self.inp(x)
        for l in self.layers:
            x = l(x)
        return self.head(x)


def _pred(n, p):
    return "proj" in n and p.ndim == 2


def _data(step):
    g = torch.Generator().manual_seed(77 + step)
    return torch.randn(8, 8, generator=g), torch.randn(8, 4, generator=g)


def _oracle(steps):
    from dmuon_b200.optim.newton_schulz import gram_newton_schulz

    torch.manual_seed(0)
    model = Net()
    params = dict(model.named_parameters())
    mom = {n: torch.zeros_like(p) for n, p in params.items() if _pred(n, p)}
    adam = {n: [torch.zeros_like(p), torch.zeros_like(p), 0] for n, p in params.items() if not _pred(n, p)}
    losses = []
    for s in range(steps):
        x, y = _data(s)
        loss = (model(x) - y).pow(2).mean()
        model.zero_grad()
        loss.backward()
        losses.append(loss.item())
        with torch.no_grad():
            for n, p in params.items():
                g = p.grad
                if n in mom:
                    mom[n].mul_(MU).add_(g)
                    o = gram_newton_schulz(g.add(mom[n], alpha=MU))
                    p.mul_(1 - LR * WD).add_(o, alpha=-LR * 0.2 * math.sqrt(max(p.shape)))
                else:
                    st = adam[n]
                    st[2] += 1
                    p.mul_(1 - ALR * 0.01)
                    st[0].mul_(0.9).add_(g, alpha=0.1)
                    st[1].mul_(0.999).addcmul_(g, g, value=0.001)
                    den = (st[1].sqrt() / math.sqrt(1 - 0.999 ** st[2])).add_(1e-8)
                    p.addcdiv_(st[0], den, value=-ALR / (1 - 0.9 ** st[2]))
    return losses, {n: p.detach().clone() for n, p in params.items()}


def _body(rank, world, mode, steps):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    torch.manual_seed(0)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    if mode in ("fsdp", "fsdp_gram"):
        # the plain run also exercises reuse of the gather / scatter buffers across steps
        owners = dmuon.dedicate_params(model, mesh["dp"], _pred, reshard_after_forward=False,
                                       tp_buffer_reuse=(mode == "fsdp"))
        for blk in model.layers:
            fully_shard(blk, mesh=mesh["dp"])
        fully_shard(model, mesh=mesh["dp"])
    else:
        owners = dmuon.dedicate_params_ddp_tp(model, mesh["dp"], _pred)
        dmuon.replicate_tp(model, mesh["dp"])
    extra = dict(tp_distributed_gram=True, tp_distributed_gram_policy="all") if mode == "fsdp_gram" else {}
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, **extra)
    if mode == "fsdp_gram":
        # both orientations qualify: column-parallel tall and row-parallel wide matrices
        assert all(opt._tp_gram_rejection_reason(p) is None for p in dmuon.get_dedicated_params(model))
    dp_rank = mesh["dp"].get_local_rank()
    losses = []
    for s in range(steps):
        x, y = _data(s)
        x, y = x[dp_rank * 4 : dp_rank * 4 + 4], y[dp_rank * 4 : dp_rank * 4 + 4]
        opt.zero_grad()
        loss = (model(x) - y).pow(2).mean()
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt, group=mesh["dp"].get_group())
        losses.append((lt / 2).item())
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    tp_owned = sum(1 for p in dmuon.get_dedicated_params(model) if p.is_owner and p.is_tp_owner)
    osd = dmuon.get_optimizer_state_dict(model, opt, rank0_only=False)
    mshape = tuple(osd["dedicated"]["layers.0.up_proj.weight"]["momentum_buffer"].shape)
    return losses, sd, tp_owned, mshape


@pytest.mark.parametrize("mode", ["fsdp", "ddp_tp", "fsdp_gram"])
def test_tp_muon_matches_single_process(mode):
    steps = 4
    ref_losses, ref_params = _oracle(steps)
    res = run_ranks(_body, 4, args=(mode, steps))
    losses, sd, _, mshape = res[0]
    assert mshape == (64, 32)
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (losses, ref_losses)
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 2e-4, n
    # six TP matrices, every one orthogonalised on exactly one rank
    assert sum(r[2] for r in res) == 6


def _llama_body(rank, world, steps):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    cfg = LlamaConfig.tiny(n_layers=2, loss_chunk=0)
    torch.manual_seed(0)
    model = LlamaModel(cfg)
    ids = torch.randint(0, cfg.vocab_size, (4, 33), generator=torch.Generator().manual_seed(9))
    if world == 1:
        mesh = init_device_mesh("cpu", (1,), mesh_dim_names=("dp",))
        dp_rank, dp = 0, 1
    else:
        mesh2 = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
        plan = {
            "self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(),
            "self_attn.v_proj": ColwiseParallel(), "self_attn.o_proj": RowwiseParallel(),
            "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel(),
        }
        for layer in model.layers:
            parallelize_module(layer, mesh2["tp"], plan)
        mesh = mesh2["dp"]
        dp_rank, dp = mesh.get_local_rank(), 2
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3, weight_decay=0.1, first_step_progress_log=False)
    per = 4 // dp
    losses = []
    for _ in range(steps):
        b = ids[dp_rank * per : (dp_rank + 1) * per]
        opt.zero_grad()
        loss = model(b[:, :-1], labels=b[:, 1:])
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt)
        losses.append(lt.item() / world)
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return losses, {k: v for k, v in sd.items() if "layers.1" in k}


def test_llama_decoder_under_tensor_parallelism_matches_single_rank():
    """The package's own decoder (heads split over the TP group) trained on a
    DP2 x TP2 mesh follows the single-rank trajectory."""
    steps = 3
    ref_losses, ref_sd = run_ranks(_llama_body, 1, args=(steps,))[0]
    losses, sd = run_ranks(_llama_body, 4, args=(steps,))[0]
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    for n, p in ref_sd.items():
        assert (sd[n].float() - p.float()).abs().max().item() < 5e-4, n


def _body_3d(rank, world, steps):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (2, 2, 2), mesh_dim_names=("replicate", "shard", "tp"))
    torch.manual_seed(0)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    owners = dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=False,
                                   replicate_mesh=mesh["replicate"])
    hsdp = mesh["replicate", "shard"]
    for blk in model.layers:
        fully_shard(blk, mesh=hsdp)
    fully_shard(model, mesh=hsdp)
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR)
    dp_rank = mesh["replicate"].get_local_rank() * 2 + mesh["shard"].get_local_rank()
    losses = []
    for s in range(steps):
        x, y = _data(s)
        x, y = x[dp_rank * 2 : dp_rank * 2 + 2], y[dp_rank * 2 : dp_rank * 2 + 2]
        opt.zero_grad()
        loss = (model(x) - y).pow(2).mean()
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt)
        losses.append((lt / world).item())
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    coords = sorted({tuple(v) if isinstance(v, tuple) else (v,) for v in owners.values()})
    return losses, sd, coords


def test_three_dimensional_mesh_replicate_shard_tp_matches_single_process():
    """R2 x S2 x T2 on eight gloo ranks: two-stage reduce to a 2-D owner
    coordinate, TP gather/scatter inside each owner's TP group, replicate
    publish -- same trajectory as one process."""
    steps = 3
    ref_losses, ref_params = _oracle(steps)
    res = run_ranks(_body_3d, 8, args=(steps,), timeout=480)
    losses, sd, coords = res[0]
    assert all(len(c) == 2 for c in coords) and len(coords) > 1      # 2-D owner coordinates, more than one owner
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (losses, ref_losses)
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 2e-4, n
    for r in range(1, 8):
        for n in sd:
            assert torch.equal(sd[n], res[r][1][n]), (r, n)


def _clip_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    torch.manual_seed(0)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    dmuon.dedicate_params(model, mesh["dp"], _pred, reshard_after_forward=False)
    for blk in model.layers:
        fully_shard(blk, mesh=mesh["dp"])
    fully_shard(model, mesh=mesh["dp"])
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, first_step_progress_log=False)
    dp_rank = mesh["dp"].get_local_rank()
    out = []
    for s in range(2):
        x, y = _data(s)
        x, y = x[dp_rank * 4 : dp_rank * 4 + 4], y[dp_rank * 4 : dp_rank * 4 + 4]
        opt.zero_grad()
        (model(x) - y).pow(2).mean().backward()
        if s == 1:
            before = {id(p): opt.state[id(p)]["momentum_buffer"].clone()
                      for p in dmuon.get_dedicated_params(model) if p.is_owner and p.is_tp_owner}
            stats = dmuon.clip_grad_norm_(opt, 1e-6)          # coefficient ~1e-6 / norm: the step-2 gradient vanishes
            assert float(stats.clip_coef) < 1e-3
        opt.step()
        if s == 1:
            for p in dmuon.get_dedicated_params(model):
                if p.is_owner and p.is_tp_owner:
                    buf = opt.state[id(p)]["momentum_buffer"]
                    out.append(((buf - MU * before[id(p)]).abs().max() / before[id(p)].abs().max()).item())
    return out


def test_clipped_tp_gradients_stay_clipped_in_the_step():
    """Clipping prepares (gathers) the tensor-parallel gradients and scales the
    gathered matrices; the optimizer step that follows must use those, not
    gather the unclipped shards a second time.  With a vanishing clip
    coefficient the momentum after the step is ``mu *`` the old momentum."""
    res = run_ranks(_clip_body, 4, timeout=300)
    rel = [v for r in res for v in r]
    assert len(rel) == 6 and max(rel) < 1e-3, rel


def _tp_save_body(rank, world, steps):
    """DP2 x TP2: train, then hand back the full-tensor checkpoint."""
    import torch.distributed as dist  # noqa: F401
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    torch.manual_seed(0)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    dmuon.dedicate_params(model, mesh["dp"], _pred, reshard_after_forward=False)
    for blk in model.layers:
        fully_shard(blk, mesh=mesh["dp"])
    fully_shard(model, mesh=mesh["dp"])
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, first_step_progress_log=False)
    dp_rank = mesh["dp"].get_local_rank()
    for s in range(steps):
        x, y = _data(s)
        opt.zero_grad()
        (model(x[dp_rank * 4 : dp_rank * 4 + 4]) - y[dp_rank * 4 : dp_rank * 4 + 4]).pow(2).mean().backward()
        opt.step()
    # the summaries also describe tensor-parallel set-ups (and stay JSON-friendly)
    import json

    plan = dmuon.summarize_comm_plan(model)
    rows = dmuon.summarize_param_groups(model, opt)["parameters"]
    json.dumps(plan), json.dumps(rows)
    assert plan["groups"][0]["tp_param_count"] == 2 and all(r["is_dtensor"] for r in rows if "proj" in r["name"])
    assert all(c["tp_owner_local_rank"] in (0, 1) for c in plan["groups"][0]["param_collectives"])
    return (dmuon.get_model_state_dict(model, rank0_only=False),
            dmuon.get_optimizer_state_dict(model, opt, rank0_only=False))


def _plain_resume_body(rank, world, msd, osd, start, steps):
    """Four data-parallel ranks, no tensor parallelism: load the TP run's checkpoint and go on."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(123)                    # other initial weights: everything must come from the checkpoint
    model = Net()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for blk in model.layers:
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, first_step_progress_log=False)
    dmuon.set_model_state_dict(model, msd)
    dmuon.set_optimizer_state_dict(model, opt, osd)
    per = 8 // world
    for s in range(start, start + steps):
        x, y = _data(s)
        opt.zero_grad()
        (model(x[rank * per : (rank + 1) * per]) - y[rank * per : (rank + 1) * per]).pow(2).mean().backward()
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


def test_checkpoint_of_a_tensor_parallel_run_resumes_without_tensor_parallelism():
    """Momentum of TP matrices is saved as the full matrix (it lives on the TP
    owner), weights as full tensors: a DP2 x TP2 checkpoint continues on four
    plain data-parallel ranks along the single-process trajectory."""
    _, ref_params = _oracle(4)
    msd, osd = run_ranks(_tp_save_body, 4, args=(2,))[0]
    assert tuple(osd["dedicated"]["layers.0.up_proj.weight"]["momentum_buffer"].shape) == (64, 32)
    sd = run_ranks(_plain_resume_body, 4, args=(msd, osd, 2, 2))[0]
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 2e-4, n


def _plain_save_body(rank, world, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(0)
    model = Net()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for blk in model.layers:
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, first_step_progress_log=False)
    per = 8 // world
    for s in range(steps):
        x, y = _data(s)
        opt.zero_grad()
        (model(x[rank * per : (rank + 1) * per]) - y[rank * per : (rank + 1) * per]).pow(2).mean().backward()
        opt.step()
    return (dmuon.get_model_state_dict(model, rank0_only=False),
            dmuon.get_optimizer_state_dict(model, opt, rank0_only=False))


def _tp_resume_body(rank, world, msd, osd, start, steps, gram):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    torch.manual_seed(123)
    model = Net()
    for blk in model.layers:
        parallelize_module(blk, mesh["tp"], {"up_proj": ColwiseParallel(), "down_proj": RowwiseParallel()})
    dmuon.dedicate_params(model, mesh["dp"], _pred, reshard_after_forward=False)
    for blk in model.layers:
        fully_shard(blk, mesh=mesh["dp"])
    fully_shard(model, mesh=mesh["dp"])
    extra = dict(tp_distributed_gram=True, tp_distributed_gram_policy="all") if gram else {}
    opt = dmuon.Muon(model, lr=LR, momentum=MU, weight_decay=WD, adamw_lr=ALR, first_step_progress_log=False, **extra)
    dmuon.set_model_state_dict(model, msd)
    dmuon.set_optimizer_state_dict(model, opt, osd)
    dp_rank = mesh["dp"].get_local_rank()
    for s in range(start, start + steps):
        x, y = _data(s)
        opt.zero_grad()
        (model(x[dp_rank * 4 : dp_rank * 4 + 4]) - y[dp_rank * 4 : dp_rank * 4 + 4]).pow(2).mean().backward()
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


@pytest.mark.parametrize("gram", [False, True])
def test_plain_checkpoint_resumes_under_tensor_parallelism(gram):
    """The other direction: full momentum matrices land on the TP owners (and,
    for the Gram-factor route, their slices on every TP rank)."""
    _, ref_params = _oracle(4)
    msd, osd = run_ranks(_plain_save_body, 4, args=(2,))[0]
    sd = run_ranks(_tp_resume_body, 4, args=(msd, osd, 2, 2, gram))[0]
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 2e-4, (gram, n)

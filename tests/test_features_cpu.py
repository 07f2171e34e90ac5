"""Feature coverage on CPU/gloo: hook boundaries, direct weight access, routes,
semantic param groups, clipping across ranks, profiles, async-publish contract,
process-group policy."""
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from dist_utils import run_ranks


class Expert(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.w_proj = nn.Linear(d, d, bias=False)

    def forward(self, x):
        # direct attribute access instead of calling the Linear
        return F.linear(x, self.w_proj.weight)


class Toy(nn.Module):
    def __init__(self, d=16):
        super().__init__()
        self.embed = nn.Embedding(32, d)
        self.towers = nn.ModuleDict({"a": nn.Sequential(Expert(d), Expert(d)), "b": nn.Sequential(Expert(d))})
        self.norm = nn.LayerNorm(d)
        self.head_proj = nn.Linear(d, 32, bias=False)

    def forward(self, ids):
        x = self.embed(ids)
        x = self.towers["a"](x) + self.towers["b"](x)
        return self.head_proj(self.norm(x))


def _pred(n, p):
    return "proj" in n and p.ndim == 2


def _toy_setup(rank, world, **kw):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = Toy()
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    if not any(k.startswith("hook_boundary") for k in kw):
        # Expert reads `.weight` directly, so the boundary has to be a module that is called
        kw["hook_boundary_predicate"] = lambda m: isinstance(m, (nn.Sequential, Toy))
    owners = dmuon.dedicate_params(model, mesh, _pred, **kw)
    fully_shard(model, mesh=mesh)
    return dmuon, model, mesh, owners


def _body_hook_boundaries(rank, world):
    import dmuon_b200 as dmuon

    # predicate: one boundary per tower
    d, model, _, _ = _toy_setup(rank, world, hook_boundary_predicate=lambda m: isinstance(m, nn.Sequential),
                                hook_boundary_strict=False)
    names_pred = sorted(g.name for g in d.utils.iter_groups(model))
    # resolver: everything at the root
    d2, model2, _, _ = _toy_setup(rank, world, hook_boundary_resolver=lambda fqn, p: None, hook_boundary_strict=False)
    names_res = sorted(g.name for g in d2.utils.iter_groups(model2))
    # strict predicate that cannot place head_proj raises
    try:
        _toy_setup(rank, world, hook_boundary_predicate=lambda m: isinstance(m, nn.Sequential))
        raised = False
    except ValueError:
        raised = True
    opt = d.Muon(model, lr=0.05, adamw_lr=1e-2)
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss = F.cross_entropy(model(ids).flatten(0, 1), ids.flatten())
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return names_pred, names_res, raised, losses


def test_hook_boundary_predicate_resolver_and_direct_weight_access():
    names_pred, names_res, raised, losses = run_ranks(_body_hook_boundaries, 2)[0]
    assert names_pred == ["head_proj", "towers.a", "towers.b"]
    assert names_res == ["head_proj", "towers.a.0", "towers.a.1", "towers.b.0"] or len(names_res) == 4
    assert raised
    assert losses[-1] < losses[0]


def _body_routes_and_groups(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = Toy()
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    # every parameter is dedicated: matrices -> muon, embedding -> sharded AdamW, norm -> owner AdamW
    dmuon.dedicate_params(
        model, mesh, lambda n, p: True,
        param_policy={"overrides": [{"contains": "embed", "set": {"route": "sharded_adamw"}},
                                    {"contains": "norm", "set": {"route": "adamw"}}]},
        hook_boundary_resolver=lambda fqn, p: model,        # one boundary: the whole model
    )
    named = dict(model.named_parameters())
    groups = [
        {"params": [p for n, p in named.items() if "towers" in n], "name": "towers", "lr": 0.03, "adamw_lr": 1e-3},
        {"params": [p for n, p in named.items() if "towers" not in n], "name": "rest", "muon_lr": 0.01, "adamw_lr": 5e-3},
    ]
    opt = dmuon.Muon(model, param_groups=groups, record_step_profile=True)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 0.5)
    names = [g["group_name"] for g in opt.param_groups]
    lrs = [g["lr"] for g in opt.param_groups]
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
    losses = []
    for _ in range(4):
        opt.zero_grad()
        loss = F.cross_entropy(model(ids).flatten(0, 1), ids.flatten())
        loss.backward()
        opt.step()
        sched.step()
        losses.append(loss.item())
    prof = opt.consume_last_step_profile()
    summary = dmuon.summarize_param_groups(opt)["groups"]
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    osd = dmuon.get_optimizer_state_dict(model, opt, rank0_only=False)
    bad = None
    try:
        dmuon.Muon(model, param_groups=[groups[0]])
    except RuntimeError as exc:
        bad = str(exc)
    return names, lrs, losses, sorted(prof), [s["dedicated_param_count"] for s in summary], sorted(sd), \
        sorted(osd["dedicated_adamw"]), bad


def test_routes_semantic_groups_scheduler_and_profile():
    names, lrs, losses, prof, counts, sd_keys, adamw_keys, bad = run_ranks(_body_routes_and_groups, 2)[0]
    assert names == ["towers/muon", "towers/adamw", "rest/muon", "rest/adamw"]
    assert lrs == [0.015, 0.0005, 0.005, 0.0025]            # scheduler (x0.5) reaches every lowered group
    assert losses[-1] < losses[0]
    assert {"muon_ms", "adamw_ms", "prepare_muon_grads_ms", "post_step_publish_ms", "dedicated_adamw_ms"} <= set(prof)
    assert counts == [3, 0, 1, 3]
    assert "embed.weight" in sd_keys and "norm.weight" in sd_keys
    assert adamw_keys == ["embed.weight", "norm.bias", "norm.weight"]
    assert bad and "omitted" in bad


def _body_clip(rank, world):
    import torch.distributed as dist

    d, model, _, _ = _toy_setup(rank, world)
    opt = d.Muon(model, lr=0.05)
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
    F.cross_entropy(model(ids).flatten(0, 1), ids.flatten()).backward()
    stats0 = d.clip_grad_norm_(opt, None)                       # measure only
    owned = [p._reduced_grad.clone() for p in d.get_owned_params(model)]
    local_sq = sum(float(g.pow(2).sum()) for g in owned)
    t = torch.tensor(float(local_sq))        # a rank that owns nothing sums to the int 0
    dist.all_reduce(t)
    stats1 = d.clip_grad_norm_(opt, 0.5 * float(stats0.total_norm))
    after = sum(float(p._reduced_grad.pow(2).sum()) for p in d.get_owned_params(model))
    t2 = torch.tensor(float(after))
    dist.all_reduce(t2)
    regular = [p.grad for p in model.parameters() if p.grad is not None]
    res = d.try_clip_optimizer_grad_norm_buckets_(opt, regular_grads=regular, adamw_grads=[], max_norm=1e9)
    # a rank-local inf must not desynchronise anybody: same collective count everywhere
    if rank == 0:
        d.get_owned_params(model)[0]._reduced_grad[0, 0] = float("inf")
    s_inf = d.clip_grad_norm_(opt, 1.0)
    return float(stats0.total_norm), math.sqrt(float(t)), float(stats1.clip_coef), math.sqrt(float(t2)), \
        bool(stats1.clipped), sorted(res.stats_by_name), bool(s_inf.found_inf), opt.last_muon_grad_clip_stats is s_inf


def test_global_clip_across_ranks_and_inf_liveness():
    res = run_ranks(_body_clip, 2, timeout=120)
    for total, ref, coef, after, clipped, buckets, found_inf, last_ok in res:
        assert abs(total - ref) < 1e-5 * ref
        assert abs(coef - 0.5) < 1e-3 and clipped
        assert abs(after - 0.5 * ref) < 1e-3 * ref
        assert buckets == ["adamw", "muon", "regular"]
        assert found_inf and last_ok


def _body_eval_then_step(rank, world):
    d, model, _, _ = _toy_setup(rank, world, reshard_after_forward=False)
    opt = d.Muon(model, lr=0.05)
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
    opt.zero_grad()
    F.cross_entropy(model(ids).flatten(0, 1), ids.flatten()).backward()
    with torch.no_grad():
        before = model(ids).clone()                    # evaluation forward between backward and step
    opt.step()
    with torch.no_grad():
        after = model(ids)
    return float((after - before).abs().max())


def test_evaluation_forward_does_not_leave_stale_weights():
    assert all(v > 1e-4 for v in run_ranks(_body_eval_then_step, 2))


def _body_hsdp_contract(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = Toy()
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("replicate", "shard"))
    dmuon.dedicate_params(model, mesh["shard"], _pred, replicate_mesh=mesh["replicate"],
                          replicate_broadcast_bucket_mb=0.0001,
                          hook_boundary_predicate=lambda m: isinstance(m, (nn.Sequential, Toy)))
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.05, replicate_async=True)
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
    opt.zero_grad()
    F.cross_entropy(model(ids).flatten(0, 1), ids.flatten()).backward()
    opt.step()
    pending = any(g.has_pending_post_step() for g in dmuon.utils.iter_groups(model))
    # replicate peers agree once the publish is drained
    dmuon.wait_all_replicate_broadcasts(model)
    import torch.distributed as dist

    worst = 0.0
    for p in dmuon.get_dedicated_params(model):
        if p._owned_data is not None:
            t = p._owned_data.clone()
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=p.replicate_group)
            worst = max(worst, float((t - p._owned_data).abs().max()))
    owners = sorted({p.owner_rank for p in dmuon.get_dedicated_params(model)})
    with_master = sum(1 for p in dmuon.get_dedicated_params(model) if p._owned_data is not None)
    return pending, worst, owners, with_master, len(dmuon.get_dedicated_params(model))


def test_hsdp_async_publish_contract_and_column_masters():
    res = run_ranks(_body_hsdp_contract, 4)
    assert all(r[1] == 0.0 for r in res)
    assert all(isinstance(o, tuple) for o in res[0][2])
    total = res[0][4]
    # every parameter has its master on exactly one shard column = two of the four ranks
    assert sum(r[3] for r in res) == 2 * total


def _body_pg_policy(rank, world):
    import torch.distributed as dist

    from dmuon_b200.parallel import topology

    d, model, mesh, _ = _toy_setup(rank, world)
    ctx = d.get_comm_ctx(model)
    isolated = topology.is_isolated_process_group(ctx.dp_group)
    same = ctx.dp_group is mesh.get_group()
    d2, model2, mesh2, _ = _toy_setup(rank, world, process_group_policy="shared")
    shared_same = d2.get_comm_ctx(model2).dp_group is mesh2.get_group()
    d.utils.fence_isolated_process_groups(force=True)
    return isolated, same, shared_same


def test_process_group_policy():
    for isolated, same, shared_same in run_ranks(_body_pg_policy, 2):
        assert isolated and not same and shared_same


def _body_profile_counters(rank, world):
    import os

    os.environ["DMUON_RECORD_FORWARD_PROFILE"] = "1"
    try:
        d, model, _, _ = _toy_setup(rank, world, reshard_after_forward=True)
        opt = d.Muon(model, lr=0.05, first_step_progress_log=False)
        ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(rank))
        for _ in range(2):
            opt.zero_grad()
            F.cross_entropy(model(ids).flatten(0, 1), ids.flatten()).backward()
            opt.step()
        prof = d.collect_forward_unshard_profile(model)
        again = d.collect_forward_unshard_profile(model)          # draining resets the counters
        post = d.utils.collect_post_step_profile(model)
    finally:
        os.environ.pop("DMUON_RECORD_FORWARD_PROFILE", None)
    return prof, again, post


def test_forward_profile_counters_are_collected_and_drained():
    for prof, again, post in run_ranks(_body_profile_counters, 2):
        assert prof and all(isinstance(v, dict) for v in prof.values())
        keys = set().union(*[set(v) for v in prof.values()])
        # Z3: every group is published for forward and again for backward, two steps -> dispatches and waits were counted
        assert {"demand_dispatch_calls", "wait_calls", "owner_broadcast_bytes"} <= keys or "prefetch_dispatch_calls" in keys
        total_dispatch = sum(v.get("demand_dispatch_calls", 0) + v.get("prefetch_dispatch_calls", 0) for v in prof.values())
        assert total_dispatch >= 2 * 2 * len(prof) - 2
        assert all(not v for v in again.values()) and isinstance(post, dict)


def _first_step_log_body(rank, world, enabled, limit):
    import contextlib
    import io

    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import _build_model, _data, _pred

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, first_step_progress_log=enabled, first_step_progress_log_limit=limit)
    per = 4 // world
    outs = []
    for s in range(2):
        x, y = _data(s)
        model(x[rank * per : (rank + 1) * per], labels=y[rank * per : (rank + 1) * per]).backward()
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            opt.step()
        opt.zero_grad()
        outs.append(buf.getvalue())
    return outs


def test_first_step_progress_lines_are_rank_tagged_limited_and_only_on_the_first_step():
    on = run_ranks(_first_step_log_body, 2, args=(True, 2))
    for rank, (first, second) in enumerate(on):
        lines = [ln for ln in first.splitlines() if ln.startswith("[dmuon_b200]")]
        assert lines and all(f"[rank={rank}/2]" in ln for ln in lines)
        assert "first optimizer step started" in lines[0] and "owned_muon_params=" in lines[0]
        shape_lines = [ln for ln in lines if "Newton-Schulz" in ln and " x " in ln]
        assert 1 <= len(shape_lines) <= 2                      # first_step_progress_log_limit
        assert "queued after" in lines[-1]
        assert second == ""                                    # later steps are silent
    off = run_ranks(_first_step_log_body, 2, args=(False, 8))
    assert all(first == "" and second == "" for first, second in off)


def _spans_hosts_body(rank, world):
    import os

    from dmuon_b200.parallel.peer import spans_hosts

    out = []
    for val in (None, str(world), "1", "not-a-number"):
        if val is None:
            os.environ.pop("LOCAL_WORLD_SIZE", None)
        else:
            os.environ["LOCAL_WORLD_SIZE"] = val
        out.append(spans_hosts())
    return out


def test_peer_plane_stays_off_when_the_launcher_reports_several_hosts():
    """``LOCAL_WORLD_SIZE`` smaller than the world size means ranks on other
    hosts: peer memory is then not considered (no variable: nothing is assumed)."""
    from dmuon_b200.parallel.peer import spans_hosts

    assert spans_hosts() is False                      # no process group here
    for got in run_ranks(_spans_hosts_body, 2):
        assert got == [False, False, True, False]

"""Asynchronous post-step publish must be bit-identical to the synchronous one
(HSDP replicate broadcast, DDP post-step broadcast), and the sharded-AdamW
route must behave the same on a 1-D and on a replicate x shard mesh."""
import pytest
import torch

from dist_utils import run_ranks
from test_e2e_cpu import HP, _build_model, _data, _pred


def _train(model, opt, rank, world, steps):
    per = 4 // world
    for s in range(steps):
        x, y = _data(s)
        x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
        opt.zero_grad()
        model(x, labels=y).backward()
        opt.step()


def _body_async(rank, world, mode, replicate_async):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    model = _build_model()
    if mode == "hsdp":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=False, replicate_mesh=mesh["replicate"])
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params_ddp(model, mesh, _pred)
        dmuon.replicate(model, mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], replicate_async=replicate_async, first_step_progress_log=False)
    _train(model, opt, rank, world, 3)
    pending = sum(1 for g in dmuon.utils.iter_groups(model) if g.has_pending_post_step())
    dmuon.wait_all_replicate_broadcasts(model)
    after = sum(1 for g in dmuon.utils.iter_groups(model) if g.has_pending_post_step())
    return dmuon.get_model_state_dict(model, rank0_only=False), pending, after


@pytest.mark.parametrize("mode", ["hsdp", "ddp"])
def test_async_publish_is_bit_identical_to_sync(mode):
    a = run_ranks(_body_async, 4, args=(mode, True))
    b = run_ranks(_body_async, 4, args=(mode, False))
    assert all(r[2] == 0 for r in a + b)                   # the drain call leaves nothing pending
    assert all(r[1] == 0 for r in b)                       # synchronous mode never leaves an event behind
    for r in range(4):
        for n, t in a[r][0].items():
            assert torch.equal(t, b[r][0][n]), (mode, r, n)


def _body_sharded_adamw(rank, world, hsdp):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    model = _build_model()
    policy = {"overrides": [{"contains": "embed", "set": {"route": "sharded_adamw"}}]}
    pred = lambda n, p: _pred(n, p) or "embed" in n         # noqa: E731
    if hsdp:
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        dmuon.dedicate_params(model, mesh["shard"], pred, replicate_mesh=mesh["replicate"], param_policy=policy,
                              hook_boundary_strict=False)
        fsdp_mesh = mesh
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params(model, mesh, pred, param_policy=policy, hook_boundary_strict=False)
        fsdp_mesh = mesh
    for layer in model.layers:
        fully_shard(layer, mesh=fsdp_mesh)
    fully_shard(model, mesh=fsdp_mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], first_step_progress_log=False)
    routes = sorted({p._dmuon_route for p in dmuon.get_dedicated_params(model)})
    _train(model, opt, rank, world, 3)
    return dmuon.get_model_state_dict(model, rank0_only=False), routes


def test_sharded_adamw_route_matches_between_one_axis_and_hsdp():
    flat = run_ranks(_body_sharded_adamw, 4, args=(False,))
    grid = run_ranks(_body_sharded_adamw, 4, args=(True,))
    assert flat[0][1] == grid[0][1] == ["muon", "sharded_adamw"]
    for n, t in flat[0][0].items():
        assert (t.float() - grid[0][0][n].float()).abs().max().item() < 5e-4, n


def _body_stage2(rank, world, delay):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    model = _build_model()
    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
    dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=False, replicate_mesh=mesh["replicate"],
                          delay_stage2_to_optimizer=delay)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], first_step_progress_log=False)
    per = 4 // world
    x, y = _data(0)
    x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
    opt.zero_grad()
    model(x, labels=y).backward()
    # right after backward: was the replicate-axis reduce already issued?
    launched = sum(1 for g in dmuon.utils.iter_groups(model) if g._stage2_ticket is not None or (not g._pending and not g._pending_flat))
    groups = sum(1 for _ in dmuon.utils.iter_groups(model))
    opt.step()
    _train(model, opt, rank, world, 2)
    return dmuon.get_model_state_dict(model, rank0_only=False), launched, groups


def test_replicate_axis_reduce_can_be_delayed_to_the_optimizer():
    now = run_ranks(_body_stage2, 4, args=(False,))
    later = run_ranks(_body_stage2, 4, args=(True,))
    assert all(r[1] == r[2] for r in now)                    # issued inside backward for every group
    assert all(r[1] < r[2] for r in later)                   # held back until the optimizer asks
    for r in range(4):
        for n, t in now[r][0].items():
            assert torch.equal(t, later[r][0][n]), (r, n)


def _body_pipeline(rank, world, mode, prepare_ahead):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    model = _build_model()
    if mode == "hsdp":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=False, replicate_mesh=mesh["replicate"])
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params_ddp(model, mesh, _pred)
        dmuon.replicate(model, mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], group_prepare_ahead=prepare_ahead, record_step_profile=True,
                     first_step_progress_log=False)
    blocks = len(opt._pipeline_blocks())
    _train(model, opt, rank, world, 3)
    prof = opt.consume_last_step_profile()
    dmuon.wait_all_replicate_broadcasts(model)
    return dmuon.get_model_state_dict(model, rank0_only=False), blocks, sorted(prof)


@pytest.mark.parametrize("mode", ["hsdp", "ddp"])
def test_group_pipeline_is_bit_identical_to_the_unpipelined_step(mode):
    """``group_prepare_ahead``: the step walks through blocks of groups (next
    block's gradient waits queued ahead, each block's publish dispatched right
    after its update) and must produce exactly the weights of the one-block step."""
    piped = run_ranks(_body_pipeline, 4, args=(mode, True))
    plain = run_ranks(_body_pipeline, 4, args=(mode, False))
    assert all(r[1] == 4 for r in piped) and all(r[1] == 1 for r in plain)      # 4 layers -> 4 blocks vs one
    assert "group_pipeline_ms" in piped[0][2] and "group_pipeline_ms" not in plain[0][2]
    for r in range(4):
        for n, t in piped[r][0].items():
            assert torch.equal(t, plain[r][0][n]), (mode, r, n)


def _double_dispatch_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import _build_model, _data, _pred

    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
    model = _build_model()
    dmuon.dedicate_params(model, mesh["shard"], _pred, replicate_mesh=mesh["replicate"])
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, replicate_async=True, first_step_progress_log=False)
    per = 4 // world
    x, y = _data(0)
    model(x[rank * per : (rank + 1) * per], labels=y[rank * per : (rank + 1) * per]).backward()
    opt.step()
    pending = any(g.has_pending_post_step() for g in dmuon.utils.iter_groups(model))
    # a second dispatch while the first has not been consumed by a forward must be refused ...
    err = None
    try:
        dmuon.broadcast_all_updates_async(model)
    except RuntimeError as exc:
        err = str(exc)
    # ... and draining makes the state legal again
    dmuon.wait_all_replicate_broadcasts(model)
    drained = not any(g.has_pending_post_step() for g in dmuon.utils.iter_groups(model))
    dmuon.broadcast_all_updates(model)
    return pending, err, drained


def test_second_async_publish_before_a_forward_is_refused_and_draining_recovers():
    """One pending publish per group: dispatching again before a forward (or a
    drain) consumed it raises; ``wait_all_replicate_broadcasts`` is the drain."""
    for pending, err, drained in run_ranks(_double_dispatch_body, 4):
        assert pending and drained
        assert err is not None and "already in flight" in err

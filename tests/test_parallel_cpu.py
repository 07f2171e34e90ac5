"""Placement equivalence on CPU (gloo): 1-D FSDP2, replicate x shard (HSDP),
DDP, gradient accumulation and checkpoint round trips must all reproduce the
same training trajectory."""
import pytest
import torch

from dist_utils import run_ranks
from test_e2e_cpu import HP, _build_model, _data, _pred, oracle_run


def _setup(rank, world, mode, reshard=False):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    model = _build_model()
    # "*_gather": Muon matrices rebuilt in forward by all-gather from per-rank shards
    extra = dict(muon_forward_unshard="all_gather") if mode.endswith("_gather") else {}
    mode = mode.replace("_gather", "")
    if mode == "hsdp":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=reshard, replicate_mesh=mesh["replicate"], **extra)
        # flattening the grid onto the peer plane is a single-host CUDA decision; on CPU the two-stage path runs
        assert model._dedicated_comm_ctx.hsdp_flattened is False and model._dedicated_comm_ctx.replicate_group is not None
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    elif mode == "ddp":
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params_ddp(model, mesh, _pred)
        dmuon.replicate(model, mesh)
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=reshard, **extra)
        if extra:
            assert all(p._sharded_muon_data is not None for p in dmuon.get_dedicated_params(model))
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(
        model, lr=HP["lr"], ns_steps=5, adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
        momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"],
    )
    return dmuon, model, opt


def _train(rank, world, model, opt, steps, start=0):
    import torch.distributed as dist

    per = 4 // world
    losses = []
    for s in range(start, start + steps):
        x, y = _data(s)
        x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
        opt.zero_grad()
        loss = model(x, labels=y)
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt)
        losses.append((lt / world).item())
    return losses


def _body_mode(rank, world, mode, reshard, steps):
    dmuon, model, opt = _setup(rank, world, mode, reshard)
    losses = _train(rank, world, model, opt, steps)
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    plan = dmuon.summarize_comm_plan(model)
    groups = dmuon.summarize_param_groups(model, opt)
    return losses, sd, plan["owner_imbalance"], groups["num_groups"]


@pytest.mark.parametrize(
    "mode,reshard",
    [("fsdp", False), ("hsdp", False), ("hsdp", True), ("ddp", False), ("fsdp_gather", True), ("hsdp_gather", False)],
)
def test_four_rank_placements_match_single_process(mode, reshard):
    steps = 5
    ref_losses, ref_params = oracle_run(steps)
    res = run_ranks(_body_mode, 4, args=(mode, reshard, steps))
    losses, sd, imb, ngroups = res[0]
    assert ngroups == 2
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (mode, losses, ref_losses)
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 5e-4, n
    for r in range(1, 4):
        for n in sd:
            assert torch.equal(sd[n], res[r][1][n]), (mode, r, n)


def _body_accum(rank, world, use_no_sync):
    import torch.distributed as dist

    dmuon, model, opt = _setup(rank, world, "fsdp")
    per = 4 // world
    for s in range(2):
        opt.zero_grad()
        for micro in range(2):
            x, y = _data(2 * s + micro)
            x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
            if use_no_sync and micro == 0:
                with dmuon.no_sync(model):
                    (model(x, labels=y) / 2).backward()
            else:
                (model(x, labels=y) / 2).backward()
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


def test_grad_accumulation_with_and_without_no_sync():
    a = run_ranks(_body_accum, 2, args=(False,))[0]
    b = run_ranks(_body_accum, 2, args=(True,))[0]
    for n in a:
        assert (a[n].float() - b[n].float()).abs().max().item() < 1e-4, n


def _body_hsdp_gate(rank, world, gate_off_first):
    """HSDP 2 x 2, two micro-batches per step; optionally the first one runs with
    the replicate-axis gate off on every group (shard-axis reduce only, partial
    sums kept on the owner column).  A sharded-AdamW tensor rides along."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.utils import iter_groups

    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
    model = _build_model()
    dmuon.dedicate_params(
        model, mesh["shard"], lambda n, p: _pred(n, p) or n == "norm.weight", replicate_mesh=mesh["replicate"],
        param_policy={"overrides": [{"name": "norm.weight", "set": {"route": "sharded_adamw"}}]},
    )
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"], first_step_progress_log=False)
    groups = list(iter_groups(model))
    assert all(g.reduce_grads_enabled and g.replicate_grads_enabled for g in groups)
    per = 4 // world
    kept = 0
    for s in range(2):
        opt.zero_grad()
        for micro in range(2):
            x, y = _data(2 * s + micro)
            x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
            for g in groups:
                g.replicate_grads_enabled = not (gate_off_first and micro == 0)
            (model(x, labels=y) / 2).backward()
            if gate_off_first and micro == 0:
                kept += sum(len(g._partial_packs) + len(g._partial_flat) for g in groups)
                assert not any(g.has_pending_reduce() for g in groups)       # nothing waits for the replicate axis
        opt.step()
        assert not any(g._partial_packs or g._partial_flat for g in groups)
    return dmuon.get_model_state_dict(model, rank0_only=False), kept


def test_hsdp_replicate_axis_gate_defers_stage_two_without_changing_the_result():
    a = run_ranks(_body_hsdp_gate, 4, args=(False,))
    b = run_ranks(_body_hsdp_gate, 4, args=(True,))
    assert a[0][1] == 0 and sum(r[1] for r in b) > 0          # partial sums were really kept somewhere
    for n in a[0][0]:
        assert (a[0][0][n].float() - b[0][0][n].float()).abs().max().item() < 1e-5, n


def _body_ckpt(rank, world, mode):
    dmuon, model, opt = _setup(rank, world, mode)
    _train(rank, world, model, opt, 2)
    msd = dmuon.get_model_state_dict(model, rank0_only=False)
    osd = dmuon.get_optimizer_state_dict(model, opt, rank0_only=False)
    cont = _train(rank, world, model, opt, 2, start=2)
    # fresh model + optimizer restored from the state dicts must continue identically
    dmuon2, model2, opt2 = _setup(rank, world, mode)
    dmuon2.set_model_state_dict(model2, msd)
    dmuon2.set_optimizer_state_dict(model2, opt2, osd)
    cont2 = _train(rank, world, model2, opt2, 2, start=2)
    keys = (sorted(osd), sorted(osd["dedicated"])[:2], len(osd["fsdp"]), len(osd["dedicated"]))
    mom = next(iter(osd["dedicated"].values()))["momentum_buffer"]
    return cont, cont2, keys, tuple(mom.shape), str(mom.dtype), sorted(msd)


@pytest.mark.parametrize("mode", ["fsdp", "hsdp", "ddp", "fsdp_gather"])
def test_checkpoint_roundtrip_resumes_identically(mode):
    world = 4 if mode == "hsdp" else 2
    res = run_ranks(_body_ckpt, world, args=(mode,))
    cont, cont2, keys, mshape, mdtype, names = res[0]
    assert keys[0] == ["dedicated", "dedicated_adamw", "fsdp", "param_groups"]
    assert keys[3] == 28 and keys[2] == 10      # 28 matrices; embedding + 9 norms
    assert len(mshape) == 2 and mdtype == "torch.float32"
    ref = _build_model()
    assert names == sorted(dict(ref.named_parameters(remove_duplicate=False)))
    for a, b in zip(cont, cont2):
        assert abs(a - b) < 1e-5, (cont, cont2)


def _body_plain_load(rank, world, mode):
    dmuon, model, opt = _setup(rank, world, mode)
    torch.manual_seed(123)                          # a different initialisation than the one _setup used
    donor = _build_model()
    plain = {k: v.detach().clone() for k, v in donor.state_dict().items()}
    dmuon.set_model_state_dict(model, plain if rank == 0 else {}, broadcast_from_rank0=True)
    back = dmuon.get_model_state_dict(model, rank0_only=False)
    x, y = _data(0)
    with torch.no_grad():
        loss = model(x, labels=y).item()
        want = donor(x, labels=y).item()
    return back, plain, loss, want


@pytest.mark.parametrize("mode", ["fsdp", "hsdp", "ddp"])
def test_loading_a_plain_single_process_state_dict(mode):
    """A state dict saved from an unsharded model loads into any placement
    (only rank 0 holds it), round-trips exactly and gives the same loss."""
    world = 4 if mode == "hsdp" else 2
    for back, plain, loss, want in run_ranks(_body_plain_load, world, args=(mode,)):
        assert sorted(back) == sorted(plain)
        for k in plain:
            assert torch.equal(back[k], plain[k]), k
        assert abs(loss - want) < 1e-5 * max(1.0, abs(want))


def _body_invariants(rank, world):
    import torch.distributed as dist

    dmuon, model, opt = _setup(rank, world, "hsdp")
    dps = dmuon.get_dedicated_params(model)
    facts = {
        p.fqn: (tuple(p.owner_rank), bool(p.is_owner), bool(p.in_owner_column), p._owned_data is not None,
                (p.shard_rank, p.replicate_rank))
        for p in dps
    }
    # one backward without a step: who ends up holding a reduced gradient?
    x, y = _data(0)
    per = 4 // world
    model(x[rank * per : (rank + 1) * per], labels=y[rank * per : (rank + 1) * per]).backward()
    dmuon.prepare_muon_grads(model)
    has_grad = {p.fqn: p._reduced_grad is not None for p in dps}
    opt.step()
    dmuon.wait_all_replicate_broadcasts(model)
    # after the publish every rank of the owner's shard column holds the same master
    digests = {}
    for p in dps:
        if p._owned_data is not None:
            digests[p.fqn] = float(p._owned_data.double().sum())
    gathered = [None] * world
    dist.all_gather_object(gathered, digests)
    return facts, has_grad, gathered


def test_ownership_invariants_on_a_replicate_by_shard_grid():
    """One global owner per matrix; master weights exactly on the owner's shard
    column (all replicate indices of the owner's shard index); only the owner ends
    up with a reduced gradient; after the post-step publish the column's copies
    agree."""
    res = run_ranks(_body_invariants, 4)
    names = list(res[0][0])
    for n in names:
        owners = [r for r in range(4) if res[r][0][n][1]]
        assert len(owners) == 1, (n, owners)                                   # I1
        coord = res[0][0][n][0]
        for r in range(4):
            _, is_owner, in_col, has_master, (srank, rrank) = res[r][0][n]
            assert in_col == (srank == coord[0])
            assert has_master == in_col, (n, r)                                # I2
            assert is_owner == (in_col and rrank == coord[1])
            assert res[r][1][n] == is_owner, (n, r)                            # I3
        column = [r for r in range(4) if res[r][0][n][2]]
        vals = [res[0][2][r][n] for r in column]
        assert len(column) == 2 and abs(vals[0] - vals[1]) < 1e-9, (n, vals)   # I4


def _body_state_dtype(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))

    def build(optim_dtype):
        model = _build_model()
        dmuon.dedicate_params(model, mesh, lambda n, p: _pred(n, p) or n == "norm.weight", reshard_after_forward=False,
                              param_policy={"defaults": {"optim_dtype": optim_dtype}})
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
        return model, dmuon.Muon(model, first_step_progress_log=False)

    # train with fp32 optimizer state, save ...
    model, opt = build("fp32")
    per = 4 // world
    x, y = _data(0)
    model(x[rank * per : (rank + 1) * per], labels=y[rank * per : (rank + 1) * per]).backward()
    opt.step()
    msd = dmuon.get_model_state_dict(model, rank0_only=False)
    osd = dmuon.get_optimizer_state_dict(model, opt, rank0_only=False)
    saved = {k: v["momentum_buffer"].dtype for k, v in osd["dedicated"].items()}
    # ... and restore into a set-up whose policy keeps optimizer state in bf16
    model2, opt2 = build("bf16")
    dmuon.set_model_state_dict(model2, msd)
    dmuon.set_optimizer_state_dict(model2, opt2, osd)
    got = {}
    for dp in dmuon.get_owned_params(model2):
        st = opt2.state[id(dp)]
        for key in ("momentum_buffer", "exp_avg", "exp_avg_sq"):
            if key in st:
                ref = osd["dedicated" if key == "momentum_buffer" else "dedicated_adamw"][dp.fqn][key]
                got[(dp.fqn, key)] = (st[key].dtype, float((st[key].float() - ref.float().reshape(st[key].shape)).abs().max()),
                                      float(ref.float().abs().max()))
    return saved, got


def test_restored_optimizer_state_takes_the_policy_dtype():
    """Momentum and dedicated-AdamW moments saved in fp32 load into a set-up whose
    ``optim_dtype`` is bf16 as bf16 tensors with the same values (to bf16
    rounding), as the reference does for the momentum
    (tests/unit/test_checkpoint_state_dtype.py:13-39)."""
    seen = 0
    for saved, got in run_ranks(_body_state_dtype, 2):
        assert saved and all(d == torch.float32 for d in saved.values())
        for (name, key), (dtype, err, scale) in got.items():
            assert dtype == torch.bfloat16, (name, key, dtype)
            assert err <= 8e-3 * max(scale, 1e-12), (name, key, err, scale)
            seen += 1
    assert seen >= 28        # every Muon matrix on its owner, plus the AdamW-routed norm weight's two moments


def _body_save(rank, world, steps):
    dmuon, model, opt = _setup(rank, world, "fsdp")
    _train(rank, world, model, opt, steps)
    return (dmuon.get_model_state_dict(model, rank0_only=False),
            dmuon.get_optimizer_state_dict(model, opt, rank0_only=False))


def _body_resume_elsewhere(rank, world, mode, msd, osd, start, steps):
    dmuon, model, opt = _setup(rank, world, mode)
    dmuon.set_model_state_dict(model, msd)
    dmuon.set_optimizer_state_dict(model, opt, osd)
    losses = _train(rank, world, model, opt, steps, start=start)
    return losses, dmuon.get_model_state_dict(model, rank0_only=False)


@pytest.mark.parametrize("mode", ["hsdp", "ddp", "fsdp_gather"])
def test_checkpoint_written_on_two_ranks_resumes_under_another_placement(mode):
    """Model and optimizer state saved by a 2-rank FSDP run load into a 4-rank
    replicate x shard, replicated or all-gather placement (other owners, other
    shards) and training continues on the single-process trajectory: the
    checkpoint is a property of the model, not of the topology."""
    ref_losses, ref_params = oracle_run(4)
    msd, osd = run_ranks(_body_save, 2, args=(2,))[0]
    res = run_ranks(_body_resume_elsewhere, 4, args=(mode, msd, osd, 2, 2))
    losses, sd = res[0]
    for a, b in zip(losses, ref_losses[2:]):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (mode, losses, ref_losses)
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 5e-4, (mode, n)

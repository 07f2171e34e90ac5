"""End-to-end correctness on CPU: 2 gloo ranks, FSDP2 + dedicated Muon on a
4-layer decoder with tied embeddings, against a single-process Muon."""
import pytest
import torch

from dist_utils import run_ranks

STEPS = 10
HP = dict(lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-3, adamw_wd=0.01, betas=(0.9, 0.999), eps=1e-8)


def _pred(name, p):
    return "proj" in name and p.ndim == 2


def _data(step: int):
    g = torch.Generator().manual_seed(1000 + step)
    ids = torch.randint(0, 1024, (4, 129), generator=g)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def _build_model():
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    torch.manual_seed(0)
    return LlamaModel(LlamaConfig.tiny())


def oracle_run(steps=STEPS):
    """Single-process Muon + AdamW from ``tests/oracle.py``: the update rules
    written out independently of the package, with a textbook float64
    Newton-Schulz (not the package's Gram recurrence)."""
    from oracle import muon_adamw_run

    model = _build_model()
    losses = muon_adamw_run(
        model, _pred, [_data(s) for s in range(steps)], lambda m, b: m(b[0], labels=b[1]),
        lr=HP["lr"], momentum=HP["momentum"], weight_decay=HP["weight_decay"], adamw_lr=HP["adamw_lr"],
        adamw_wd=HP["adamw_wd"], betas=HP["betas"], eps=HP["eps"],
    )
    return losses, {n: p.detach().clone() for n, p in model.named_parameters()}


def _dist_body(rank, world, reshard, steps):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    owners = dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=reshard)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(
        model, lr=HP["lr"], ns_steps=5, adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
        momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"],
    )
    losses = []
    per = 4 // world
    for s in range(steps):
        x, y = _data(s)
        x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
        loss = model(x, labels=y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt)
        losses.append((lt / world).item())
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    n_owned = len(dmuon.get_owned_params(model))
    return losses, sd, n_owned, sorted(set(int(v) for v in owners.values()))


@pytest.mark.parametrize("reshard", [False, True])
def test_two_rank_fsdp2_muon_matches_single_process(reshard):
    ref_losses, ref_params = oracle_run()
    results = run_ranks(_dist_body, 2, args=(reshard, STEPS))
    losses, sd, n0, owners = results[0]
    assert owners == [0, 1]
    assert n0 + results[1][2] == 28
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    assert set(sd) == set(ref_params) | {"lm_head.weight"} or set(sd) == set(ref_params)
    for n, p in ref_params.items():
        err = (sd[n].float() - p).abs().max().item()
        assert err < 5e-4, (n, err)
    # both ranks return identical full state
    for n in sd:
        assert torch.equal(sd[n], results[1][1][n])


def test_single_rank_world():
    ref_losses, _ = oracle_run(3)
    (losses, sd, n_owned, owners), = run_ranks(_dist_body, 1, args=(True, 3))
    assert n_owned == 28 and owners == [0]
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4


def _variant_body(rank, world, nesterov, backend, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(
        model, lr=HP["lr"], ns_steps=5, adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"], momentum=HP["momentum"],
        adamw_weight_decay=HP["adamw_wd"], nesterov=nesterov, ns_backend=backend, first_step_progress_log=False,
    )
    per = 4 // world
    for s in range(steps):
        x, y = _data(s)
        opt.zero_grad()
        model(x[rank * per : (rank + 1) * per], labels=y[rank * per : (rank + 1) * per]).backward()
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


@pytest.mark.parametrize("nesterov,backend", [(False, "gram"), (True, "direct"), (False, "direct")])
def test_plain_momentum_and_the_direct_formulation_follow_the_oracle(nesterov, backend):
    """``nesterov=False`` feeds the momentum buffer itself to Newton-Schulz; the
    direct formulation iterates on the matrix instead of its Gram matrix.  Both
    must land on the single-process trajectory (the oracle's iteration IS the
    direct one, in float64, with the same coefficients)."""
    from oracle import muon_adamw_run

    steps = 4
    ref = _build_model()
    muon_adamw_run(
        ref, _pred, [_data(s) for s in range(steps)], lambda m, b: m(b[0], labels=b[1]),
        lr=HP["lr"], momentum=HP["momentum"], weight_decay=HP["weight_decay"], adamw_lr=HP["adamw_lr"],
        adamw_wd=HP["adamw_wd"], betas=HP["betas"], eps=HP["eps"], nesterov=nesterov,
    )
    sd = run_ranks(_variant_body, 2, args=(nesterov, backend, steps))[0]
    for n, p in ref.named_parameters():
        assert (sd[n].float() - p.detach()).abs().max().item() < 5e-4, (nesterov, backend, n)

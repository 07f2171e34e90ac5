"""Placements on real GPUs over NCCL (the COLLECTIVE data plane, ``comm_backend=
"nccl"``: lanes are CUDA streams, tickets are events) against the single-process
oracle of ``tests/oracle.py``: 1-D FSDP2, replicate x shard with the two-stage
reduce (not flattened onto the peer plane), the replicated (DDP) placement and
DP x TP.  Newton-Schulz runs on the PyTorch fp32 path here so that the comparison
with the float64 oracle is tight: what is under test is the communication and its
stream ordering, not the fp16 kernels (``tests/test_kernels_gpu.py`` covers those).

Reference counterparts: tests/distributed/test_hsdp_correctness.py:222-239,
tests/distributed/test_correctness.py:237-257.
"""
import pytest
import torch

from dist_utils import run_ranks
from test_e2e_cpu import HP, _build_model, _data, _pred, oracle_run

pytestmark = pytest.mark.gpu

STEPS = 4


def _body(rank, world, mode, reshard, steps):
    import os

    os.environ["DMUON_TP_PEER"] = "0"          # collectives for the TP gather / scatter as well
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    dev = torch.device("cuda", rank)
    model = _build_model().to(dev)
    data_ranks, data_rank = world, rank
    if mode == "hsdp":
        mesh = init_device_mesh("cuda", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        dmuon.dedicate_params(model, mesh["shard"], _pred, reshard_after_forward=reshard,
                              replicate_mesh=mesh["replicate"], comm_backend="nccl")
        ctx = model._dedicated_comm_ctx
        assert ctx.hsdp_flattened is False and ctx.replicate_group is not None
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    elif mode == "ddp":
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params_ddp(model, mesh, _pred, comm_backend="nccl")
        dmuon.replicate(model, mesh)
    elif mode == "tp":
        from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

        tp = 2
        mesh = init_device_mesh("cuda", (world // tp, tp), mesh_dim_names=("dp", "tp"))
        plan = {
            "self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(),
            "self_attn.v_proj": ColwiseParallel(), "self_attn.o_proj": RowwiseParallel(),
            "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel(),
        }
        for layer in model.layers:
            parallelize_module(layer, mesh["tp"], plan)
        dmuon.dedicate_params(model, mesh["dp"], _pred, reshard_after_forward=reshard, comm_backend="nccl")
        for layer in model.layers:
            fully_shard(layer, mesh=mesh["dp"])
        fully_shard(model, mesh=mesh["dp"])
        data_ranks, data_rank = world // tp, mesh["dp"].get_local_rank()      # TP peers see the same rows
    else:
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
        dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=reshard, comm_backend="nccl")
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
    assert getattr(model._dedicated_comm_ctx, "peer_runtime", None) is None
    opt = dmuon.Muon(
        model, lr=HP["lr"], ns_steps=5, adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
        momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"], first_step_progress_log=False,
        ns_backend=dmuon.NewtonSchulz(kernel="torch", compute_dtype=torch.float32),
    )
    per = 4 // data_ranks
    losses = []
    for s in range(steps):
        x, y = _data(s)
        x = x[data_rank * per : (data_rank + 1) * per].to(dev)
        y = y[data_rank * per : (data_rank + 1) * per].to(dev)
        opt.zero_grad()
        loss = model(x, labels=y)
        loss.backward()
        opt.step()
        lt = loss.detach().float().clone()
        dist.all_reduce(lt)
        losses.append(float(lt) / world)
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return losses, {k: v.detach().float().cpu() for k, v in sd.items()}


def _check(res, steps, what):
    ref_losses, ref_params = oracle_run(steps)
    losses, sd = res[0]
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (what, losses, ref_losses)
    worst = {n: (sd[n] - p).abs().max().item() for n, p in ref_params.items()}
    top = sorted(worst.items(), key=lambda kv: -kv[1])[:6]
    print(what, "losses", [f"{a:.5f}" for a in losses], "oracle", [f"{b:.5f}" for b in ref_losses], "largest differences", top)
    assert top[0][1] < 5e-4, (what, top)
    for r in range(1, len(res)):
        for n in sd:
            assert torch.equal(sd[n], res[r][1][n]), (what, r, n)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode,reshard", [("fsdp", False), ("fsdp", True), ("ddp", False)])
def test_one_axis_placements_over_nccl_match_single_process(mode, reshard):
    world = 4 if torch.cuda.device_count() >= 4 else 2
    _check(run_ranks(_body, world, args=(mode, reshard, STEPS), backend="nccl", timeout=600), STEPS, (mode, reshard, world))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_over_nccl_matches_single_process():
    """DP x TP = (1 or 2) x 2 with NCCL gather / scatter; the optimizer works
    through the layers in blocks, so gathers and scatters of the TP communicator
    are in flight on two lanes."""
    world = 4 if torch.cuda.device_count() >= 4 else 2
    _check(run_ranks(_body, world, args=("tp", False, STEPS), backend="nccl", timeout=600), STEPS, ("tp", world))


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("reshard", [False, True])
def test_two_stage_hsdp_over_nccl_matches_single_process(reshard):
    """Replicate 2 x shard 2 on the collective plane: shard-axis reduce, then the
    replicate-axis reduce issued when the optimizer asks, replicate publish after
    the step."""
    _check(run_ranks(_body, 4, args=("hsdp", reshard, STEPS), backend="nccl", timeout=600), STEPS, ("hsdp", reshard))

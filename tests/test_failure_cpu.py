"""Failure detection on the host (gloo, no GPU involved): a rank that leaves
between steps must surface as an error on the surviving rank within the
process-group timeout, never as a hang; a bounded device wait that runs out is
reported through ``KernelTimeout`` (the status-word decoding is checked here,
the wait itself in the GPU tests)."""
import os
import socket
import tempfile
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=8))
    import torch.nn as nn
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 16, bias=False), nn.Tanh(), nn.Linear(16, 16, bias=False))
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: p.ndim == 2, hook_boundary_predicate=lambda m: isinstance(m, nn.Sequential),
                          reshard_after_forward=True)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, first_step_progress_log=False)
    x = torch.randn(4, 16)

    def step():
        opt.zero_grad()
        model(x).pow(2).mean().backward()
        opt.step()

    step()                                   # one healthy step on both ranks
    result = {"rank": rank, "healthy_step": True}
    if rank == 1:
        # leaves between steps, with nothing in flight
        torch.save(result, os.path.join(outdir, f"r{rank}.pt"))
        os._exit(0)
    t0 = time.time()
    try:
        step()                               # the peer is gone: the first collective must fail, not hang
        result["error"] = None
    except Exception as exc:                 # noqa: BLE001 - any transport / timeout error is the expected outcome
        result["error"] = type(exc).__name__
    result["seconds"] = time.time() - t0
    torch.save(result, os.path.join(outdir, f"r{rank}.pt"))
    os._exit(0)                              # the process group is broken; skip its destructor


def test_survivor_sees_an_error_when_a_rank_leaves_between_steps():
    port = _free_port()
    with tempfile.TemporaryDirectory() as outdir:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_worker, args=(r, 2, port, outdir), daemon=True) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.kill()
        assert not alive, "a rank hung instead of failing"
        r0 = torch.load(os.path.join(outdir, "r0.pt"), weights_only=False)
        r1 = torch.load(os.path.join(outdir, "r1.pt"), weights_only=False)
    assert r0["healthy_step"] and r1["healthy_step"]
    assert r0["error"] is not None, "the surviving rank completed a step without its peer"
    assert r0["seconds"] < 60


def test_status_words_decode_to_kernel_timeout():
    from dmuon_b200.ops import gemm as G

    assert issubclass(G.KernelTimeout, RuntimeError)
    assert "peer" in G.describe_status(4) and "did not signal" in G.describe_status(4)
    assert "TMA" in G.describe_status(1) and "unknown" in G.describe_status(99)

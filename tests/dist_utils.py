"""Spawn gloo (CPU) or nccl ranks for a test body and collect their results."""
from __future__ import annotations

import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fn, args, outdir: str, backend: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    os.environ["LOCAL_RANK"] = str(rank)
    torch.set_num_threads(2)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world)
        result = fn(rank, world, *args)
        torch.save({"ok": True, "result": result}, os.path.join(outdir, f"r{rank}.pt"))
    except Exception:
        torch.save({"ok": False, "error": traceback.format_exc()}, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_ranks(fn, world: int, args=(), backend: str = "gloo", timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` ranks; returns the list of
    per-rank results, raising with the first traceback if any rank failed."""
    port = _free_port()
    with tempfile.TemporaryDirectory() as outdir:
        ctx = mp.get_context("spawn")
        procs = [
            ctx.Process(target=_worker, args=(r, world, port, fn, args, outdir, backend), daemon=True)
            for r in range(world)
        ]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        hung = [p for p in procs if p.is_alive()]
        for p in hung:
            p.kill()
        if hung:
            raise TimeoutError(f"{len(hung)} rank(s) did not finish within {timeout}s")
        results = []
        for r in range(world):
            path = os.path.join(outdir, f"r{r}.pt")
            if not os.path.exists(path):
                raise RuntimeError(f"rank {r} exited without a result (exit code {procs[r].exitcode})")
            rec = torch.load(path, weights_only=False)
            if not rec["ok"]:
                raise RuntimeError(f"rank {r} failed:\n{rec['error']}")
            results.append(rec["result"])
        return results

#!/usr/bin/env python
"""Topology matrix: run ``bench.py`` once per placement (and optimizer, and
implementation) on N GPUs of this host and print one table.

    python benchmarks/bench_topologies.py --gpus 8
    python benchmarks/bench_topologies.py --gpus 8 --topologies fsdp,hsdp2x4,tp2xdp4 --optimizers muon,adamw
    python benchmarks/bench_topologies.py --gpus 8 --impls ours,reference --model-impls own,hf

Every cell is a separate ``torchrun`` of ``bench.py`` (device-timed step, max
over ranks); the table shows step / optimizer / forward+backward ms, tokens/s,
model FLOP utilisation and peak memory, and the Muon-over-AdamW ratio when both
optimizers were run.  JSON lines of all cells go to ``--out``.

Counterpart of the reference's ``benchmarks/bench_tp_llm.py:764-812`` and its
``run_tp_llm_benchmark.sh`` (topology matrix with p50/p90, tokens/s, MFU, peak
memory), driven by flags instead of environment variables.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cell(gpus: int, port: int, extra: list[str], timeout: int) -> dict:
    if gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "bench.py")]
    else:
        cmd = [sys.executable, os.path.join(ROOT, "bench.py")]
    cmd += ["--gpus", str(gpus)] + extra
    try:
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=timeout, text=True)
    except subprocess.TimeoutExpired:
        return {"error": f"timed out after {timeout} s"}
    for line in reversed(res.stdout.splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    return {"error": (res.stderr or res.stdout)[-400:].strip() or f"exit code {res.returncode}"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--topologies", default="fsdp,hsdp2x4,tp2xdp4,ddp")
    ap.add_argument("--optimizers", default="muon")
    ap.add_argument("--impls", default="ours")
    ap.add_argument("--model-impls", default="own")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--timeout", type=int, default=900)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rows = []
    port = 29700
    for topo in args.topologies.split(","):
        for impl in args.impls.split(","):
            for mimpl in (args.model_impls.split(",") if impl == "ours" else ["hf"]):
                for optim in args.optimizers.split(","):
                    if topo == "ddp" and optim == "adamw":
                        continue            # the AdamW baseline of every placement is FSDP2
                    extra = ["--steps", str(args.steps), "--warmup", str(args.warmup), "--model", args.model,
                             "--parallelism", topo, "--optimizer", optim, "--impl", impl, "--no-e2e"]
                    if impl == "ours":
                        extra += ["--model-impl", mimpl]
                    if topo.startswith("tp") and optim == "muon":
                        extra += ["--clip-norm", "1.0"]
                    port += 1
                    rec = run_cell(args.gpus, port, extra, args.timeout)
                    rec.update(topology=topo, impl_arg=impl, model_impl_arg=mimpl, optimizer_arg=optim)
                    rows.append(rec)
                    print(json.dumps(rec), flush=True)
    if args.out:
        with open(args.out, "w") as fh:
            for r in rows:
                fh.write(json.dumps(r) + "\n")

    adamw = {(r["topology"], r["impl_arg"], r["model_impl_arg"]): r.get("value") for r in rows
             if r["optimizer_arg"] == "adamw" and "value" in r}
    print(f"\n{'topology':10s} {'impl':10s} {'model':5s} {'optim':6s} {'step ms':>9s} {'optim ms':>9s} {'fwd+bwd':>9s} "
          f"{'tok/s':>10s} {'MFU':>6s} {'GiB':>7s} {'vs AdamW':>9s}")
    for r in rows:
        if "value" not in r:
            print(f"{r['topology']:10s} {r['impl_arg']:10s} {r['model_impl_arg']:5s} {r['optimizer_arg']:6s} "
                  f"{(r.get('unavailable') or r.get('error') or '?')[:80]}")
            continue
        base = adamw.get((r["topology"], r["impl_arg"], r["model_impl_arg"]))
        ratio = f"{r['value'] / base:9.3f}" if (base and r["optimizer_arg"] == "muon") else f"{'':>9s}"
        print(f"{r['topology']:10s} {r['impl_arg']:10s} {r['model_impl_arg']:5s} {r['optimizer_arg']:6s} "
              f"{r['value']:9.1f} {r.get('optimizer_step_ms', 0):9.1f} {r.get('fwd_bwd_ms', 0):9.1f} "
              f"{r.get('tokens_per_s', 0):10.0f} {100 * (r.get('mfu') or 0):5.1f}% {r.get('peak_mem_gib', 0):7.1f} {ratio}")


if __name__ == "__main__":
    main()

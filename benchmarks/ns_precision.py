#!/usr/bin/env python
"""Precision study of the Newton-Schulz variants on matrices with controlled
spectra, without an SVD in the metrics.

For every (spectrum, shape, variant) it prints one JSON line with

    orth_err      ||U U^T - I||_F / sqrt(m)            (0 for an exact polar factor)
    sym_err       ||U^T G - (U^T G)^T||_F / ||G||_F     (U^T G is symmetric for the polar factor)
    psd_violation most negative Rayleigh quotient of U^T G over random probes, relative to ||G||_2 estimate
    dual_gap      1 - <U, G> / ||G||_*  with the nuclear norm known from the construction
    vs_fp32       ||U - U_fp32||_max for the same schedule in fp32

Variants: fp32 oracle (PyTorch), and on a B200 the kernels with fp16 operands
(production) and bf16 operands.  Spectra: flat, uniform, Marchenko-Pastur
(plain Gaussian), power law, low rank plus noise, one dominant direction.
The reference keeps the same kind of study under ``tests/precision``
(matrix_zoo.py, polar_metrics.py, ref_ns.py).

    python benchmarks/ns_precision.py --shapes 256x1024,1024x4096 --schedules polar,classic
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

SPECTRA = ("flat", "uniform", "marchenko_pastur", "power_law", "low_rank_noise", "spike")


def _orthonormal(rows: int, cols: int, gen, device) -> torch.Tensor:
    q, _ = torch.linalg.qr(torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float64))
    return q


def make_matrix(kind: str, m: int, n: int, seed: int, device="cpu") -> tuple[torch.Tensor, float]:
    """An ``m x n`` fp32 matrix (m <= n) with the named singular-value profile
    and its nuclear norm."""
    gen = torch.Generator(device=device).manual_seed(seed)
    if kind == "marchenko_pastur":
        G = torch.randn(m, n, generator=gen, device=device, dtype=torch.float64)
        return G.float(), float(torch.linalg.svdvals(G).sum())
    if kind == "flat":
        s = torch.ones(m, dtype=torch.float64, device=device)
    elif kind == "uniform":
        s = torch.linspace(1.0, 0.05, m, dtype=torch.float64, device=device)
    elif kind == "power_law":
        s = torch.arange(1, m + 1, dtype=torch.float64, device=device).pow(-1.0)
    elif kind == "low_rank_noise":
        s = torch.full((m,), 1e-2, dtype=torch.float64, device=device)
        s[: max(1, m // 16)] = 1.0
    elif kind == "spike":
        s = torch.full((m,), 0.05, dtype=torch.float64, device=device)
        s[0] = 10.0
    else:
        raise ValueError(kind)
    U = _orthonormal(m, m, gen, device)
    V = _orthonormal(n, m, gen, device)
    return ((U * s) @ V.T).float(), float(s.sum())


def metrics(U: torch.Tensor, G: torch.Tensor, nuclear: float, probes: int = 16) -> dict:
    U, G = U.double(), G.double()
    m = U.shape[0]
    orth = ((U @ U.T - torch.eye(m, dtype=U.dtype, device=U.device)).norm() / math.sqrt(m)).item()
    H = U.T @ G                                           # n x n, symmetric PSD for the exact factor
    sym = ((H - H.T).norm() / G.norm()).item()
    gen = torch.Generator(device=U.device).manual_seed(0)
    z = torch.randn(H.shape[0], probes, generator=gen, device=U.device, dtype=U.dtype)
    z = z / z.norm(dim=0, keepdim=True)
    rq = ((z * (0.5 * (H + H.T) @ z)).sum(dim=0))
    spec = (G @ z).norm(dim=0).max().item() + 1e-30       # lower bound of ||G||_2, good enough as a scale
    psd = max(0.0, -rq.min().item()) / spec
    dual = 1.0 - (U * G).sum().item() / nuclear
    return {"orth_err": orth, "sym_err": sym, "psd_violation": psd, "dual_gap": dual}


def variants(device: torch.device):
    import dmuon_b200 as dmuon

    out = [("fp32", dmuon.NewtonSchulz(kernel="torch", compute_dtype=torch.float32))]
    if device.type == "cuda":
        out.append(("kernels_fp16", dmuon.NewtonSchulz(compute_dtype=torch.float16)))
        out.append(("kernels_bf16", dmuon.NewtonSchulz(compute_dtype=torch.bfloat16)))
    return out


def schedule(name: str):
    from dmuon_b200.optim import newton_schulz as NS

    return {"polar": None, "you": NS.YOU_COEFFICIENTS, "classic": NS.CLASSIC_COEFFICIENTS}[name]


def run(shapes, schedules, spectra, device, seed=0):
    import dmuon_b200 as dmuon

    rows = []
    for sched in schedules:
        coefs = schedule(sched)
        for m, n in shapes:
            for kind in spectra:
                G, nuclear = make_matrix(kind, m, n, seed, device="cpu")
                G = G.to(device)
                base = None
                for vname, proto in variants(device):
                    ns = dmuon.NewtonSchulz(
                        kernel="torch" if vname == "fp32" else "auto", compute_dtype=proto.compute_dtype, coefficients=coefs
                    )
                    U = ns.local(G, 5).float()
                    if base is None:
                        base = U
                    rec = {"schedule": sched, "shape": [m, n], "spectrum": kind, "variant": vname}
                    rec.update({k: round(v, 6) for k, v in metrics(U, G, nuclear).items()})
                    rec["vs_fp32"] = round((U - base).abs().max().item(), 6)
                    rows.append(rec)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="256x1024,1024x1024")
    ap.add_argument("--schedules", default="polar,classic")
    ap.add_argument("--spectra", default=",".join(SPECTRA))
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args()
    device = torch.device("cuda", 0) if torch.cuda.is_available() and not args.cpu else torch.device("cpu")
    shapes = [tuple(int(x) for x in s.split("x")) for s in args.shapes.split(",")]
    for rec in run(shapes, args.schedules.split(","), args.spectra.split(","), device):
        print(json.dumps(rec))


if __name__ == "__main__":
    main()

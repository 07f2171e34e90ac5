"""A single-process Muon + AdamW written from the published update rules, for
tests to compare the framework against.  Nothing here imports the package:
the Newton-Schulz below is the textbook form of the iteration (normalise by the
Frobenius norm, odd quintic ``a X + b (X X^T) X + c (X X^T)^2 X`` per step,
applied to the matrix itself), not the package's Gram recurrence, so a wrong
specification inside the package cannot pass by agreeing with itself.
"""
from __future__ import annotations

import math

import torch

# Polar Express coefficients (arXiv 2505.16932, Algorithm 1, first five steps) with the 1.05 safety factor
_RAW = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
]
COEFFICIENTS = [(a / 1.05, b / 1.05**3, c / 1.05**5) for a, b, c in _RAW]


def newton_schulz_reference(G: torch.Tensor, coefficients=None, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz on the matrix itself, in float64."""
    X = G.reshape(G.shape[0], -1).double()
    tall = X.shape[0] > X.shape[1]
    if tall:
        X = X.T
    X = X / (X.norm() + eps)
    for a, b, c in (coefficients or COEFFICIENTS):
        A = X @ X.T
        X = a * X + (b * A + c * (A @ A)) @ X
    if tall:
        X = X.T
    return X.to(G.dtype).reshape(G.shape)


def polar_factor(G: torch.Tensor) -> torch.Tensor:
    """``U V^T`` of the thin SVD: what Newton-Schulz approximates."""
    U, _, Vh = torch.linalg.svd(G.double(), full_matrices=False)
    return (U @ Vh).to(G.dtype)


def muon_adamw_run(model, is_muon, batches, loss_fn, *, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-3,
                   adamw_wd=0.01, betas=(0.9, 0.999), eps=1e-8, nesterov=True):
    """Train ``model`` in place, one step per batch.  ``is_muon(name, param)``
    selects the matrices that get Muon; the rest gets AdamW.  Returns the losses."""
    params = dict(model.named_parameters())
    mom = {n: torch.zeros_like(p) for n, p in params.items() if is_muon(n, p)}
    adam = {n: dict(m=torch.zeros_like(p), v=torch.zeros_like(p), t=0) for n, p in params.items() if n not in mom}
    losses = []
    for batch in batches:
        loss = loss_fn(model, batch)
        model.zero_grad()
        loss.backward()
        losses.append(float(loss.detach()))
        with torch.no_grad():
            for n, p in params.items():
                g = p.grad
                if g is None:
                    continue
                if n in mom:
                    buf = mom[n]
                    buf.mul_(momentum).add_(g)
                    u = g.add(buf, alpha=momentum) if nesterov else buf
                    o = newton_schulz_reference(u)
                    rows, cols = p.shape[0], p.numel() // p.shape[0]
                    p.mul_(1 - lr * weight_decay)
                    p.add_(o, alpha=-lr * 0.2 * math.sqrt(max(rows, cols)))
                else:
                    st = adam[n]
                    st["t"] += 1
                    b1, b2 = betas
                    p.mul_(1 - adamw_lr * adamw_wd)
                    st["m"].mul_(b1).add_(g, alpha=1 - b1)
                    st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    denom = (st["v"].sqrt() / math.sqrt(1 - b2 ** st["t"])).add_(eps)
                    p.addcdiv_(st["m"], denom, value=-adamw_lr / (1 - b1 ** st["t"]))
    return losses

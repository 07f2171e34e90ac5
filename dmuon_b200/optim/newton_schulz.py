"""Newton-Schulz orthogonalisation: the numerical specification.

Everything in this file is plain PyTorch and runs on any device; it is the
oracle the sm_100a kernels are tested against and the path CPU (gloo) runs
use.  The batched tcgen05 implementation lives in ``ops/ns_sm100.py`` and is
selected automatically for CUDA tensors.

Two formulations, as in the reference (dmuon/optim/newton_schulz.py:225-448):

direct   X <- a X + (b A + c A A) X  with  A = X X^T, per step
gram     evolve the small Gram matrix R = X X^T and an accumulated left factor
         Q instead of X; X is touched only at restarts and at the end.  With
         P_i = c R^2 + b R + a I (the step polynomial):  Q <- P_i Q,
         R <- R P_i P_i.  All of these are polynomials of one symmetric matrix,
         so every product is symmetric.

Both orient the matrix so that the Gram matrix is built on the smaller side
and normalise by the Frobenius norm (+ eps) first.
"""
from __future__ import annotations

import logging
from typing import Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

log = logging.getLogger(__name__)

#: per-step (a, b, c) by @YouJiacheng, tuned for 5 iterations
YOU_COEFFICIENTS = [
    [4.0848, -6.8946, 2.9270],
    [3.9505, -6.3029, 2.6377],
    [3.7418, -5.5913, 2.3037],
    [2.8769, -3.1427, 1.2046],
    [2.8366, -3.0525, 1.2012],
]

_SAFETY = 1.05
_POLAR_EXPRESS_RAW = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
]
#: Polar Express (arXiv 2505.16932) with a 1.05 safety factor: the default
POLAR_EXPRESS_COEFFICIENTS = [(a / _SAFETY, b / _SAFETY**3, c / _SAFETY**5) for a, b, c in _POLAR_EXPRESS_RAW]

#: the classic single-triple quintic of the original Muon
CLASSIC_QUINTIC = (3.4445, -4.7750, 2.0315)
CLASSIC_COEFFICIENTS = [CLASSIC_QUINTIC] * 5

DEFAULT_COEFFICIENTS = POLAR_EXPRESS_COEFFICIENTS
DEFAULT_RESTART_ITERATIONS = [2]

_KERNEL_NAMES = ("auto", "tcgen05", "torch")
_LEGACY_KERNELS = ("quack", "cute_sm80", "cublas", "compile")


def _coeffs(coefficients, steps: int):
    if coefficients is None:
        return list(DEFAULT_COEFFICIENTS)
    return [tuple(c) for c in coefficients]


def _orient(G: Tensor, eps: float, dtype: Optional[torch.dtype]):
    X = G.float()
    if X.dim() > 2:
        X = X.reshape(X.shape[0], -1)
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.T
    norm = X.norm() + eps
    X = X / norm
    if dtype is not None:
        X = X.to(dtype)
    return X.contiguous(), transposed, norm


def direct_newton_schulz(
    G: Tensor,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    compute_dtype: Optional[torch.dtype] = None,
) -> Tensor:
    """Parameter-space iteration; ``steps`` limits how many triples are used."""
    coefs = _coeffs(coefficients, steps)[: max(1, steps)]
    dtype = compute_dtype if compute_dtype is not None else (torch.bfloat16 if G.is_cuda else None)
    X, transposed, _ = _orient(G, eps, dtype)
    for a, b, c in coefs:
        A = X @ X.T
        B = torch.addmm(A, A, A, beta=b, alpha=c)
        X = torch.addmm(X, B, X, beta=a)
    if transposed:
        X = X.T
    return X.to(G.dtype).reshape(G.shape)


def _gram_iteration(X: Tensor, coefs, restarts) -> tuple[list[Tensor], Tensor]:
    """Run the Gram recurrence on an oriented, normalised ``X``.  Returns the
    left-factor segments (one per restart window) and the final ``Q X``."""
    m = X.shape[0]
    eye = torch.eye(m, device=X.device, dtype=X.dtype)
    R = X @ X.T
    Q: Optional[Tensor] = None
    segments: list[Tensor] = []
    last = len(coefs) - 1
    for i, (a, b, c) in enumerate(coefs):
        if i in restarts and i != 0:
            X = Q @ X
            R = X @ X.T
            segments.append(Q)
            Q = None
        P = torch.addmm(R, R, R, beta=b, alpha=c) + a * eye
        Q = P if Q is None else P @ Q
        if i < last and (i + 1) not in restarts:
            RP = R @ P
            R = RP @ P
    segments.append(Q)
    return segments, Q @ X


def gram_newton_schulz(
    G: Tensor,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    restart_iterations: Optional[Sequence[int]] = None,
    deterministic: bool = False,
    compute_dtype: Optional[torch.dtype] = None,
) -> Tensor:
    """Gram-space iteration.  The iteration count is ``len(coefficients)``;
    ``steps`` is accepted for signature parity and otherwise unused, as in the
    reference (dmuon/optim/newton_schulz.py:315)."""
    coefs = _coeffs(coefficients, steps)
    restarts = list(DEFAULT_RESTART_ITERATIONS if restart_iterations is None else restart_iterations)
    if G.is_cuda and not deterministic:
        from ..ops import ns_sm100

        if ns_sm100.available():
            return ns_sm100.newton_schulz_single(G, coefs, restarts, eps, "gram", compute_dtype)
    dtype = compute_dtype if compute_dtype is not None else (torch.float16 if G.is_cuda else None)
    X, transposed, _ = _orient(G, eps, dtype)
    _, out = _gram_iteration(X, coefs, restarts)
    if transposed:
        out = out.T
    return out.to(G.dtype).reshape(G.shape)


def gram_newton_schulz_factors(
    G: Tensor,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    restart_iterations: Optional[Sequence[int]] = None,
    deterministic: bool = False,
    compute_dtype: Optional[torch.dtype] = None,
) -> tuple[tuple[Tensor, ...], bool, Tensor]:
    """``(segments, transposed, normalizer)``: applying the segments in order
    to the oriented ``G / normalizer`` reproduces :func:`gram_newton_schulz`."""
    coefs = _coeffs(coefficients, steps)
    restarts = list(DEFAULT_RESTART_ITERATIONS if restart_iterations is None else restart_iterations)
    dtype = compute_dtype if compute_dtype is not None else (torch.float16 if G.is_cuda else None)
    X, transposed, norm = _orient(G, eps, dtype)
    segments, _ = _gram_iteration(X, coefs, restarts)
    return tuple(s.clone() for s in segments), transposed, norm


gram_newton_schulz_q = gram_newton_schulz_factors


def apply_gram_factors(G: Tensor, segments: Sequence[Tensor], transposed: bool, normalizer: Tensor) -> Tensor:
    """Apply factor segments to (a column shard of) the oriented matrix."""
    X = G.float()
    if transposed:
        X = X.T
    X = (X / normalizer).to(segments[0].dtype)
    for Q in segments:
        X = Q @ X
    if transposed:
        X = X.T
    return X.to(G.dtype)


def _multi_rank(group) -> bool:
    return group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def gram_newton_schulz_distributed_local_batched(
    G_local: Tensor,
    group,
    *,
    transposed: bool,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    restart_iterations: Optional[Sequence[int]] = None,
) -> Tensor:
    """Gram iteration on column shards ``[batch, rows, cols]`` of the oriented
    matrices: the squared norm and every Gram matrix are summed over ``group``
    (fp32 on the wire), the full matrix is never gathered."""
    if G_local.dim() != 3:
        raise ValueError(
            "gram_newton_schulz_distributed_local_batched expects a 3D [batch, rows, cols] tensor, "
            f"got shape={tuple(G_local.shape)}"
        )
    coefs = _coeffs(coefficients, steps)
    restarts = list(DEFAULT_RESTART_ITERATIONS if restart_iterations is None else restart_iterations)
    multi = _multi_rank(group)
    X = G_local.float()
    if transposed:
        X = X.transpose(1, 2)
    sq = (X * X).sum(dim=(1, 2))
    if multi:
        dist.all_reduce(sq, group=group)
    X = X / (sq.sqrt() + eps).view(-1, 1, 1)
    work = torch.float16 if G_local.is_cuda else torch.float32
    X = X.to(work).contiguous()

    def gram(x: Tensor) -> Tensor:
        r = torch.bmm(x, x.transpose(1, 2)).float()
        if multi:
            dist.all_reduce(r, group=group)
        return r.to(work)

    m = X.shape[1]
    eye = torch.eye(m, device=X.device, dtype=work).expand(X.shape[0], m, m)
    R = gram(X)
    Q = None
    last = len(coefs) - 1
    for i, (a, b, c) in enumerate(coefs):
        if i in restarts and i != 0:
            X = torch.bmm(Q, X)
            R = gram(X)
            Q = None
        P = torch.baddbmm(R, R, R, beta=b, alpha=c) + a * eye
        Q = P if Q is None else torch.bmm(P, Q)
        if i < last and (i + 1) not in restarts:
            R = torch.bmm(torch.bmm(R, P), P)
    X = torch.bmm(Q, X)
    if transposed:
        X = X.transpose(1, 2)
    return X.to(G_local.dtype)


def gram_newton_schulz_distributed_local(
    G_local: Tensor,
    group,
    *,
    transposed: bool,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    restart_iterations: Optional[Sequence[int]] = None,
) -> Tensor:
    return gram_newton_schulz_distributed_local_batched(
        G_local.unsqueeze(0),
        group,
        transposed=transposed,
        steps=steps,
        eps=eps,
        coefficients=coefficients,
        restart_iterations=restart_iterations,
    ).squeeze(0)


def newton_schulz(
    G: Tensor,
    steps: int = 5,
    eps: float = 1e-7,
    coefficients: Optional[Sequence[Sequence[float]]] = None,
    restart_iterations: Optional[Sequence[int]] = None,
    backend: str = "gram",
    **kwargs,
) -> Tensor:
    """Orthogonalise ``G`` with the default coefficients (positional arguments
    as in the reference, dmuon/optim/newton_schulz.py:299); ``backend`` is
    ``"gram"`` or ``"direct"``."""
    if backend == "gram":
        return gram_newton_schulz(G, steps=steps, eps=eps, coefficients=coefficients,
                                  restart_iterations=restart_iterations, **kwargs)
    if backend == "direct":
        return direct_newton_schulz(G, steps=steps, eps=eps, coefficients=coefficients, **kwargs)
    raise ValueError(f"backend must be 'gram' or 'direct', got {backend!r}")


gram_newton_schulz_local = gram_newton_schulz      # alias kept by the reference (dmuon/optim/newton_schulz.py:779)


class NewtonSchulz:
    """Configuration object handed to ``Muon(ns_backend=...)``.

    ``backend``            "gram" (default) or "direct"
    ``kernel``             "auto" / "tcgen05" run the sm_100a kernels on CUDA
                           tensors, "torch" forces the plain PyTorch path.  The
                           reference's backend names ("quack", "cute_sm80",
                           "cublas", "compile") are accepted and mean "auto":
                           there is one GPU implementation here, not a
                           dispatch between several.
    ``coefficients``       per-step triples, default Polar Express / 1.05
    ``restart_iterations`` Gram restarts, default ``[2]``
    ``deterministic``      force the PyTorch path (library GEMMs)
    ``compute_dtype``      operand dtype of the products: bf16 (default on
                           CUDA) or fp16
    """

    def __init__(
        self,
        backend: str = "gram",
        kernel: str = "auto",
        coefficients: Optional[Sequence[Sequence[float]]] = None,
        restart_iterations: Optional[Sequence[int]] = None,
        deterministic: bool = False,
        compute_dtype: Optional[torch.dtype] = None,
    ):
        if backend not in ("gram", "direct"):
            raise ValueError(f"backend must be 'gram' or 'direct', got '{backend}'")
        k = str(kernel).strip().lower()
        if k == "auto":
            # as in the reference: the environment variable is consulted only when the argument says "auto"
            env = __import__("os").environ.get("DMUON_NS_KERNEL", "").strip().lower()
            if env:
                if env not in _KERNEL_NAMES + _LEGACY_KERNELS:
                    raise ValueError(
                        f"DMUON_NS_KERNEL={env!r} is not valid; choose one of: {', '.join(_KERNEL_NAMES + _LEGACY_KERNELS)}")
                k = env
        if k in _LEGACY_KERNELS:
            log.info("NewtonSchulz: kernel=%r names a backend of the reference; using the sm_100a kernels", kernel)
            if k == "cublas":
                deterministic = True
            k = "auto"
        if k not in _KERNEL_NAMES:
            raise ValueError(f"kernel={kernel!r} is not valid; choose one of: {', '.join(_KERNEL_NAMES)}")
        if compute_dtype not in (None, torch.bfloat16, torch.float16, torch.float32):
            raise ValueError("compute_dtype must be torch.bfloat16, torch.float16 or torch.float32")
        self.backend = backend
        self.kernel = "torch" if (deterministic or k == "torch") else "tcgen05"
        self.coefficients = None if coefficients is None else [tuple(c) for c in coefficients]
        self.restart_iterations = None if restart_iterations is None else list(restart_iterations)
        self.deterministic = bool(deterministic) or k == "torch"
        self.compute_dtype = compute_dtype
        _ACTIVE["backend"] = backend
        _ACTIVE["kernel"] = self.kernel

    def resolved_coefficients(self, steps: int):
        coefs = list(DEFAULT_COEFFICIENTS) if self.coefficients is None else list(self.coefficients)
        if self.backend == "direct":
            coefs = coefs[: max(1, steps)]
        return coefs

    def resolved_restarts(self) -> list[int]:
        if self.backend == "direct":
            return []
        return list(DEFAULT_RESTART_ITERATIONS if self.restart_iterations is None else self.restart_iterations)

    def uses_kernels(self, t: Tensor) -> bool:
        if self.deterministic or not t.is_cuda:
            return False
        from ..ops import ns_sm100

        return ns_sm100.available()

    def local(self, G: Tensor, steps: int) -> Tensor:
        """Orthogonalise one full matrix."""
        if self.uses_kernels(G):
            from ..ops import ns_sm100
            from . import ns_graph

            coefs, restarts = self.resolved_coefficients(steps), self.resolved_restarts()

            def run(x: Tensor) -> Tensor:
                return ns_sm100.newton_schulz_single(x, coefs, restarts, 1e-7, self.backend, self.compute_dtype)

            if ns_graph.enabled() and not torch.cuda.is_current_stream_capturing():
                key = (
                    tuple(G.shape), G.dtype, G.device.index, self.backend, self.compute_dtype,
                    tuple(map(tuple, coefs)), tuple(restarts),
                )
                return ns_graph.cache().run(key, run, G)
            return run(G)
        if self.backend == "gram":
            return gram_newton_schulz(
                G,
                steps=steps,
                coefficients=self.coefficients,
                restart_iterations=self.restart_iterations,
                deterministic=True,
                compute_dtype=self.compute_dtype,
            )
        return direct_newton_schulz(G, steps=steps, coefficients=self.coefficients, compute_dtype=self.compute_dtype)

    def __repr__(self) -> str:
        coeff = "default" if self.coefficients is None else f"{len(self.coefficients)}-step custom"
        return f"NewtonSchulz(backend={self.backend!r}, kernel={self.kernel!r}, coefficients={coeff})"


_ACTIVE = {"backend": "gram", "kernel": "tcgen05"}


def get_ns_backend() -> str:
    """Name of the Newton-Schulz implementation CUDA tensors get."""
    from ..ops import ns_sm100

    if _ACTIVE["kernel"] == "torch" or not ns_sm100.available():
        return "torch"
    return "tcgen05"


def get_backend_status() -> dict:
    from ..ops import build as _build
    from ..ops import ns_sm100
    from . import ns_graph

    return {
        "cuda_graph_replay": ns_graph.enabled(),
        "cuda_graph_cache": ns_graph.cache().stats(),
        "ns_backend": get_ns_backend(),
        "formulation": _ACTIVE["backend"],
        "arch": "sm_100a",
        "kernel_library": str(_build.LIBPATH),
        "kernel_library_built": _build.LIBPATH.exists(),
        "kernel_library_loaded": _build.is_loaded(),
        "cuda_available": torch.cuda.is_available(),
        "kernels_usable": ns_sm100.available(),
    }

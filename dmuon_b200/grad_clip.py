"""Global-norm clipping of the gradients Muon owns.

``clip_grad_norm_(optimizer, max_norm)`` touches only the reduced gradients of
owned matrices on the ``muon`` route (the full gathered matrix on a
tensor-parallel owner, nothing on its TP peers); ordinary ``param.grad``
tensors stay with ``torch.nn.utils.clip_grad_norm_``.  The call never reads a
value back to the host: norm, coefficient, ``clipped`` and ``found_inf`` stay
0-dim device tensors, and the gradients are always multiplied by the clamped
coefficient (no host branch).  Reference: dmuon/grad_clip.py:40-75, :103-200,
:243-321.

On a B200 the 2-norm runs through the segmented sum-of-squares kernel (one
pass over the gradients) and the scaling through the in-place scale kernel; the
scalar all-reduce is the only collective.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Protocol

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class MuonGradClipEntry:
    name: str
    grad: torch.Tensor
    shape: tuple[int, ...]
    is_tp_full_grad: bool = False


@dataclass(frozen=True)
class MuonGradClipStats:
    total_norm: torch.Tensor
    max_norm: Optional[float]
    norm_type: float
    clip_coef: Any
    clipped: Any
    param_count: int
    found_inf: torch.Tensor
    strategy: str = "global_norm"

    def as_dict(self) -> dict[str, Any]:
        return {k: getattr(self, k) for k in self.__dataclass_fields__}


@dataclass(frozen=True)
class MuonGradClipContext:
    optimizer: Any
    entries: tuple[MuonGradClipEntry, ...]
    max_norm: Optional[float]
    norm_type: float
    error_if_nonfinite: bool
    foreach: Optional[bool] = None


class MuonGradClipStrategy(Protocol):
    name: str

    def __call__(self, context: MuonGradClipContext) -> MuonGradClipStats: ...


def iter_muon_grad_entries(optimizer):
    """Owned Muon gradients as the optimizer will consume them."""
    for dp in optimizer.owned_muon_params():
        if dp.tp_group is not None:
            if dp.is_tp_owner and dp._tp_full_grad is not None:
                yield MuonGradClipEntry(dp.fqn, dp._tp_full_grad, tuple(dp.full_shape), True)
        elif dp._reduced_grad is not None:
            yield MuonGradClipEntry(dp.fqn, dp._reduced_grad, tuple(dp._orig_size), False)


def _device_of(optimizer, entries) -> torch.device:
    return entries[0].grad.device if entries else optimizer.device


def _use_kernels(t: torch.Tensor) -> bool:
    if not t.is_cuda:
        return False
    from .ops import ns_sm100

    return ns_sm100.available()


def local_pow_sum(grads: list[torch.Tensor], norm_type: float, device: torch.device) -> torch.Tensor:
    """sum |g|^p over the local tensors (max |g| for p = inf), fp32, 0-dim."""
    if not grads:
        return torch.zeros((), dtype=torch.float32, device=device)
    if norm_type == float("inf"):
        return torch.stack([g.detach().abs().max().float() for g in grads]).max()
    if norm_type == 2.0 and _use_kernels(grads[0]):
        from .ops import multi_tensor as MT

        acc = torch.zeros(1, dtype=torch.float32, device=device)
        flat = [g if g.is_contiguous() else g.contiguous() for g in grads]
        MT.clip_sumsq(flat, [0] * len(flat), acc)
        return acc[0]
    norms = torch._foreach_norm([g.detach().float() for g in grads], norm_type)
    return torch.stack(norms).pow(norm_type).sum()


def _peer_plane(optimizer):
    """The peer runtime when its ranks are the whole job (then its in-kernel
    scalar sum can stand in for the world all-reduce of the norm)."""
    rt = getattr(getattr(optimizer, "comm_ctx", None), "peer_runtime", None)
    if rt is None or not (dist.is_available() and dist.is_initialized()):
        return None
    return rt if dist.get_world_size() == rt.world else None


def global_norm(local: torch.Tensor, norm_type: float, group=None, optimizer=None) -> torch.Tensor:
    rt = _peer_plane(optimizer) if (norm_type == 2.0 and local.is_cuda) else None
    if rt is not None:
        sums, _ = rt.scalar_allreduce(local.reshape(1))
        return sums[0].sqrt()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        local = local.clone()
        op = dist.ReduceOp.MAX if norm_type == float("inf") else dist.ReduceOp.SUM
        dist.all_reduce(local, op=op, group=group)
    return local if norm_type == float("inf") else local.pow(1.0 / norm_type)


def scale_grads_(grads: list[torch.Tensor], coef: torch.Tensor) -> None:
    if not grads:
        return
    if _use_kernels(grads[0]) and all(g.is_contiguous() for g in grads):
        from .ops import multi_tensor as MT

        MT.clip_scale(grads, [0] * len(grads), coef.reshape(1).float())
        return
    for g in grads:
        g.mul_(coef.to(g.dtype))


class GlobalNormMuonClipStrategy:
    name = "global_norm"

    @torch.no_grad()
    def __call__(self, context: MuonGradClipContext) -> MuonGradClipStats:
        entries = context.entries
        device = _device_of(context.optimizer, entries)
        grads = [e.grad for e in entries]
        total = global_norm(local_pow_sum(grads, context.norm_type, device), context.norm_type,
                            optimizer=context.optimizer)
        if context.error_if_nonfinite and not bool(torch.isfinite(total)):
            raise RuntimeError(f"the total norm of order {context.norm_type} of the Muon gradients is non-finite")
        coef: Any = 1.0
        clipped: Any = False
        if context.max_norm is not None:
            if context.max_norm < 0:
                raise ValueError(f"max_norm must be non-negative, got {context.max_norm}")
            raw = float(context.max_norm) / (total + 1e-6)
            coef_t = torch.clamp(raw, max=1.0)
            scale_grads_(grads, coef_t)
            coef = coef_t.detach()
            clipped = torch.isfinite(total) & (raw < 1.0)
        return MuonGradClipStats(
            total_norm=total.detach(),
            max_norm=context.max_norm,
            norm_type=context.norm_type,
            clip_coef=coef,
            clipped=clipped,
            param_count=len(entries),
            found_inf=~torch.isfinite(total),
            strategy=self.name,
        )


_STRATEGIES: dict[str, Any] = {GlobalNormMuonClipStrategy.name: GlobalNormMuonClipStrategy()}


def register_muon_grad_clip_strategy(name: str, strategy) -> None:
    """Register a custom strategy; it receives the live gradient tensors and may
    inspect or scale them in place."""
    if not name:
        raise ValueError("strategy name must be non-empty")
    _STRATEGIES[name] = strategy


def clip_grad_norm_(
    optimizer,
    max_norm: Optional[float],
    *,
    norm_type: float = 2.0,
    error_if_nonfinite: bool = False,
    foreach: Optional[bool] = None,
    strategy="global_norm",
) -> MuonGradClipStats:
    """``max_norm=None`` only measures.  Every rank must call this (the scalar
    all-reduce spans the world), owners and non-owners alike."""
    if not hasattr(optimizer, "_ensure_grads_ready") or not hasattr(optimizer, "owned_muon_params"):
        raise TypeError("clip_grad_norm_ expects a dmuon_b200.Muon optimizer")
    optimizer._ensure_grads_ready(materialize=True)
    if isinstance(strategy, str):
        if strategy not in _STRATEGIES:
            raise ValueError(f"unknown Muon grad clip strategy {strategy!r}; registered: {sorted(_STRATEGIES)}")
        fn = _STRATEGIES[strategy]
    else:
        fn = strategy
    ctx = MuonGradClipContext(
        optimizer=optimizer,
        entries=tuple(iter_muon_grad_entries(optimizer)),
        max_norm=max_norm,
        norm_type=float(norm_type),
        error_if_nonfinite=error_if_nonfinite,
        foreach=foreach,
    )
    stats = fn(ctx)
    optimizer._last_clip_stats = stats
    return stats

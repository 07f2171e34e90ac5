"""Segmented gradient clipping: several independently clipped buckets, one
collective.

Each bucket (for example "regular" FSDP gradients, "muon" owned gradients,
"adamw" dedicated AdamW gradients) gets its own 2-norm and its own clip
coefficient.  The local sums of squares of all buckets are computed by one
multi-tensor kernel pass, all-reduced as ONE small vector (entries of buckets
with ``reduce=False`` are kept local), and the gradients are scaled in place by
a second kernel pass.  Whether a tensor takes the kernel or the PyTorch path is
a purely local decision and never changes the number of collectives, so ranks
stay in lockstep.  Same stages and result types as the reference
(dmuon/fast_clip.py:40-92, :382-436, :439-493; kernels
dmuon/csrc/fast_clip_kernel.cu:34-106).
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .grad_clip import MuonGradClipStats, iter_muon_grad_entries


@dataclass(frozen=True)
class GradClipBucket:
    name: str
    grads: Sequence[torch.Tensor]
    reduce: bool = True


@dataclass(frozen=True)
class GradClipBucketStats:
    name: str
    total_norm: torch.Tensor
    max_norm: Optional[float]
    clip_coef: torch.Tensor
    clipped: torch.Tensor
    param_count: int
    found_inf: torch.Tensor
    fastpath: bool

    def as_dict(self) -> dict[str, object]:
        return {k: getattr(self, k) for k in self.__dataclass_fields__}


@dataclass(frozen=True)
class SegmentedGradClipResult:
    total_norm: torch.Tensor
    bucket_stats: tuple[GradClipBucketStats, ...]
    fastpath: bool
    fallback_reason: Optional[str] = None

    @property
    def stats_by_name(self) -> dict[str, GradClipBucketStats]:
        return {s.name: s for s in self.bucket_stats}


def fast_clip_enabled() -> bool:
    """``DMUON_FAST_CLIP=0`` sends every tensor through the PyTorch path
    (reference toggle: dmuon/fast_clip.py:105)."""
    return os.environ.get("DMUON_FAST_CLIP", "1").strip().lower() not in ("0", "false", "no", "off")


def _verbose() -> bool:
    return os.environ.get("DMUON_FAST_CLIP_VERBOSE", "0").strip().lower() in ("1", "true", "yes", "on")


def _kernels_usable(device: torch.device) -> tuple[bool, Optional[str]]:
    """(use the kernels?, why not).  With ``DMUON_FAST_CLIP_VERBOSE=1`` a kernel
    library that cannot be loaded on a CUDA device raises instead of degrading
    (reference dmuon/fast_clip.py:106-129)."""
    if device.type != "cuda":
        return False, "gradients are not on a CUDA device"
    if not fast_clip_enabled():
        return False, "disabled by DMUON_FAST_CLIP=0"
    from .ops import ns_sm100

    try:
        ok = ns_sm100.available()
    except Exception as exc:
        if _verbose():
            raise
        return False, f"kernel library unavailable: {exc}"
    return ok, None if ok else "sm_100a kernels unavailable on this device"


def _local(t: torch.Tensor) -> torch.Tensor:
    return getattr(t, "_local_tensor", t)


def _device(buckets: Sequence[GradClipBucket]) -> torch.device:
    for b in buckets:
        for g in b.grads:
            return _local(g).device
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def _eligible(g: torch.Tensor) -> bool:
    return g.is_cuda and g.is_contiguous() and g.dtype in (torch.float32, torch.float16, torch.bfloat16)


def _local_sumsq(buckets, device, fast: bool) -> torch.Tensor:
    acc = torch.zeros(len(buckets), dtype=torch.float32, device=device)
    k_t, k_s = [], []
    for i, b in enumerate(buckets):
        for g in b.grads:
            g = _local(g).detach()
            if g.numel() == 0:
                continue
            if fast and _eligible(g):
                k_t.append(g)
                k_s.append(i)
            else:
                acc[i] += g.float().pow(2).sum()
    if k_t:
        from .ops import multi_tensor as MT

        MT.clip_sumsq(k_t, k_s, acc)
    return acc


def _scale(buckets, coefs: torch.Tensor, fast: bool) -> None:
    k_t, k_s = [], []
    for i, b in enumerate(buckets):
        for g in b.grads:
            g = _local(g).detach()
            if g.numel() == 0:
                continue
            if fast and _eligible(g):
                k_t.append(g)
                k_s.append(i)
            else:
                g.mul_(coefs[i].to(g.dtype))
    if k_t:
        from .ops import multi_tensor as MT

        MT.clip_scale(k_t, k_s, coefs)


@torch.no_grad()
def clip_grad_norm_buckets_(
    buckets: Sequence[GradClipBucket],
    max_norm: Optional[float],
    *,
    process_group=None,
    chunk_size: Optional[int] = None,
) -> SegmentedGradClipResult:
    # The kernels size their own grid (one launch per ~320 tensors, 128-bit accesses), so the
    # reference's per-job chunk length (``chunk_size`` / ``DMUON_FAST_CLIP_CHUNK_SIZE``) has nothing to
    # tune here; both are accepted and validated so that callers and launch scripts carry over.
    if chunk_size is None and os.environ.get("DMUON_FAST_CLIP_CHUNK_SIZE"):
        chunk_size = int(os.environ["DMUON_FAST_CLIP_CHUNK_SIZE"])
    if chunk_size is not None and int(chunk_size) < 1:
        raise ValueError("chunk_size must be positive")
    buckets = tuple(buckets)
    device = _device(buckets)
    fast, why_not = _kernels_usable(device)
    local = _local_sumsq(buckets, device, fast)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(process_group) > 1:
        mask = torch.tensor([1.0 if b.reduce else 0.0 for b in buckets], dtype=torch.float32, device=device)
        summed = local * mask
        dist.all_reduce(summed, group=process_group)
        global_sq = summed + local * (1.0 - mask)
    else:
        global_sq = local
    norms = global_sq.sqrt()
    if max_norm is None:
        raw = torch.full_like(norms, float("inf"))
        coefs = torch.ones_like(norms)
    else:
        raw = float(max_norm) / (norms + 1e-6)
        coefs = raw.clamp(max=1.0)
        _scale(buckets, coefs, fast)
    finite = torch.isfinite(norms)
    stats = tuple(
        GradClipBucketStats(
            name=b.name,
            total_norm=norms[i],
            max_norm=max_norm,
            clip_coef=coefs[i],
            clipped=finite[i] & (raw[i] < 1.0),
            param_count=len(b.grads),
            found_inf=~finite[i],
            fastpath=fast,
        )
        for i, b in enumerate(buckets)
    )
    return SegmentedGradClipResult(
        total_norm=torch.linalg.vector_norm(norms, 2.0),
        bucket_stats=stats,
        fastpath=fast,
        fallback_reason=why_not,
    )


@torch.no_grad()
def try_clip_optimizer_grad_norm_buckets_(
    optimizer,
    *,
    regular_grads: Sequence[torch.Tensor],
    adamw_grads: Sequence[torch.Tensor],
    max_norm: float,
    process_group=None,
) -> Optional[SegmentedGradClipResult]:
    """Clip "regular" (already-reduced FSDP/DDP, local only), "muon" and
    dedicated-"adamw" gradients in one call.  Returns ``None`` when ``optimizer``
    is not a Muon optimizer of this package."""
    ensure = getattr(optimizer, "_ensure_grads_ready", None)
    if ensure is None or not hasattr(optimizer, "owned_muon_params"):
        return None
    ensure(materialize=True)
    muon =[e.grad for e in iter_muon_grad_entries(optimizer)]
    res = clip_grad_norm_buckets_(
        (
            GradClipBucket("regular", regular_grads, reduce=False),
            GradClipBucket("muon", muon, reduce=True),
            GradClipBucket("adamw", adamw_grads, reduce=True),
        ),
        max_norm,
        process_group=process_group,
    )
    ms = res.stats_by_name["muon"]
    optimizer._last_clip_stats = MuonGradClipStats(
        total_norm=ms.total_norm,
        max_norm=ms.max_norm,
        norm_type=2.0,
        clip_coef=ms.clip_coef,
        clipped=ms.clipped,
        param_count=ms.param_count,
        found_inf=ms.found_inf,
        strategy="segmented_sm100_kernels" if res.fastpath else "segmented_torch",
    )
    return res

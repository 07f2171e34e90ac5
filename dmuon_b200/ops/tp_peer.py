"""ctypes front end of the tensor-parallel gather / scatter kernels
(``csrc/tp_peer_sm100.cu``)."""
from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import Optional, Sequence

import torch

from . import build as _build
from .multi_tensor import _DT, MAX_TENSORS, _check, _chunks, _stream

_VP = ctypes.c_void_p * MAX_TENSORS
_LL = ctypes.c_longlong * MAX_TENSORS
_IA = ctypes.c_int * MAX_TENSORS
_FA = ctypes.c_float * MAX_TENSORS


class _GatherArgs(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("mom", _VP), ("x", _VP), ("rows", _IA), ("cols", _IA), ("pitch", _LL), ("slot", _IA),
        ("n", ctypes.c_int), ("src_dtype", ctypes.c_int), ("mom_dtype", ctypes.c_int), ("x_dtype", ctypes.c_int),
        ("mu", ctypes.c_float), ("nesterov", ctypes.c_int), ("gscale", ctypes.c_void_p), ("sumsq", ctypes.c_void_p),
        ("xscale", ctypes.c_void_p),
    ]


class _ApplyArgs(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("dst", _VP), ("rows", _IA), ("cols", _IA), ("pitch", _LL), ("decay", _FA),
        ("n", ctypes.c_int), ("dst_dtype", ctypes.c_int),
    ]


@lru_cache(maxsize=None)
def _lib():
    lib = _build.load()
    for name, typ in (("dmuon_tp_gather_prologue", _GatherArgs), ("dmuon_tp_apply_delta", _ApplyArgs)):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(typ), ctypes.c_void_p]
        fn.restype = ctypes.c_int
    return lib


class ShardJob:
    """One shard of one matrix: where it is read (``src``: address of a
    contiguous ``rows x cols`` block, local or peer-mapped) and where it sits in
    the full matrix (element offset ``dst_offset``, row pitch ``pitch``);
    ``index`` names the matrix of the batch it belongs to."""

    __slots__ = ("index", "src", "rows", "cols", "dst_offset", "pitch")

    def __init__(self, index: int, src: int, rows: int, cols: int, dst_offset: int, pitch: int):
        self.index, self.src, self.rows, self.cols = int(index), int(src), int(rows), int(cols)
        self.dst_offset, self.pitch = int(dst_offset), int(pitch)


def gather_prologue(
    jobs: Sequence[ShardJob],
    src_dtype: torch.dtype,
    moms: Sequence[Optional[torch.Tensor]],
    xs: Sequence[torch.Tensor],
    slots: Sequence[int],
    sumsq: Optional[torch.Tensor],
    *,
    mu: float,
    nesterov: bool,
    gscale: Optional[torch.Tensor] = None,
    xscale: Optional[torch.Tensor] = None,
) -> None:
    """Momentum / Nesterov / cast / sum of squares of full matrices whose
    gradient arrives as shards (``jobs``): every shard is read where it lies --
    on this GPU or, through its peer mapping, on another one -- and written into
    the rows / columns it occupies in ``moms[i]`` and ``xs[i]`` (full matrices,
    row-major, contiguous).  ``moms[i] is None`` for all ``i`` switches the
    momentum off (``x = cast(g)``)."""
    if not jobs:
        return
    dev = xs[0].device
    has_mom = moms[0] is not None
    md = moms[0].dtype if has_mom else torch.float32
    xd = xs[0].dtype
    for lo, hi in _chunks(len(jobs)):
        a = _GatherArgs()
        for k, job in enumerate(jobs[lo:hi]):
            x = xs[job.index]
            assert x.dtype == xd and x.is_contiguous()
            a.src[k] = job.src
            a.x[k] = x.data_ptr() + job.dst_offset * x.element_size()
            if has_mom:
                m = moms[job.index]
                assert m.dtype == md and m.is_contiguous() and m.numel() == x.numel()
                a.mom[k] = m.data_ptr() + job.dst_offset * m.element_size()
            a.rows[k], a.cols[k], a.pitch[k], a.slot[k] = job.rows, job.cols, job.pitch, int(slots[job.index])
        a.n = hi - lo
        a.src_dtype, a.mom_dtype, a.x_dtype = _DT[src_dtype], _DT[md], _DT[xd]
        a.mu, a.nesterov = float(mu), int(bool(nesterov))
        a.gscale = gscale.data_ptr() if gscale is not None else None
        a.sumsq = sumsq.data_ptr() if sumsq is not None else None
        a.xscale = xscale.data_ptr() if xscale is not None else None
        _check(_lib().dmuon_tp_gather_prologue(ctypes.byref(a), _stream(dev)), "dmuon_tp_gather_prologue")


def apply_delta(
    srcs: Sequence[int],
    pitches: Sequence[int],
    dsts: Sequence[torch.Tensor],
    decays: Sequence[float],
) -> None:
    """``dsts[i] = dsts[i] * decays[i] + slice_i`` where ``slice_i`` is the
    ``rows x cols`` block (shape of ``dsts[i]`` viewed as a matrix) that starts
    at address ``srcs[i]`` inside an fp32 matrix with row pitch ``pitches[i]``
    -- the owner's pre-scaled update, read through its peer mapping."""
    n = len(srcs)
    if n == 0:
        return
    dev = dsts[0].device
    dd = dsts[0].dtype
    for lo, hi in _chunks(n):
        a = _ApplyArgs()
        for i in range(lo, hi):
            k = i - lo
            d = dsts[i]
            assert d.dtype == dd and d.is_contiguous()
            rows = int(d.shape[0])
            a.src[k], a.dst[k] = int(srcs[i]), d.data_ptr()
            a.rows[k], a.cols[k], a.pitch[k], a.decay[k] = rows, d.numel() // rows, int(pitches[i]), float(decays[i])
        a.n, a.dst_dtype = hi - lo, _DT[dd]
        _check(_lib().dmuon_tp_apply_delta(ctypes.byref(a), _stream(dev)), "dmuon_tp_apply_delta")

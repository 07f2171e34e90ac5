"""ctypes front end of the peer-memory kernels (``csrc/peer_sm100.cu``)."""
from __future__ import annotations

import ctypes
import os
from functools import lru_cache
from typing import Optional, Sequence

import torch

from . import build as _build
from .multi_tensor import _DT, MAX_TENSORS, _check, _chunks, _stream

MAX_PEERS = 8
_VP = ctypes.c_void_p * MAX_TENSORS
_LL = ctypes.c_longlong * MAX_TENSORS
_IA = ctypes.c_int * MAX_TENSORS
_PP = ctypes.c_void_p * MAX_PEERS


class _SignalArgs(ctypes.Structure):
    _fields_ = [("peer_flags", _PP), ("world", ctypes.c_int), ("slot", ctypes.c_int), ("value", ctypes.c_int)]


class _WaitArgs(ctypes.Structure):
    _fields_ = [
        ("local_flags", ctypes.c_void_p), ("first", ctypes.c_int), ("count", ctypes.c_int), ("want", ctypes.c_int),
        ("budget_cycles", ctypes.c_longlong), ("status", ctypes.c_void_p),
    ]


class _PeerPrologueArgs(ctypes.Structure):
    _fields_ = [
        ("peer_base", _PP), ("world", ctypes.c_int), ("scale", ctypes.c_float),
        ("offset", _LL), ("mom", _VP), ("x", _VP), ("numel", _LL), ("slot", _IA),
        ("n", ctypes.c_int), ("grad_dtype", ctypes.c_int), ("mom_dtype", ctypes.c_int), ("x_dtype", ctypes.c_int),
        ("mu", ctypes.c_float), ("nesterov", ctypes.c_int), ("gscale", ctypes.c_void_p), ("sumsq", ctypes.c_void_p),
        ("ready_flags", ctypes.c_void_p), ("ready_want", ctypes.c_int), ("budget_cycles", ctypes.c_longlong),
        ("status", ctypes.c_void_p), ("max_blocks_per_tensor", ctypes.c_int), ("xscale", ctypes.c_void_p),
    ]


class _MulticastArgs(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("dst", _VP), ("nbytes", _LL), ("n", ctypes.c_int), ("mode", ctypes.c_int),
        ("dtype", ctypes.c_int), ("blocks_per_tensor", ctypes.c_int),
    ]


class _PullArgs(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("dst", _VP), ("nbytes", _LL), ("flag_slot", _IA), ("n", ctypes.c_int),
        ("local_flags", ctypes.c_void_p), ("want", ctypes.c_int), ("budget_cycles", ctypes.c_longlong),
        ("status", ctypes.c_void_p), ("blocks_per_tensor", ctypes.c_int),
    ]


@lru_cache(maxsize=None)
def _lib():
    lib = _build.load()
    for name, typ in (
        ("dmuon_signal_peers", _SignalArgs),
        ("dmuon_wait_flags", _WaitArgs),
        ("dmuon_peer_prologue", _PeerPrologueArgs),
        ("dmuon_peer_pull", _PullArgs),
        ("dmuon_multicast_copy", _MulticastArgs),
    ):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(typ), ctypes.c_void_p]
        fn.restype = ctypes.c_int
    lib.dmuon_copy_async.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    lib.dmuon_copy_async.restype = ctypes.c_int
    return lib


SCALAR_MAX = 8


class _ScalarAllreduceArgs(ctypes.Structure):
    _fields_ = [
        ("peer_vals", _PP), ("peer_flags", _PP),
        ("world", ctypes.c_int), ("rank", ctypes.c_int), ("n", ctypes.c_int), ("epoch", ctypes.c_int),
        ("local", ctypes.c_void_p), ("out", ctypes.c_void_p), ("coef", ctypes.c_void_p),
        ("max_norm", ctypes.c_float), ("budget_cycles", ctypes.c_longlong), ("status", ctypes.c_void_p),
    ]


def scalar_allreduce(
    peer_vals: Sequence[int], peer_flags: Sequence[int], rank: int, epoch: int, local: torch.Tensor, out: torch.Tensor,
    status: torch.Tensor, coef: Optional[torch.Tensor] = None, max_norm: float = 0.0,
    budget_cycles: Optional[int] = None,
) -> None:
    """``out[i] = sum over ranks of local[i]`` (fp32, rank order, identical bits
    everywhere) in one single-warp kernel over symmetric scratch rows; with
    ``coef`` also ``coef[i] = min(1, max_norm / (sqrt(out[i]) + 1e-6))``."""
    a = _ScalarAllreduceArgs()
    world = len(peer_vals)
    for r in range(world):
        a.peer_vals[r], a.peer_flags[r] = int(peer_vals[r]), int(peer_flags[r])
    a.world, a.rank, a.n, a.epoch = world, int(rank), int(local.numel()), int(epoch)
    assert local.dtype == out.dtype == torch.float32 and local.is_contiguous() and out.numel() >= local.numel()
    a.local, a.out = local.data_ptr(), out.data_ptr()
    a.coef = coef.data_ptr() if coef is not None else None
    a.max_norm = float(max_norm)
    a.budget_cycles = int(budget_cycles if budget_cycles is not None else wait_budget_cycles())
    a.status = status.data_ptr()
    fn = _lib().dmuon_scalar_allreduce
    fn.argtypes = [ctypes.POINTER(_ScalarAllreduceArgs), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    _check(fn(ctypes.byref(a), _stream(local.device)), "dmuon_scalar_allreduce")


def copy_async(dst_ptr: int, src_ptr: int, nbytes: int, device: torch.device) -> None:
    """Queue one copy-engine transfer on the current stream of ``device``;
    either address may lie in a peer's symmetric buffer."""
    _check(_lib().dmuon_copy_async(dst_ptr, src_ptr, int(nbytes), _stream(device)), "dmuon_copy_async")


def wait_budget_cycles() -> int:
    """Cycle budget of one cross-GPU flag wait (``DMUON_PEER_WAIT_SECONDS``,
    default 20 s at ~1.9 GHz).  Ranks legitimately drift apart by seconds (the
    first step loads kernels and builds workspaces at different speeds, one
    rank may be slower through a data loader), so the default is several times
    the longest wait seen in training and still short for a kernel that only
    spins; jobs whose ranks stall longer (one rank writing a checkpoint to
    slow storage inside the step loop) raise it, tests set it to milliseconds
    to exercise the timeout path."""
    secs = float(os.environ.get("DMUON_PEER_WAIT_SECONDS", "20"))
    return int(secs * 1.9e9)


def signal_peers(peer_flag_ptrs: Sequence[int], slot: int, value: int, device) -> None:
    """``flags[slot] = value`` on every peer (release, system scope), ordered
    after everything queued before on the current stream."""
    a = _SignalArgs()
    for r, p in enumerate(peer_flag_ptrs):
        a.peer_flags[r] = p
    a.world, a.slot, a.value = len(peer_flag_ptrs), int(slot), int(value)
    _check(_lib().dmuon_signal_peers(ctypes.byref(a), _stream(device)), "dmuon_signal_peers")


def wait_flags(local_flags: torch.Tensor, first: int, count: int, want: int, status: torch.Tensor,
               budget_cycles: Optional[int] = None) -> None:
    """Queue a bounded device-side wait for ``local_flags[first:first+count] >= want``."""
    a = _WaitArgs()
    a.local_flags = local_flags.data_ptr()
    a.first, a.count, a.want = int(first), int(count), int(want)
    a.budget_cycles = int(budget_cycles if budget_cycles is not None else wait_budget_cycles())
    a.status = status.data_ptr()
    _check(_lib().dmuon_wait_flags(ctypes.byref(a), _stream(local_flags.device)), "dmuon_wait_flags")


def peer_prologue(
    peer_bases: Sequence[int],
    offsets: Sequence[int],
    numels: Sequence[int],
    grad_dtype: torch.dtype,
    moms: Sequence[Optional[torch.Tensor]],
    xs: Sequence[torch.Tensor],
    slots: Sequence[int],
    sumsq: Optional[torch.Tensor],
    *,
    scale: float,
    mu: float,
    nesterov: bool,
    gscale: Optional[torch.Tensor] = None,
    ready_flags: Optional[torch.Tensor] = None,
    ready_want: int = 0,
    status: Optional[torch.Tensor] = None,
    budget_cycles: Optional[int] = None,
    max_blocks_per_tensor: int = 0,
    xscale: Optional[torch.Tensor] = None,
) -> None:
    """Sum the gradient of every listed tensor over all ranks' arenas (peer
    loads, rank order), scale, then momentum / Nesterov / cast / sum of squares
    exactly like :func:`multi_tensor.muon_prologue`.  ``moms[i] is None`` turns
    the momentum off for that launch (all entries of one call must agree)."""
    n = len(offsets)
    if n == 0:
        return
    dev = xs[0].device
    has_mom = moms[0] is not None
    md = moms[0].dtype if has_mom else torch.float32
    xd = xs[0].dtype
    for lo, hi in _chunks(n):
        a = _PeerPrologueArgs()
        for r, p in enumerate(peer_bases):
            a.peer_base[r] = p
        a.world, a.scale = len(peer_bases), float(scale)
        for i in range(lo, hi):
            k = i - lo
            assert (moms[i] is not None) == has_mom and xs[i].dtype == xd and xs[i].is_contiguous()
            a.offset[k], a.numel[k], a.slot[k] = int(offsets[i]), int(numels[i]), int(slots[i])
            a.mom[k] = moms[i].data_ptr() if has_mom else None
            a.x[k] = xs[i].data_ptr()
        a.n = hi - lo
        a.grad_dtype, a.mom_dtype, a.x_dtype = _DT[grad_dtype], _DT[md], _DT[xd]
        a.mu, a.nesterov = float(mu), int(bool(nesterov))
        a.gscale = gscale.data_ptr() if gscale is not None else None
        a.sumsq = sumsq.data_ptr() if sumsq is not None else None
        a.ready_flags = ready_flags.data_ptr() if ready_flags is not None else None
        a.ready_want = int(ready_want)
        a.budget_cycles = int(budget_cycles if budget_cycles is not None else wait_budget_cycles())
        a.status = status.data_ptr() if status is not None else None
        a.max_blocks_per_tensor = int(max_blocks_per_tensor)
        a.xscale = xscale.data_ptr() if xscale is not None else None
        _check(_lib().dmuon_peer_prologue(ctypes.byref(a), _stream(dev)), "dmuon_peer_prologue")


def peer_pull(
    srcs: Sequence[int],
    dsts: Sequence[int],
    nbytes: Sequence[int],
    flag_slots: Sequence[int],
    local_flags: Optional[torch.Tensor],
    want: int,
    status: Optional[torch.Tensor],
    device,
    budget_cycles: Optional[int] = None,
    blocks_per_tensor: int = 0,
) -> None:
    """Copy ``nbytes[i]`` from ``srcs[i]`` (peer-mapped address on the owner) to
    ``dsts[i]`` (local) once ``local_flags[flag_slots[i]] >= want``."""
    n = len(srcs)
    for lo, hi in _chunks(n):
        a = _PullArgs()
        for i in range(lo, hi):
            k = i - lo
            a.src[k], a.dst[k], a.nbytes[k], a.flag_slot[k] = srcs[i], dsts[i], int(nbytes[i]), int(flag_slots[i])
        a.n = hi - lo
        a.local_flags = local_flags.data_ptr() if local_flags is not None else None
        a.want = int(want)
        a.budget_cycles = int(budget_cycles if budget_cycles is not None else wait_budget_cycles())
        a.status = status.data_ptr() if status is not None else None
        a.blocks_per_tensor = int(blocks_per_tensor)
        _check(_lib().dmuon_peer_pull(ctypes.byref(a), _stream(device)), "dmuon_peer_pull")


def multicast_reduce(mc_srcs: Sequence[int], dsts: Sequence[int], nbytes: Sequence[int], dtype: torch.dtype, device,
                     blocks_per_tensor: int = 0) -> None:
    """``dsts[i]`` (local addresses) = element-wise sum over all ranks of the
    spans at ``mc_srcs[i]`` (addresses in the NVSwitch multicast mapping of a
    symmetric buffer).  The sum is formed inside the switch
    (``multimem.ld_reduce``): this rank receives one copy instead of one per
    peer.  16-bit element types accumulate in fp32 and are rounded once; the
    summation order is the switch's, not rank order."""
    _multicast(mc_srcs, dsts, nbytes, 0, dtype, device, blocks_per_tensor)


def multicast_broadcast(srcs: Sequence[int], mc_dsts: Sequence[int], nbytes: Sequence[int], device,
                        blocks_per_tensor: int = 0) -> None:
    """Store the local spans ``srcs[i]`` to ``mc_dsts[i]`` (multicast
    addresses): every rank's buffer receives them (``multimem.st``)."""
    _multicast(srcs, mc_dsts, nbytes, 1, torch.float32, device, blocks_per_tensor)


def _multicast(srcs, dsts, nbytes, mode, dtype, device, blocks_per_tensor) -> None:
    n = len(srcs)
    for lo, hi in _chunks(n):
        a = _MulticastArgs()
        for i in range(lo, hi):
            k = i - lo
            a.src[k], a.dst[k], a.nbytes[k] = int(srcs[i]), int(dsts[i]), int(nbytes[i])
        a.n, a.mode, a.dtype, a.blocks_per_tensor = hi - lo, int(mode), _DT[dtype], int(blocks_per_tensor)
        _check(_lib().dmuon_multicast_copy(ctypes.byref(a), _stream(device)), "dmuon_multicast_copy")

"""ctypes front end of the multi-tensor elementwise kernels
(``csrc/multi_tensor.cu``): Muon prologue, AdamW, clip sum-of-squares / scale
and casts.  Each call covers any number of tensors; they are split into
launches of at most ``MAX_TENSORS`` whose pointers travel as kernel arguments.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import Optional, Sequence

import torch

from . import build as _build

MAX_TENSORS = 48
_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_VP = ctypes.c_void_p * MAX_TENSORS
_LL = ctypes.c_longlong * MAX_TENSORS
_IA = ctypes.c_int * MAX_TENSORS
_FA = ctypes.c_float * MAX_TENSORS


class _PrologueArgs(ctypes.Structure):
    _fields_ = [
        ("grad", _VP), ("mom", _VP), ("x", _VP), ("numel", _LL), ("slot", _IA),
        ("n", ctypes.c_int), ("grad_dtype", ctypes.c_int), ("mom_dtype", ctypes.c_int), ("x_dtype", ctypes.c_int),
        ("mu", ctypes.c_float), ("nesterov", ctypes.c_int),
        ("gscale", ctypes.c_void_p), ("sumsq", ctypes.c_void_p), ("xscale", ctypes.c_void_p),
    ]


class _NormArgs(ctypes.Structure):
    _fields_ = [
        ("sumsq", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("scale2", ctypes.c_void_p),
        ("n", ctypes.c_int), ("eps", ctypes.c_float),
    ]


class _AdamWArgs(ctypes.Structure):
    _fields_ = [
        ("param", _VP), ("grad", _VP), ("exp_avg", _VP), ("exp_avg_sq", _VP), ("publish", _VP),
        ("numel", _LL), ("step_size", _FA), ("inv_sqrt_bc2", _FA),
        ("n", ctypes.c_int), ("param_dtype", ctypes.c_int), ("grad_dtype", ctypes.c_int), ("state_dtype", ctypes.c_int),
        ("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
        ("weight_decay", ctypes.c_float), ("gscale", ctypes.c_void_p),
    ]


class _ClipArgs(ctypes.Structure):
    _fields_ = [
        ("tensor", _VP), ("numel", _LL), ("segment", _IA), ("dtype", _IA), ("n", ctypes.c_int),
        ("seg_sumsq", ctypes.c_void_p), ("seg_coef", ctypes.c_void_p),
    ]


class _CastArgs(ctypes.Structure):
    _fields_ = [
        ("src", _VP), ("dst", _VP), ("numel", _LL), ("slot", _IA), ("n", ctypes.c_int),
        ("src_dtype", ctypes.c_int), ("dst_dtype", ctypes.c_int), ("scale", ctypes.c_void_p),
    ]


@lru_cache(maxsize=None)
def _lib():
    lib = _build.load()
    for name, typ in (
        ("dmuon_muon_prologue", _PrologueArgs),
        ("dmuon_norm_scales", _NormArgs),
        ("dmuon_adamw", _AdamWArgs),
        ("dmuon_clip_sumsq", _ClipArgs),
        ("dmuon_clip_scale", _ClipArgs),
        ("dmuon_cast", _CastArgs),
    ):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(typ), ctypes.c_void_p]
        fn.restype = ctypes.c_int
    lib.dmuon_launch_count.restype = ctypes.c_longlong
    return lib


def launch_count() -> int:
    """Kernel launches issued through the library since it was loaded."""
    return int(_lib().dmuon_launch_count()) if _build.is_loaded() or _build.is_current() else 0


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def _chunks(n: int):
    for lo in range(0, n, MAX_TENSORS):
        yield lo, min(n, lo + MAX_TENSORS)


def _flat_ok(t: torch.Tensor) -> bool:
    return t.is_contiguous()


def muon_prologue(
    grads: Sequence[torch.Tensor],
    moms: Sequence[torch.Tensor],
    xs: Sequence[torch.Tensor],
    slots: Sequence[int],
    sumsq: torch.Tensor,
    mu: float,
    nesterov: bool,
    gscale: Optional[torch.Tensor] = None,
    xscale: Optional[torch.Tensor] = None,
) -> None:
    """``mom = mu*mom + g``; ``u = g + mu*mom`` (or ``mom``); ``x = cast(u)``;
    accumulate ``sum(u^2)`` into ``sumsq[slot]`` (``sumsq`` must be zeroed by the
    caller).  With ``xscale`` (fp32, one entry per slot) the stored operand is
    ``cast(u * xscale[slot])`` while the sum of squares stays that of ``u``."""
    n = len(grads)
    assert n == len(moms) == len(xs) == len(slots)
    if n == 0:
        return
    dev = grads[0].device
    gd, md, xd = grads[0].dtype, moms[0].dtype, xs[0].dtype
    for lo, hi in _chunks(n):
        a = _PrologueArgs()
        for i in range(lo, hi):
            g, m, x = grads[i], moms[i], xs[i]
            assert g.dtype == gd and m.dtype == md and x.dtype == xd
            assert _flat_ok(g) and _flat_ok(m) and _flat_ok(x) and g.numel() == m.numel() == x.numel()
            k = i - lo
            a.grad[k], a.mom[k], a.x[k] = g.data_ptr(), m.data_ptr(), x.data_ptr()
            a.numel[k] = g.numel()
            a.slot[k] = int(slots[i])
        a.n = hi - lo
        a.grad_dtype, a.mom_dtype, a.x_dtype = _DT[gd], _DT[md], _DT[xd]
        a.mu, a.nesterov = float(mu), int(bool(nesterov))
        a.gscale = gscale.data_ptr() if gscale is not None else None
        a.sumsq = sumsq.data_ptr()
        a.xscale = xscale.data_ptr() if xscale is not None else None
        _check(_lib().dmuon_muon_prologue(ctypes.byref(a), _stream(dev)), "dmuon_muon_prologue")


def norm_scales(sumsq: torch.Tensor, scale: torch.Tensor, scale2: torch.Tensor, eps: float = 1e-7) -> None:
    a = _NormArgs()
    a.sumsq, a.scale, a.scale2 = sumsq.data_ptr(), scale.data_ptr(), scale2.data_ptr()
    a.n, a.eps = sumsq.numel(), float(eps)
    _check(_lib().dmuon_norm_scales(ctypes.byref(a), _stream(sumsq.device)), "dmuon_norm_scales")


def adamw(
    params: Sequence[torch.Tensor],
    grads: Sequence[torch.Tensor],
    exp_avgs: Sequence[torch.Tensor],
    exp_avg_sqs: Sequence[torch.Tensor],
    steps: Sequence[int],
    *,
    lr: float,
    beta1: float,
    beta2: float,
    eps: float,
    weight_decay: float,
    publish: Optional[Sequence[Optional[torch.Tensor]]] = None,
    gscale: Optional[torch.Tensor] = None,
) -> None:
    """One fused AdamW update per tensor; ``steps[i]`` is the (already
    incremented) step count of tensor ``i`` used for bias correction."""
    n = len(params)
    if n == 0:
        return
    dev = params[0].device
    pd, gd, sd = params[0].dtype, grads[0].dtype, exp_avgs[0].dtype
    for lo, hi in _chunks(n):
        a = _AdamWArgs()
        for i in range(lo, hi):
            p, g, m, v = params[i], grads[i], exp_avgs[i], exp_avg_sqs[i]
            assert p.dtype == pd and g.dtype == gd and m.dtype == sd and v.dtype == sd
            assert _flat_ok(p) and _flat_ok(g) and _flat_ok(m) and _flat_ok(v)
            k = i - lo
            a.param[k], a.grad[k], a.exp_avg[k], a.exp_avg_sq[k] = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
            pub = publish[i] if publish is not None else None
            a.publish[k] = pub.data_ptr() if pub is not None else None
            a.numel[k] = p.numel()
            t = int(steps[i])
            a.step_size[k] = lr / (1.0 - beta1**t)
            a.inv_sqrt_bc2[k] = 1.0 / (1.0 - beta2**t) ** 0.5
        a.n = hi - lo
        a.param_dtype, a.grad_dtype, a.state_dtype = _DT[pd], _DT[gd], _DT[sd]
        a.lr, a.beta1, a.beta2, a.eps, a.weight_decay = float(lr), float(beta1), float(beta2), float(eps), float(weight_decay)
        a.gscale = gscale.data_ptr() if gscale is not None else None
        _check(_lib().dmuon_adamw(ctypes.byref(a), _stream(dev)), "dmuon_adamw")


def _clip_call(fn_name: str, tensors, segments, seg_sumsq, seg_coef) -> None:
    n = len(tensors)
    if n == 0:
        return
    dev = tensors[0].device
    for lo, hi in _chunks(n):
        a = _ClipArgs()
        for i in range(lo, hi):
            t = tensors[i]
            assert _flat_ok(t)
            k = i - lo
            a.tensor[k], a.numel[k], a.segment[k], a.dtype[k] = t.data_ptr(), t.numel(), int(segments[i]), _DT[t.dtype]
        a.n = hi - lo
        a.seg_sumsq = seg_sumsq.data_ptr() if seg_sumsq is not None else None
        a.seg_coef = seg_coef.data_ptr() if seg_coef is not None else None
        _check(getattr(_lib(), fn_name)(ctypes.byref(a), _stream(dev)), fn_name)


def clip_sumsq(tensors: Sequence[torch.Tensor], segments: Sequence[int], seg_sumsq: torch.Tensor) -> None:
    """``seg_sumsq[segments[i]] += sum(tensors[i]^2)`` in fp32."""
    _clip_call("dmuon_clip_sumsq", tensors, segments, seg_sumsq, None)


def clip_scale(tensors: Sequence[torch.Tensor], segments: Sequence[int], seg_coef: torch.Tensor) -> None:
    """``tensors[i] *= seg_coef[segments[i]]`` in place."""
    _clip_call("dmuon_clip_scale", tensors, segments, None, seg_coef)


def cast(
    srcs: Sequence[torch.Tensor],
    dsts: Sequence[torch.Tensor],
    scale: Optional[torch.Tensor] = None,
    slots: Optional[Sequence[int]] = None,
) -> None:
    """``dst = cast(src * scale[slot])`` for many tensors in few launches."""
    n = len(srcs)
    if n == 0:
        return
    dev = srcs[0].device
    sd, dd = srcs[0].dtype, dsts[0].dtype
    for lo, hi in _chunks(n):
        a = _CastArgs()
        for i in range(lo, hi):
            s, d = srcs[i], dsts[i]
            assert s.dtype == sd and d.dtype == dd and _flat_ok(s) and _flat_ok(d) and s.numel() == d.numel()
            k = i - lo
            a.src[k], a.dst[k], a.numel[k] = s.data_ptr(), d.data_ptr(), s.numel()
            a.slot[k] = int(slots[i]) if slots is not None else 0
        a.n = hi - lo
        a.src_dtype, a.dst_dtype = _DT[sd], _DT[dd]
        a.scale = scale.data_ptr() if scale is not None else None
        _check(_lib().dmuon_cast(ctypes.byref(a), _stream(dev)), "dmuon_cast")

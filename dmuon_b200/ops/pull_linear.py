"""Forward publish fused into its first consumer (``csrc/pull_linear_sm100.cu``).

``pull_linear(x, w_local, w_remote_ptr, ...)`` computes ``y = x @ w^T`` while
the same kernel pulls ``w`` from its owner's GPU into ``w_local`` tile by tile.
``PulledLinearFn`` is the autograd wrapper: backward uses ``w_local`` (which the
forward kernel filled), so the weight crosses NVLink once per step.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import Optional

import torch

from . import build as _build
from .gemm import status_buffer
from .multi_tensor import _check, _stream

BN = 256


class _Args(ctypes.Structure):
    _fields_ = [
        ("X", ctypes.c_void_p), ("Y", ctypes.c_void_p), ("W_local", ctypes.c_void_p), ("W_remote", ctypes.c_void_p),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("ldx", ctypes.c_longlong), ("ldy", ctypes.c_longlong),
        ("tile_ready", ctypes.c_void_p), ("pub_flag", ctypes.c_void_p), ("pub_want", ctypes.c_int),
        ("budget_cycles", ctypes.c_longlong), ("status", ctypes.c_void_p), ("max_ctas", ctypes.c_int),
    ]


@lru_cache(maxsize=None)
def _fn():
    fn = _build.load().dmuon_pull_linear_sm100
    fn.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


_ready_bufs: dict[tuple, torch.Tensor] = {}


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """bf16, contiguous weight with K a multiple of 32, 16-byte aligned rows."""
    return (
        x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
        and w.shape[1] % 32 == 0 and x.shape[-1] == w.shape[1] and x.stride(-1) == 1
    )


def pull_linear(
    x: torch.Tensor,
    w_local: torch.Tensor,
    w_remote_ptr: Optional[int] = None,
    *,
    pub_flag: Optional[torch.Tensor] = None,
    pub_want: int = 0,
    budget_cycles: int = 0,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``out = x @ w^T``; when ``w_remote_ptr`` is given the kernel first-touches
    ``w`` through that peer address and leaves a copy in ``w_local``."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w_local.shape[0]
    dev = x.device
    if out is None:
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    a = _Args()
    a.X, a.Y, a.W_local = x2.data_ptr(), out.data_ptr(), w_local.data_ptr()
    a.W_remote = int(w_remote_ptr) if w_remote_ptr else None
    a.M, a.N, a.K = M, N, K
    a.ldx, a.ldy = x2.stride(0), out.stride(0)
    if w_remote_ptr:
        nt = (N + BN - 1) // BN
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        buf = _ready_bufs.get(key)
        if buf is None or buf.numel() < nt:
            buf = torch.zeros(max(nt, 1024), dtype=torch.int32, device=dev)
            _ready_bufs[key] = buf
        buf[:nt].zero_()                # scratch counters, reused by launches on this stream
        a.tile_ready = buf.data_ptr()
    a.pub_flag = pub_flag.data_ptr() if pub_flag is not None else None
    a.pub_want = int(pub_want)
    a.budget_cycles = int(budget_cycles)
    a.status = status_buffer(dev).data_ptr()
    _check(_fn()(ctypes.byref(a), _stream(dev)), "dmuon_pull_linear_sm100")
    return out.view(*x.shape[:-1], N)


class PulledLinearFn(torch.autograd.Function):
    """``y = x w^T (+ bias)`` whose forward also fetches ``w`` from its owner."""

    @staticmethod
    def forward(ctx, x, w_param, bias, w_remote_ptr, pub_flag, pub_want, budget):
        w_local = w_param.detach()
        with torch.autograd._unsafe_preserve_version_counter((w_param,)):
            y = pull_linear(x, w_local, w_remote_ptr, pub_flag=pub_flag, pub_want=pub_want, budget_cycles=budget)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x, w_param)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        gx = gw = gb = None
        g2 = gy.reshape(-1, gy.shape[-1])
        if ctx.needs_input_grad[0]:
            gx = (g2 @ w).view_as(x)
        if ctx.needs_input_grad[1]:
            gw = g2.t() @ x.reshape(-1, x.shape[-1])
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g2.sum(0)
        return gx, gw, gb, None, None, None, None

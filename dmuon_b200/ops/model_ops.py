"""Fused activation-side ops of the decoder models (``csrc/model_ops.cu``):
SwiGLU, rotary embedding applied in place to the projection outputs, and a
chunked linear + softmax cross-entropy that computes its gradients while the
logits of a chunk are still in L2.

Each op is a ``torch.autograd.Function`` over the CUDA kernel with a plain
PyTorch formulation for CPU tensors (that formulation is also the oracle of
the GPU numerics tests).  The reference ships no model code; these ops serve
the models under ``dmuon_b200.models``.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache
from typing import Optional

import torch
import torch.nn.functional as F

from . import build as _build

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_P, _LL, _I, _F = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float


@lru_cache(maxsize=None)
def _lib():
    lib = _build.load()
    lib.dmuon_swiglu_fwd.argtypes = [_P, _P, _P, _LL, _I, _I, _P]
    lib.dmuon_swiglu_bwd.argtypes = [_P, _P, _P, _P, _P, _LL, _I, _I, _P]
    lib.dmuon_rope_inplace.argtypes = [_P, _P, _P, _P, _LL, _I, _I, _I, _I, _LL, _LL, _I, _I, _P]
    lib.dmuon_softmax_xent_inplace.argtypes = [_P, _P, _P, _LL, _I, _LL, _F, _I, _P]
    for name in ("dmuon_swiglu_fwd", "dmuon_swiglu_bwd", "dmuon_rope_inplace", "dmuon_softmax_xent_inplace"):
        getattr(lib, name).restype = ctypes.c_int
    return lib


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def kernels_apply(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a GPU and has a dtype the kernels take."""
    return t.is_cuda and t.dtype in _DT


# ---------------------------------------------------------------------------- gated MLP activations
ACT_SILU, ACT_GELU_TANH = 0, 1


def swiglu_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


def geglu_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.gelu(gate, approximate="tanh") * up


class _GatedAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: torch.Tensor, up: torch.Tensor, act: int) -> torch.Tensor:
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty_like(gate)
        _check(
            _lib().dmuon_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), act, _DT[gate.dtype], _stream(gate)),
            "dmuon_swiglu_fwd",
        )
        ctx.save_for_backward(gate, up)
        ctx.act = act
        return out

    @staticmethod
    def backward(ctx, d_out: torch.Tensor):
        gate, up = ctx.saved_tensors
        d_out = d_out.contiguous()
        d_gate, d_up = torch.empty_like(gate), torch.empty_like(up)
        _check(
            _lib().dmuon_swiglu_bwd(
                gate.data_ptr(), up.data_ptr(), d_out.data_ptr(), d_gate.data_ptr(), d_up.data_ptr(),
                gate.numel(), ctx.act, _DT[gate.dtype], _stream(gate),
            ),
            "dmuon_swiglu_bwd",
        )
        return d_gate, d_up, None


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` in one pass (three in the backward: gate, up and
    the incoming gradient are read once, both gradients written once)."""
    if kernels_apply(gate) and gate.dtype == up.dtype and gate.shape == up.shape:
        return _GatedAct.apply(gate, up, ACT_SILU)
    return swiglu_reference(gate, up)


def geglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(gate) * up``, same kernels as :func:`swiglu`."""
    if kernels_apply(gate) and gate.dtype == up.dtype and gate.shape == up.shape:
        return _GatedAct.apply(gate, up, ACT_GELU_TANH)
    return geglu_reference(gate, up)


# ---------------------------------------------------------------------------- rotary embedding
def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x``: [batch, seq, heads, head_dim]; tables [seq, head_dim / 2];
    rotate-half pairing.  Arithmetic in fp32, result in ``x.dtype``."""
    d = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d], xf[..., d:]
    c, s = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


def _rope_launch(q: torch.Tensor, k: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor, d: int, inverse: bool) -> None:
    b, s, qw = q.shape
    kw = k.shape[2] if k is not None else 0
    _check(
        _lib().dmuon_rope_inplace(
            q.data_ptr(), k.data_ptr() if k is not None else None, cos.data_ptr(), sin.data_ptr(),
            b * s, s, qw // d, kw // d, d, q.stride(1), k.stride(1) if k is not None else 0, int(inverse),
            _DT[q.dtype], _stream(q),
        ),
        "dmuon_rope_inplace",
    )


def _rope_layout_ok(t: torch.Tensor, d: int) -> bool:
    # [b, s, heads * d]: dense rows, rows of one batch entry back to back, 16-byte aligned rows
    b, s, w = t.shape
    return (
        t.stride(2) == 1 and w % d == 0 and (b == 1 or t.stride(0) == s * t.stride(1))
        and (t.stride(1) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0
    )


class _RopeQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, d):
        _rope_launch(q, k, cos, sin, d, inverse=False)
        ctx.mark_dirty(q, k)
        ctx.save_for_backward(cos, sin)
        ctx.head_dim = d
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        d = ctx.head_dim
        # q and k each feed exactly one consumer (the attention), so the buffers
        # that carry their gradients belong to this node: rotate them in place
        # when they already have the row layout, otherwise rotate a dense copy
        if not _rope_layout_ok(dq, d):
            dq = dq.contiguous()
        if not _rope_layout_ok(dk, d):
            dk = dk.contiguous()
        _rope_launch(dq, dk, cos, sin, d, inverse=True)
        return dq, dk, None, None, None


def rope_qk_(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, head_dim: int):
    """Rotate the heads of ``q`` [b, s, hq * head_dim] and ``k`` [b, s, hk *
    head_dim] by the position tables ``cos`` / ``sin`` [s, head_dim / 2]
    (fp32), rotate-half pairing.  On a GPU both are rotated in place by one
    launch -- pass the projection outputs themselves (nothing else may need
    them unrotated); elsewhere new tensors are returned."""
    d = int(head_dim)
    if (
        kernels_apply(q) and k.dtype == q.dtype and d % 16 == 0 and q.dim() == 3 and k.dim() == 3
        and _rope_layout_ok(q, d) and _rope_layout_ok(k, d)
        and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        and not (q._is_view() or k._is_view())
    ):
        return _RopeQK.apply(q, k, cos, sin, d)
    b, s, _ = q.shape
    qr = rope_reference(q.reshape(b, s, -1, d), cos, sin).reshape(q.shape)
    kr = rope_reference(k.reshape(b, s, -1, d), cos, sin).reshape(k.shape)
    return qr, kr


# ---------------------------------------------------------------------------- linear + cross-entropy
def linear_cross_entropy_reference(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    return F.cross_entropy(F.linear(h, weight).float(), labels, ignore_index=ignore_index)


def softmax_xent_(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float) -> torch.Tensor:
    """Per-row loss of ``logits`` [rows, vocab]; ``logits`` is overwritten by
    ``(softmax - onehot) * grad_scale`` (zero rows where the label is negative)."""
    rows, vocab = logits.shape
    assert logits.stride(1) == 1 and labels.dtype == torch.int64 and labels.is_contiguous() and labels.numel() == rows
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _check(
        _lib().dmuon_softmax_xent_inplace(
            logits.data_ptr(), labels.data_ptr(), row_loss.data_ptr(), rows, vocab, logits.stride(0),
            float(grad_scale), _DT[logits.dtype], _stream(logits),
        ),
        "dmuon_softmax_xent_inplace",
    )
    return row_loss


class _LinearXent(torch.autograd.Function):
    """Forward computes the loss chunk by chunk and, while a chunk's logits
    are hot, their gradient and its two products (``d_h`` and the chunk's
    contribution to ``d_weight``); backward only scales by the incoming
    gradient.  The logits of one chunk are the only vocabulary-sized
    activation that ever exists, and the vocabulary GEMM is not recomputed."""

    @staticmethod
    def forward(ctx, h, weight, labels, chunk, ignore_index):
        rows = h.shape[0]
        lab = labels
        if ignore_index >= 0:
            lab = labels.masked_fill(labels == ignore_index, -1)
        valid = (lab >= 0).sum().clamp_(min=1).to(torch.float32)
        need_h, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        d_h = torch.empty_like(h) if need_h else None
        d_w = torch.zeros_like(weight) if need_w else None
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        for lo in range(0, rows, chunk):
            hc = h[lo : lo + chunk]
            logits = hc @ weight.t()
            # gradient of the summed loss; the 1 / valid factor is applied to the small results
            row_loss = softmax_xent_(logits, lab[lo : lo + chunk].contiguous(), 1.0)
            total += row_loss.sum()
            if need_h:
                torch.mm(logits, weight, out=d_h[lo : lo + chunk])
            if need_w:
                d_w.addmm_(logits.t(), hc)
        inv = 1.0 / valid
        if need_h:
            d_h.mul_(inv.to(d_h.dtype))
        if need_w:
            d_w.mul_(inv.to(d_w.dtype))
        ctx.save_for_backward(d_h, d_w)
        return total * inv

    @staticmethod
    def backward(ctx, g):
        d_h, d_w = ctx.saved_tensors
        if d_h is not None:
            d_h = d_h * g.to(d_h.dtype)
        if d_w is not None:
            d_w = d_w * g.to(d_w.dtype)
        return d_h, d_w, None, None, None


def linear_cross_entropy(
    h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, chunk: int = 2048, ignore_index: int = -100
) -> torch.Tensor:
    """Mean cross-entropy of ``softmax(h @ weight.T)`` against ``labels``
    (``h`` [rows, d], ``weight`` [vocab, d]); positions whose label equals
    ``ignore_index`` (or is negative) do not count."""
    if kernels_apply(h) and weight.dtype == h.dtype and h.dim() == 2:
        return _LinearXent.apply(h.contiguous(), weight, labels.contiguous(), int(chunk) if chunk > 0 else h.shape[0], int(ignore_index))
    return linear_cross_entropy_reference(h, weight, labels, ignore_index)

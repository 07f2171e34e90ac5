"""Batched Newton-Schulz and the fused Muon update on the sm_100a kernels.

All matrices of one shape that a rank owns are stacked and pushed through the
iteration together: every product below is ONE launch of the tcgen05 GEMM over
the whole batch, so small Gram dimensions (1024, 256) still fill 148 SMs.

Data flow for a batch of ``L`` matrices ``m0 x n0`` (natural orientation, no
transposed copy is ever made):

    prologue      mom = mu*mom + g ; u = g + mu*mom ; sumsq += u^2
                  (with the peer data plane the same kernel first sums g over
                  all ranks' gradient arenas: reduce-to-owner costs no extra pass)
    scales        s = 1/(||u||_F + eps), s^2
    operand       Gram form (default): X = fp16(K s u), K a power of two near
                  sqrt(min(m0, n0)) that keeps entries clear of fp16 subnormals;
                  the products carry 1/K^2 and 1/K in their alpha.
                  bf16 operands (compute_dtype=bf16): X = bf16(u) written by the
                  prologue itself, s and s^2 applied per matrix in the epilogues.
    gram          R = X X^T   (m0 <= n0)   or   X^T X   (m0 > n0)
    per step      P = c R R + b R + a I ;  Q = P Q ;  R = (R P) P      symmetric
    restart       X = Q X  (or X Q) ;  R = X X^T
    final         W = (1 - lr wd) W - lr * scale * Q X   written straight into
                  the fp32 master weights (and a bf16 publish copy)

Symmetric products compute only the tiles that touch the lower triangle (the
CTA-pair kernel, 256 x 256 tiles, whenever the shape fills it).
Replaces the reference's per-matrix Python loop around SYRK / cuBLAS calls and
its CUDA-graph cache (dmuon/optim/muon.py:1582-1747,
dmuon/optim/newton_schulz.py:333-448, dmuon/optim/ns_graph.py:61-128).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import build as _build
from . import gemm as G
from . import multi_tensor as MT

_avail: Optional[bool] = None


def available() -> bool:
    """True on a CUDA device of compute capability 10.x with the kernel
    library present (built on demand when nvcc exists)."""
    global _avail
    if _avail is None:
        ok = torch.cuda.is_available()
        if ok:
            major, _ = torch.cuda.get_device_capability()
            ok = major == 10
        if ok:
            _build.load()   # raises when the library is missing: no silent fallback on a B200
        _avail = ok
    return _avail


class _Workspace:
    def __init__(self, L: int, m0: int, n0: int, dtype: torch.dtype, device):
        self.key = (L, m0, n0, dtype)
        m = min(m0, n0)
        e = dict(device=device, dtype=dtype)
        self.X = torch.empty(L, m0, n0, **e)
        self.X2 = torch.empty(L, m0, n0, **e)
        self.R = torch.empty(L, m, m, **e)
        self.R2 = torch.empty(L, m, m, **e)
        self.RP = torch.empty(L, m, m, **e)
        self.P = torch.empty(L, m, m, **e)
        self.Qa = torch.empty(L, m, m, **e)
        self.Qb = torch.empty(L, m, m, **e)
        self.sumsq = torch.zeros(L, device=device, dtype=torch.float32)
        self.scale = torch.empty(L, device=device, dtype=torch.float32)
        self.scale2 = torch.empty(L, device=device, dtype=torch.float32)
        self.Xf32: Optional[torch.Tensor] = None
        # single-pass fp16 operand: the per-matrix correction factors of the current call
        self.fix = torch.empty(L, device=device, dtype=torch.float32)
        self.fix2 = torch.empty(L, device=device, dtype=torch.float32)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in vars(self).values() if isinstance(t, torch.Tensor))


#: fp16 Gram operands written by the prologue itself from the second step on (no fp32 staging pass);
#: ``DMUON_NS_SINGLE_PASS=0`` keeps the two-pass form (norm first, then cast)
SINGLE_PASS_FP16 = __import__("os").environ.get("DMUON_NS_SINGLE_PASS", "1").strip().lower() not in ("0", "false", "no", "off")

#: per batch of matrices (keyed by their momentum buffers): K / ||u|| of their previous step
_prescales: dict[tuple, torch.Tensor] = {}
_workspaces: dict[tuple, _Workspace] = {}
_ptr_tables: dict[tuple, torch.Tensor] = {}
MAX_WORKSPACE_BYTES = 6 << 30


def workspace(L: int, m0: int, n0: int, dtype: torch.dtype, device) -> _Workspace:
    key = (L, m0, n0, dtype, device.index)
    ws = _workspaces.get(key)
    if ws is None:
        # keep at most one workspace per (shape, dtype): drop other batch sizes of this shape
        for k in [k for k in _workspaces if k[1:] == key[1:]]:
            del _workspaces[k]
        ws = _Workspace(L, m0, n0, dtype, device)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    _workspaces.clear()
    _ptr_tables.clear()
    _prescales.clear()


def max_batch(m0: int, n0: int, itemsize: int = 2) -> int:
    """Largest batch whose workspace stays under ``MAX_WORKSPACE_BYTES``."""
    m = min(m0, n0)
    per = (2 * m0 * n0 + 6 * m * m) * itemsize
    return max(1, MAX_WORKSPACE_BYTES // per)


def _ptr_table(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    key = tuple(t.data_ptr() for t in tensors)
    tab = _ptr_tables.get(key)
    if tab is None:
        if len(_ptr_tables) > 4096:
            _ptr_tables.clear()
        tab = torch.tensor(key, dtype=torch.int64).to(tensors[0].device, non_blocking=True)
        _ptr_tables[key] = tab
    return tab


def _addr_table(addrs: Sequence[int], device) -> torch.Tensor:
    key = tuple(int(a) for a in addrs)
    tab = _ptr_tables.get(key)
    if tab is None:
        if len(_ptr_tables) > 4096:
            _ptr_tables.clear()
        tab = torch.tensor(key, dtype=torch.int64).to(device, non_blocking=True)
        _ptr_tables[key] = tab
    return tab


def _gram(ws: _Workspace, X: torch.Tensor, out: torch.Tensor, left: bool, alpha_vec=None) -> None:
    if left:
        G.gemm(X, X, out, symmetric=True, alpha_vec=alpha_vec)
    else:
        G.gemm(X, X, out, a_mn=True, b_mn=True, symmetric=True, alpha_vec=alpha_vec)


def _apply(Q: torch.Tensor, X: torch.Tensor, left: bool, **kw) -> None:
    """``out = Q X`` (left) or ``X Q`` (right) with the epilogue given in kw."""
    if left:
        G.gemm(Q, X, kw.pop("out", None), b_mn=True, **kw)
    else:
        G.gemm(X, Q, kw.pop("out", None), **kw)


class _XScale:
    """How the stored operand relates to the normalised matrix:
    ``X_true = X_stored * vec[b] * h`` with an optional per-matrix device vector
    (``vec``; ``vec2`` holds its squares) and a host factor ``h``.

    bf16 operands are stored unnormalised (``vec = 1/||u||``, written by the
    norm kernel, ``h = 1``) because bf16 has the range for raw gradients.  fp16
    operands are stored normalised and multiplied by a power of two ``K`` near
    ``sqrt(min(m, n))`` (``h = 1/K``) so their entries sit around
    ``1/sqrt(max(m, n))`` instead of ``1/sqrt(m n)``, which would graze the fp16
    subnormal range."""

    def __init__(self, vec=None, vec2=None, h: float = 1.0):
        self.vec, self.vec2, self.h = vec, vec2, float(h)


def fp16_prescale(m0: int, n0: int) -> float:
    import math

    return float(2 ** round(math.log2(math.sqrt(min(m0, n0)))))


def _iterate(ws: _Workspace, coefs, restarts, formulation: str, left: bool, xs: _XScale, segments=None):
    """Run all products but the final application.  Returns ``(Q, X)``: the
    result is ``Q X_true`` (gram) or ``X`` itself (direct, which needs
    ``X_stored == X_true``).  With a list in ``segments`` (gram only) a copy of
    the accumulated factor of every restart window is appended to it."""
    X = ws.X
    if formulation == "direct":
        # X <- a X + (b A + c A A) X, A = X X^T
        Xn = ws.X2
        for a, b, c in coefs:
            _gram(ws, X, ws.R, left)
            G.gemm(ws.R, ws.R, ws.P, C=ws.R, alpha=c, beta=b, symmetric=True)
            _apply(ws.P, X, left, out=Xn, C=X, beta=a)
            X, Xn = Xn, X
        return None, X

    def gram_of(Xs, out):
        if left:
            G.gemm(Xs, Xs, out, symmetric=True, alpha=xs.h * xs.h, alpha_vec=xs.vec2)
        else:
            G.gemm(Xs, Xs, out, a_mn=True, b_mn=True, symmetric=True, alpha=xs.h * xs.h, alpha_vec=xs.vec2)

    gram_of(X, ws.R)
    R, Rn = ws.R, ws.R2
    pool = (ws.Qa, ws.Qb, ws.P)

    def free(*busy):
        return next(t for t in pool if all(t is not b for b in busy))

    Q = None
    last = len(coefs) - 1
    for i, (a, b, c) in enumerate(coefs):
        if i in restarts and i != 0:
            # the new operand keeps the scale of the old one: Q X_stored
            Xn = ws.X2 if X is ws.X else ws.X
            _apply(Q, X, left, out=Xn)
            X = Xn
            gram_of(X, R)
            if segments is not None:
                segments.append(Q.clone())
            Q = None
        # step polynomial P = c R R + b R + a I
        P = free(Q)
        G.gemm(R, R, P, C=R, alpha=c, beta=b, diag=a, symmetric=True)
        if Q is None:
            Q = P                       # first step of a window: the factor IS the polynomial
        else:
            T = free(Q, P)
            G.gemm(P, Q, T, symmetric=True)
            Q = T
        if i < last and (i + 1) not in restarts:
            G.gemm(R, P, ws.RP, symmetric=True)
            G.gemm(ws.RP, P, Rn, symmetric=True)
            R, Rn = Rn, R
    if segments is not None:
        segments.append(Q.clone())
    return Q, X


def _run(ws: _Workspace, coefs, restarts, formulation: str, left: bool, xs: _XScale, final_kw: dict) -> None:
    Q, X = _iterate(ws, coefs, restarts, formulation, left, xs)
    if formulation == "direct":
        final_kw["copy_from"] = X       # the iterate itself is the result
        return
    final_kw["alpha"] = float(final_kw.get("alpha", 1.0)) * xs.h
    if xs.vec is not None:
        final_kw["alpha_vec"] = xs.vec
    _apply(Q, X, left, **final_kw)


def _resolve_dtype(compute_dtype, formulation: str) -> torch.dtype:
    if compute_dtype in (torch.bfloat16, torch.float16):
        return compute_dtype
    return torch.float16 if formulation == "gram" else torch.bfloat16


def newton_schulz_batched(
    X_in: torch.Tensor,
    coefs,
    restarts,
    eps: float = 1e-7,
    formulation: str = "gram",
    compute_dtype: Optional[torch.dtype] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Orthogonalise every matrix of ``X_in`` ``[L, m0, n0]``; returns a tensor
    of the input dtype.  ``compute_dtype`` is the operand dtype of the products
    (default: fp16 for the Gram form, bf16 for the direct form)."""
    assert X_in.dim() == 3 and X_in.is_cuda
    L, m0, n0 = X_in.shape
    cd = _resolve_dtype(compute_dtype, formulation)
    ws = workspace(L, m0, n0, cd, X_in.device)
    left = m0 <= n0
    K = fp16_prescale(m0, n0) if (cd == torch.float16 and formulation == "gram") else 1.0
    if X_in.is_contiguous() and X_in.dtype in MT._DT:
        # one read for the norms, one read + one write for the normalised operand
        mats = [X_in[i] for i in range(L)]
        slots = list(range(L))
        ws.sumsq.zero_()
        MT.clip_sumsq(mats, slots, ws.sumsq)
        MT.norm_scales(ws.sumsq, ws.scale, ws.scale2, eps)
        if K != 1.0:
            ws.scale.mul_(K)
        MT.cast(mats, [ws.X[i] for i in range(L)], scale=ws.scale, slots=slots)
    else:
        Xf = X_in.float()
        sumsq = (Xf * Xf).sum(dim=(1, 2))
        ws.scale.copy_(K / (sumsq.sqrt() + eps))
        ws.X.copy_(Xf * ws.scale.view(-1, 1, 1))
    xs = _XScale(h=1.0 / K)
    if out is None:
        out = torch.empty(L, m0, n0, device=X_in.device, dtype=X_in.dtype)
    kw: dict = {}
    if formulation == "direct":
        _run(ws, coefs, restarts, formulation, left, xs, kw)
        out.copy_(kw["copy_from"])
        return out
    if out.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise TypeError(f"unsupported output dtype {out.dtype}")
    kw["out"] = out
    _run(ws, coefs, restarts, formulation, left, xs, kw)
    return out


def gram_factors(U: torch.Tensor, coefs, restarts, eps: float = 1e-7):
    """Left-factor segments of the Gram iteration for ONE matrix, on the kernels.

    Returns ``(segments, transposed, normalizer)`` with the meaning of
    :func:`dmuon_b200.optim.newton_schulz.gram_newton_schulz_factors`: with
    ``X`` the matrix oriented wide (transposed when it has more rows than
    columns) and divided by ``normalizer``, ``segments[-1] @ ... @ segments[0] @ X``
    is the orthogonalised matrix.  Every segment is a symmetric fp16 matrix of
    the small dimension.  Because the segments multiply from the left they can
    be applied to any subset of ``X``'s columns: a tensor-parallel owner sends
    them instead of the full update (reference dmuon/optim/muon.py:1097-1278,
    there on library GEMMs)."""
    assert U.dim() == 2 and U.is_cuda
    m0, n0 = int(U.shape[0]), int(U.shape[1])
    ws = workspace(1, m0, n0, torch.float16, U.device)
    left = m0 <= n0
    K = fp16_prescale(m0, n0)
    Uc = U if (U.is_contiguous() and U.dtype in MT._DT) else U.float().contiguous()
    ws.sumsq.zero_()
    MT.clip_sumsq([Uc], [0], ws.sumsq)
    MT.norm_scales(ws.sumsq, ws.scale, ws.scale2, eps)
    normalizer = 1.0 / ws.scale[0].clone()          # ||U||_F + eps
    ws.scale.mul_(K)
    MT.cast([Uc], [ws.X[0]], scale=ws.scale, slots=[0])
    segs: list[torch.Tensor] = []
    _iterate(ws, coefs, restarts, "gram", left, _XScale(h=1.0 / K), segments=segs)
    return [s[0] for s in segs], not left, normalizer


def apply_factors(U_local: torch.Tensor, segments, transposed: bool, normalizer: torch.Tensor) -> torch.Tensor:
    """Apply factor segments from :func:`gram_factors` to this rank's part of
    the matrix with the tcgen05 GEMM: ``U_local`` is a column block of the wide
    orientation, i.e. ``[m, n_local]`` when ``transposed`` is false and
    ``[m_local, n]`` (a row block of the tall matrix) when it is true.  Returns
    the matching block of the orthogonalised matrix in fp32."""
    rows, cols = int(U_local.shape[0]), int(U_local.shape[1])
    d = int(segments[0].shape[-1])
    assert (cols if transposed else rows) == d
    K = float(2 ** round(__import__("math").log2(__import__("math").sqrt(d))))
    scale = (K / normalizer).reshape(1).float()
    Uc = U_local if (U_local.is_contiguous() and U_local.dtype in MT._DT) else U_local.float().contiguous()
    X = torch.empty(rows, cols, device=U_local.device, dtype=torch.float16)
    MT.cast([Uc], [X], scale=scale, slots=[0])
    last = len(segments) - 1
    for i, Q in enumerate(segments):
        out = torch.empty(rows, cols, device=U_local.device, dtype=torch.float32 if i == last else torch.float16)
        alpha = 1.0 / K if i == last else 1.0
        if transposed:
            G.gemm(X, Q, out, alpha=alpha)               # X Q  (Q symmetric)
        else:
            G.gemm(Q, X, out, b_mn=True, alpha=alpha)    # Q X
        X = out
    return X


def factors_supported(rows_local: int, cols_local: int) -> bool:
    """Operand pitches of the tcgen05 GEMM are multiples of 8 elements."""
    return rows_local % 8 == 0 and cols_local % 8 == 0


def newton_schulz_single(G_in, coefs, restarts, eps, formulation, compute_dtype) -> torch.Tensor:
    shape = G_in.shape
    X = G_in.reshape(1, shape[0], -1)
    if not X.is_contiguous():
        X = X.contiguous()
    return newton_schulz_batched(X, coefs, restarts, eps, formulation, compute_dtype).reshape(shape)


def muon_update_batched(
    grads: Sequence[torch.Tensor],
    moms: Sequence[torch.Tensor],
    masters: Optional[Sequence[torch.Tensor]],
    *,
    mu: float,
    nesterov: bool,
    coefs,
    restarts,
    formulation: str,
    lr: float,
    weight_decay: float,
    update_scale: float,
    eps: float = 1e-7,
    compute_dtype: Optional[torch.dtype] = None,
    publish: Optional[Sequence[torch.Tensor]] = None,
    deltas: Optional[Sequence[torch.Tensor]] = None,
    gscale: Optional[torch.Tensor] = None,
    peer=None,
    publish_multicast: Optional[Sequence[int]] = None,
) -> bool:
    """Momentum, Newton-Schulz and the weight update for ``L`` same-shape
    matrices.

    ``masters[i]`` (fp32, ``m0 x n0``) is updated in place:
    ``W = (1 - lr*wd) W - lr*update_scale*NS(u)``; ``publish[i]`` (bf16) receives
    a copy of the new weights.  With ``deltas`` instead of ``masters`` the
    pre-scaled update ``-lr*update_scale*NS(u)`` is written there (fp32) and no
    weight is touched (tensor-parallel owners scatter it).

    ``publish_multicast[i]`` (an address in the NVSwitch multicast mapping of the
    publish arena, same slot as ``publish[i]``) makes the last product store the
    bf16 copy with ``multimem.st``: every rank's arena receives it.

    Returns whether the bf16 copies were written (by the last product); if not,
    the caller still has to publish the new master weights.
    """
    L = len(moms)
    if L == 0:
        return False
    m0, n0 = int(moms[0].shape[0]), int(moms[0].numel() // moms[0].shape[0])
    dev = moms[0].device

    def prologue(xs_out, xscale=None):
        if peer is not None and hasattr(peer, "launch_prologue"):
            # tensor-parallel gather fused into the prologue: every shard is read where it lies
            peer.launch_prologue(moms, xs_out, slots, ws.sumsq, mu=mu, nesterov=nesterov, gscale=gscale,
                                 xscale=xscale)
        elif peer is not None:
            # reduce-to-owner fused into the prologue: gradients are read from
            # every rank's arena through its peer mapping
            from . import peer as P

            P.peer_prologue(peer.peer_bases, peer.offsets, peer.numels, peer.grad_dtype, moms, xs_out, slots,
                            ws.sumsq, scale=peer.scale, mu=mu, nesterov=nesterov, gscale=gscale,
                            ready_flags=peer.ready_flags, ready_want=peer.ready_want, status=peer.status,
                            xscale=xscale)
        else:
            MT.muon_prologue(grads, moms, xs_out, slots, ws.sumsq, mu, nesterov, gscale, xscale=xscale)

    cd = _resolve_dtype(compute_dtype, formulation)
    ws = workspace(L, m0, n0, cd, dev)
    left = m0 <= n0
    ws.sumsq.zero_()
    slots = list(range(L))
    owner_key = tuple(m.data_ptr() for m in moms)     # which matrices: their momentum buffers live as long as they do
    if cd == torch.bfloat16 and formulation == "gram":
        # one pass: the raw bf16 operand carries its scale as a per-matrix vector
        prologue([ws.X[i].reshape(-1) for i in range(L)])
        MT.norm_scales(ws.sumsq, ws.scale, ws.scale2, eps)
        xscale = _XScale(vec=ws.scale, vec2=ws.scale2)
    elif cd == torch.float16 and formulation == "gram" and SINGLE_PASS_FP16 and owner_key in _prescales:
        # one pass: the fp16 operand is stored with LAST step's K / ||u|| of the same matrices (momentum
        # makes the norm drift slowly, and fp16 has three orders of magnitude of room on either side of
        # the entries' size), and the products carry the exact correction ||u||_prev / ||u||_now per
        # matrix, so the result is scaled by this step's true norm
        K = fp16_prescale(m0, n0)
        pre = _prescales[owner_key]
        prologue([ws.X[i].reshape(-1) for i in range(L)], xscale=pre)
        MT.norm_scales(ws.sumsq, ws.scale, ws.scale2, eps)
        torch.div(ws.scale, pre, out=ws.fix)                  # (1/||u||) / (K/||u||_prev)
        torch.mul(ws.fix, ws.fix, out=ws.fix2)
        torch.mul(ws.scale, K, out=pre)                       # what the next step stores with
        xscale = _XScale(vec=ws.fix, vec2=ws.fix2)
    else:
        # two passes: fp32 staging, then normalise (and prescale fp16) while casting
        if ws.Xf32 is None:
            ws.Xf32 = torch.empty(L, m0, n0, device=dev, dtype=torch.float32)
        stage = [ws.Xf32[i] for i in range(L)]
        prologue([t.reshape(-1) for t in stage])
        MT.norm_scales(ws.sumsq, ws.scale, ws.scale2, eps)
        K = fp16_prescale(m0, n0) if (cd == torch.float16 and formulation == "gram") else 1.0
        if K != 1.0:
            ws.scale.mul_(K)
        MT.cast(stage, [ws.X[i] for i in range(L)], scale=ws.scale, slots=slots)
        xscale = _XScale(h=1.0 / K)
        if cd == torch.float16 and formulation == "gram" and SINGLE_PASS_FP16:
            # from the next step on these matrices take the single-pass path (ws.scale holds K / ||u||)
            if len(_prescales) > 4096:
                _prescales.clear()
            _prescales[owner_key] = ws.scale.clone()

    step_alpha = -float(lr) * float(update_scale)
    if formulation == "direct":
        kw: dict = {}
        _run(ws, coefs, restarts, formulation, left, xscale, kw)
        O = kw["copy_from"]
        with torch.no_grad():
            for i in range(L):
                if deltas is not None:
                    deltas[i].copy_(O[i].view_as(deltas[i]).float() * step_alpha)
                else:
                    w = masters[i].view(m0, n0)
                    if weight_decay:
                        w.mul_(1.0 - lr * weight_decay)
                    w.add_(O[i], alpha=step_alpha)
                    if publish is not None and publish[i] is not None and publish_multicast is None:
                        publish[i].view(m0, n0).copy_(w)
        return deltas is None and publish is not None and publish_multicast is None and all(
            p is not None for p in publish)

    if deltas is not None:
        kw = dict(out_ptrs=_ptr_table(deltas), out_ld=n0, out_dtype=deltas[0].dtype, alpha=step_alpha)
    else:
        tab = _ptr_table(masters)
        kw = dict(
            out_ptrs=tab,
            c_ptrs=tab,
            out_ld=n0,
            out_dtype=masters[0].dtype,
            alpha=step_alpha,
            beta=1.0 - float(lr) * float(weight_decay),
        )
        if publish_multicast is not None:
            kw["out2_ptrs"] = _addr_table(publish_multicast, dev)
            kw["out2_ld"] = n0
            kw["out2_multicast"] = True
        elif publish is not None and all(p is not None for p in publish):
            kw["out2_ptrs"] = _ptr_table(publish)
            kw["out2_ld"] = n0
    _run(ws, coefs, restarts, formulation, left, xscale, kw)
    return "out2_ptrs" in kw

"""Python front end of the tcgen05 GEMM kernel (``csrc/gemm_sm100.cu``).

``gemm`` computes, for every matrix of a batch,

    D = alpha * A @ B^T + beta * C + diag * I

where ``A`` supplies ``M x K`` and ``B`` supplies ``N x K``.  Each operand is
either stored K-major (``[M, K]`` row-major) or MN-major (``[K, M]``
row-major), so the four products Newton-Schulz needs -- ``X X^T``, ``X^T X``,
``Q X`` and ``X Q`` -- all run on the stored ``X`` without a transposed copy.
With ``symmetric=True`` only tiles that touch the lower triangle are computed
and strictly-lower tiles are also stored transposed, which halves the tensor
work of Gram products (the reference's SYRK idea,
dmuon/kernels/syrk_sm80.py:142-145, here on 128 x BN tcgen05 tiles).
"""
from __future__ import annotations

import ctypes
from functools import lru_cache

import torch

from . import build as _build

BM = 128


class _GemmArgs(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p),
        ("B", ctypes.c_void_p),
        ("lda", ctypes.c_longlong),
        ("ldb", ctypes.c_longlong),
        ("strideA", ctypes.c_longlong),
        ("strideB", ctypes.c_longlong),
        ("a_mn_major", ctypes.c_int),
        ("b_mn_major", ctypes.c_int),
        ("ab_fp16", ctypes.c_int),
        ("M", ctypes.c_int),
        ("N", ctypes.c_int),
        ("K", ctypes.c_int),
        ("batch", ctypes.c_int),
        ("tile_tab", ctypes.c_void_p),
        ("tiles_per_batch", ctypes.c_int),
        ("bn", ctypes.c_int),
        ("alpha", ctypes.c_float),
        ("beta", ctypes.c_float),
        ("diag", ctypes.c_float),
        ("alpha_vec", ctypes.c_void_p),
        ("C", ctypes.c_void_p),
        ("D", ctypes.c_void_p),
        ("D2", ctypes.c_void_p),
        ("C_tab", ctypes.c_void_p),
        ("D_tab", ctypes.c_void_p),
        ("D2_tab", ctypes.c_void_p),
        ("ldc", ctypes.c_longlong),
        ("ldd", ctypes.c_longlong),
        ("ldd2", ctypes.c_longlong),
        ("strideC", ctypes.c_longlong),
        ("strideD", ctypes.c_longlong),
        ("strideD2", ctypes.c_longlong),
        ("out_kind", ctypes.c_int),
        ("b_ready", ctypes.c_void_p),
        ("b_ready_epoch", ctypes.c_int),
        ("status", ctypes.c_void_p),
        ("max_ctas", ctypes.c_int),
        ("two_cta", ctypes.c_int),
        ("d2_multimem", ctypes.c_int),
    ]


_OUT_KIND = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

_status_bufs: dict[int, torch.Tensor] = {}
_tile_cache: dict[tuple, tuple[torch.Tensor, int]] = {}


class KernelTimeout(RuntimeError):
    """A bounded wait inside one of the kernels ran out (status word != 0)."""


def status_buffer(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_bufs[idx] = buf
    return buf


_STATUS_NAMES = {
    1: "TMA producer waited for a free pipeline stage",
    2: "MMA issuer waited for operands or a free accumulator",
    3: "epilogue waited for an accumulator",
    4: "wait on a peer / ready flag ran out (a rank did not signal in time)",
    5: "bad argument",
}


def describe_status(code: int) -> str:
    """What a non-zero status word written by one of the kernels means."""
    return _STATUS_NAMES.get(int(code), f"unknown status {int(code)}")


def check_status(device: torch.device | None = None) -> None:
    """Synchronising read of the status word; raises if any kernel gave up."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    code = int(status_buffer(device)[0].item())
    if code != 0:
        status_buffer(device).zero_()
        raise KernelTimeout(f"dmuon_b200 kernel wait ran out (code {code}: {describe_status(code)})")


def symmetric_tiles(m: int, bn: int, bm: int = BM) -> list[tuple[int, int, int]]:
    """Tiles (row_tile, col_tile, mirror) covering the lower triangle of m x m.

    A tile is kept when any of its elements has row >= col; a tile whose
    columns all lie strictly left of its rows is additionally stored
    transposed.  Tiles that straddle the diagonal store what they compute.
    """
    out = []
    mt = (m + bm - 1) // bm
    for i in range(mt):
        last_row = min(m, (i + 1) * bm) - 1
        for j in range(last_row // bn + 1):
            mirror = 1 if (j + 1) * bn <= i * bm else 0
            out.append((i, j, mirror))
    return out


def dense_tiles(m: int, n: int, bn: int, bm: int = BM) -> list[tuple[int, int, int]]:
    mt = (m + bm - 1) // bm
    nt = (n + bn - 1) // bn
    # column tile outermost: CTAs that run at the same time share B tiles in L2
    return [(i, j, 0) for j in range(nt) for i in range(mt)]


def tile_table(m: int, n: int, bn: int, symmetric: bool, device: torch.device, bm: int = BM) -> tuple[torch.Tensor, int]:
    """Device table of (row_tile, col_tile, flags, 0); row tiles are ``bm`` rows
    (128 for the single-CTA kernel, 256 for CTA pairs)."""
    key = (m, n, bn, symmetric, device.index, bm)
    hit = _tile_cache.get(key)
    if hit is None:
        tiles = symmetric_tiles(m, bn, bm) if symmetric else dense_tiles(m, n, bn, bm)
        flat = [[i, j, f, 0] for (i, j, f) in tiles]
        tab = torch.tensor(flat, dtype=torch.int32).to(device)
        hit = (tab, len(tiles))
        _tile_cache[key] = hit
    return hit


def quad_tile_list(m: int, n: int, symmetric: bool) -> list[tuple[int, int, int, int]]:
    """Entries of the CTA-quad kernel's tile list: two 256 x 256 tiles each,
    ``(m0 | m1 << 16, n0 | n1 << 16, flags, 0)`` with flag bits 0 / 1 = mirror
    tile 0 / 1, bit 2 = both tiles cover the same rows (their A operand is then
    loaded once per cluster), bit 3 = tile 1 is a filler that stores nothing.

    Tiles are paired inside a row of tiles; what is left over (rows with an odd
    number of tiles) is paired across rows without sharing, and a last single
    tile gets a filler partner."""
    mt, nt = (m + 255) // 256, (n + 255) // 256
    out: list[tuple[int, int, int, int]] = []
    left: list[tuple[int, int, int]] = []

    def emit_row(i: int, cols: list[tuple[int, int]]) -> None:
        for k in range(0, len(cols) - 1, 2):
            (j0, f0), (j1, f1) = cols[k], cols[k + 1]
            out.append((i | (i << 16), j0 | (j1 << 16), f0 | (f1 << 1) | 4, 0))
        if len(cols) % 2:
            left.append((i, cols[-1][0], cols[-1][1]))

    if symmetric:
        for i in range(mt):
            last_row = min(m, (i + 1) * 256) - 1
            emit_row(i, [(j, 1 if (j + 1) * 256 <= i * 256 else 0) for j in range(last_row // 256 + 1)])
    else:
        # column pairs outermost: clusters that run at the same time share B tiles in L2
        for jp in range(0, nt, 2):
            for i in range(mt):
                emit_row(i, [(j, 0) for j in range(jp, min(jp + 2, nt))])
    for k in range(0, len(left) - 1, 2):
        (i0, j0, f0), (i1, j1, f1) = left[k], left[k + 1]
        out.append((i0 | (i1 << 16), j0 | (j1 << 16), f0 | (f1 << 1), 0))
    if len(left) % 2:
        i0, j0, f0 = left[-1]
        out.append((i0 | (i0 << 16), j0 | (j0 << 16), f0 | 8, 0))
    return out


def quad_tile_table(m: int, n: int, symmetric: bool, device: torch.device) -> tuple[torch.Tensor, int]:
    key = ("quad", m, n, symmetric, device.index)
    hit = _tile_cache.get(key)
    if hit is None:
        tiles = quad_tile_list(m, n, symmetric)
        tab = torch.tensor([list(t) for t in tiles], dtype=torch.int32).to(device)
        hit = (tab, len(tiles))
        _tile_cache[key] = hit
    return hit


@lru_cache(maxsize=None)
def quad_max_clusters() -> int:
    """Clusters of four CTAs the quad kernel can keep resident on this device
    (0: unavailable)."""
    lib = _build.load()
    fn = lib.dmuon_gemm_quad_max_clusters
    fn.restype = ctypes.c_int
    return int(fn())


def cluster_mode() -> str:
    """``DMUON_GEMM_CLUSTER``: ``pair`` (default: one ``cta_group::2`` pair per
    256 x 256 tile) or ``quad`` (two pairs per cluster share their A rows
    through distributed shared memory: 0.75 x the L2 reads per tile, but the
    load -> forward -> consume chain is longer than the seven stages that fit
    in shared memory can cover, and only 33 clusters of four fit on 148 SMs;
    measured 3-4 x slower than pairs on a B200, kept as an option and a test
    subject)."""
    import os

    return os.environ.get("DMUON_GEMM_CLUSTER", "pair").strip().lower()


def quad_kernel_pays(m: int, n: int, batch: int, symmetric: bool) -> bool:
    """Enough tile pairs to keep every cluster busy for at least two rounds."""
    if m < 256 or n < 512 or m > 0xFFFF * 256 or n > 0xFFFF * 256:
        return False
    return _quad_entries(m, n, symmetric) * batch >= 2 * 37


@lru_cache(maxsize=None)
def _quad_entries(m: int, n: int, symmetric: bool) -> int:
    return len(quad_tile_list(m, n, symmetric))


@lru_cache(maxsize=None)
def _fn():
    lib = _build.load()
    fn = lib.dmuon_gemm_sm100
    fn.argtypes = [ctypes.POINTER(_GemmArgs), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


#: run large products on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles)
TWO_CTA_DEFAULT = True


def pair_kernel_pays(m: int, n: int, batch: int, symmetric: bool) -> bool:
    """CTA pairs need enough 256 x 256 tiles to keep 74 pairs busy."""
    if m < 256 or n < 256:
        return False
    tiles = len(symmetric_tiles(m, 256, 256)) if symmetric else ((m + 255) // 256) * ((n + 255) // 256)
    return tiles * batch >= 74


def pick_bn(m: int, n: int, batch: int, symmetric: bool) -> int:
    """128-wide tiles when 256-wide ones would leave most SMs without a tile."""
    if n <= 128:
        return 128
    t256 = len(symmetric_tiles(m, 256)) if symmetric else ((m + BM - 1) // BM) * ((n + 255) // 256)
    return 256 if t256 * batch >= 148 else 128


def gemm(
    A: torch.Tensor,
    B: torch.Tensor,
    out: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    C: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    diag: float = 0.0,
    symmetric: bool = False,
    out2: torch.Tensor | None = None,
    bn: int | None = None,
    out_ptrs: torch.Tensor | None = None,
    c_ptrs: torch.Tensor | None = None,
    out2_ptrs: torch.Tensor | None = None,
    out_ld: int | None = None,
    out2_ld: int | None = None,
    out_dtype: torch.dtype | None = None,
    alpha_vec: torch.Tensor | None = None,
    b_ready: torch.Tensor | None = None,
    b_ready_epoch: int = 0,
    max_ctas: int = 0,
    two_cta: bool | int | None = None,
    out2_multicast: bool = False,
) -> torch.Tensor:
    """Launch one batched product on the current CUDA stream.

    ``A``/``B`` are 2-D or 3-D (leading batch) bf16 or fp16 tensors whose last
    dimension is contiguous.  ``out`` (and ``C``) are bf16, fp16 or fp32 of the
    same dtype.  When ``out_ptrs`` (an int64 device tensor with one address per
    batch entry) is given, ``out`` may be ``None`` and each matrix is written to
    its own allocation (same for ``c_ptrs`` / ``out2_ptrs``).  With
    ``out2_multicast`` the addresses in ``out2_ptrs`` lie in the NVSwitch multicast
    mapping of a symmetric buffer and the bf16 copy is stored to every rank at once.
    """
    if A.dim() == 2:
        A = A.unsqueeze(0)
    if B.dim() == 2:
        B = B.unsqueeze(0)
    assert A.dtype == B.dtype and A.dtype in (torch.bfloat16, torch.float16)
    assert A.stride(-1) == 1 and B.stride(-1) == 1
    batch = A.shape[0]
    assert B.shape[0] == batch
    if a_mn:
        K, M = A.shape[1], A.shape[2]
    else:
        M, K = A.shape[1], A.shape[2]
    if b_mn:
        Kb, N = B.shape[1], B.shape[2]
    else:
        N, Kb = B.shape[1], B.shape[2]
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if symmetric:
        assert M == N
    dev = A.device
    if bn is None:
        bn = pick_bn(M, N, batch, symmetric)
    if two_cta is None:
        two_cta = TWO_CTA_DEFAULT and pair_kernel_pays(M, N, batch, symmetric)
        if two_cta and cluster_mode() == "quad" and quad_kernel_pays(M, N, batch, symmetric) and quad_max_clusters() > 0:
            two_cta = 2
    two_cta = int(two_cta)
    if two_cta:
        bn = 256
    if two_cta == 2:
        tab, ntiles = quad_tile_table(M, N, symmetric, dev)
    else:
        tab, ntiles = tile_table(M, N, bn, symmetric, dev, 256 if two_cta else BM)

    args = _GemmArgs()
    args.A = A.data_ptr()
    args.B = B.data_ptr()
    args.lda = A.stride(1)
    args.ldb = B.stride(1)
    args.strideA = A.stride(0) if batch > 1 else 0
    args.strideB = B.stride(0) if batch > 1 else 0
    args.a_mn_major = int(a_mn)
    args.b_mn_major = int(b_mn)
    args.ab_fp16 = int(A.dtype == torch.float16)
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.tile_tab = tab.data_ptr()
    args.tiles_per_batch = ntiles
    args.bn = bn
    args.alpha, args.beta, args.diag = float(alpha), float(beta), float(diag)

    if out is not None:
        if out.dim() == 2:
            out = out.unsqueeze(0)
        assert out.stride(-1) == 1 and out.shape[-2:] == (M, N)
        odt = out.dtype
        args.D = out.data_ptr()
        args.ldd = out.stride(1)
        args.strideD = out.stride(0) if batch > 1 else 0
    else:
        assert out_ptrs is not None and out_ld is not None and out_dtype is not None
        odt = out_dtype
        args.D_tab = out_ptrs.data_ptr()
        args.ldd = out_ld
    args.out_kind = _OUT_KIND[odt]
    if C is not None:
        if C.dim() == 2:
            C = C.unsqueeze(0)
        assert C.dtype == odt and C.stride(-1) == 1
        args.C = C.data_ptr()
        args.ldc = C.stride(1)
        args.strideC = C.stride(0) if batch > 1 else 0
    elif c_ptrs is not None:
        args.C_tab = c_ptrs.data_ptr()
        args.ldc = args.ldd
    if out2 is not None:
        if out2.dim() == 2:
            out2 = out2.unsqueeze(0)
        assert out2.dtype == torch.bfloat16 and out2.stride(-1) == 1
        args.D2 = out2.data_ptr()
        args.ldd2 = out2.stride(1)
        args.strideD2 = out2.stride(0) if batch > 1 else 0
    elif out2_ptrs is not None:
        args.D2_tab = out2_ptrs.data_ptr()
        args.ldd2 = out2_ld if out2_ld is not None else args.ldd
    if out2_multicast:
        # out2 / out2_ptrs are addresses in the multicast mapping of a symmetric buffer
        assert not symmetric and N % 8 == 0 and int(args.ldd2) % 8 == 0 and (args.D2 or args.D2_tab)
        args.d2_multimem = 1
    if alpha_vec is not None:
        assert alpha_vec.dtype == torch.float32 and alpha_vec.numel() >= batch
        args.alpha_vec = alpha_vec.data_ptr()
    if b_ready is not None:
        args.b_ready = b_ready.data_ptr()
        args.b_ready_epoch = int(b_ready_epoch)
    args.status = status_buffer(dev).data_ptr()
    args.max_ctas = int(max_ctas)
    args.two_cta = two_cta
    rc = _fn()(ctypes.byref(args), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"dmuon_gemm_sm100 failed with code {rc}")
    return out

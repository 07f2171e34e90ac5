"""The allocation-free symmetric-product entry point, called the way a host
that cannot allocate device memory would call it: through the exported C
symbol, with nothing but input and output pointers.

Such callers exist -- a plugin inside another runtime's memory pool, a control
loop that cannot afford an allocation's latency, a plain C program -- and for
them the kernel's tile table and status word sit in a fixed array inside the
library.  The result must equal the regular entry point's, also on a second
call that reuses (and therefore first has to reset) that array.

This file sorts last on purpose: a run that stops at the first failure has
then already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from dmuon_b200.ops import build

    lib = build.load()
    fn = lib.dmuon_syrk_noalloc
    fn.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong,
        ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_void_p,
    ]
    fn.restype = ctypes.c_int
    lib.dmuon_syrk_noalloc_status.argtypes = [ctypes.c_void_p]
    lib.dmuon_syrk_noalloc_status.restype = ctypes.c_int
    lib.dmuon_syrk_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.dmuon_syrk_noalloc_strerror.restype = ctypes.c_char_p
    return lib, fn


def _call(fn, X, D, M, K, batch, mn, alpha, diag):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(
        ctypes.c_void_p(X.data_ptr()), ctypes.c_void_p(D.data_ptr()), M, K, batch, X.stride(1), D.stride(1),
        X.stride(0) if batch > 1 else 0, D.stride(0) if batch > 1 else 0,
        int(X.dtype == torch.float16), int(mn), alpha, diag, stream,
    )


def test_no_alloc_entry_matches_regular_entry_twice_in_a_row():
    from dmuon_b200.ops import gemm as G

    lib, fn = _entry()
    dev = torch.device("cuda", 0)
    torch.manual_seed(11)
    # two different problems back to back: the second call must not see the
    # first call's tile table or status
    cases = [
        dict(M=1152, K=2048, batch=3, dtype=torch.bfloat16, mn=False, alpha=0.75, diag=0.5),
        dict(M=640, K=1024, batch=2, dtype=torch.float16, mn=True, alpha=1.25, diag=0.0),
    ]
    for n, c in enumerate(cases):
        M, K, L = c["M"], c["K"], c["batch"]
        X = (torch.randn(L, K, M, device=dev) if c["mn"] else torch.randn(L, M, K, device=dev)).mul_(0.05).to(c["dtype"])
        want = torch.empty(L, M, M, device=dev, dtype=c["dtype"])
        G.gemm(X, X, want, a_mn=c["mn"], b_mn=c["mn"], alpha=c["alpha"], diag=c["diag"], symmetric=True, bn=256)
        got = torch.full((L, M, M), float("nan"), device=dev, dtype=c["dtype"])
        torch.cuda.synchronize(dev)
        before = torch.cuda.memory_allocated(dev)
        free_before, _ = torch.cuda.mem_get_info(dev)
        rc = _call(fn, X, got, M, K, L, c["mn"], c["alpha"], c["diag"])
        assert rc == 0, lib.dmuon_syrk_noalloc_strerror(rc)
        assert lib.dmuon_syrk_noalloc_status(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        assert torch.cuda.memory_allocated(dev) == before
        if n > 0:
            # torch's counter cannot see a raw cudaMalloc; the driver's free-memory figure can.  Only
            # checked from the second call on: the first one may make the driver load the kernels.
            free_after, _ = torch.cuda.mem_get_info(dev)
            assert free_after >= free_before
        G.check_status(dev)
        scale = want.float().abs().max().item() + 1e-6
        assert not torch.isnan(got.float()).any()
        assert (got.float() - want.float()).abs().max().item() / scale < 2e-2
        # and against plain fp32 math
        Xf = X.float().transpose(1, 2) if c["mn"] else X.float()
        ref = c["alpha"] * Xf @ Xf.transpose(1, 2) + c["diag"] * torch.eye(M, device=dev)
        assert (got.float() - ref).abs().max().item() / scale < 2e-2


def test_no_alloc_entry_rejects_what_does_not_fit():
    lib, fn = _entry()
    dev = torch.device("cuda", 0)
    X = torch.zeros(1, 128, 64, device=dev, dtype=torch.bfloat16)
    D = torch.zeros(1, 128, 128, device=dev, dtype=torch.bfloat16)
    # claims a 40000 x 40000 output: more tiles than the built-in table holds; nothing is launched
    rc = _call(fn, X, D, 40000, 64, 1, False, 1.0, 0.0)
    assert rc == -22
    assert b"too large" in lib.dmuon_syrk_noalloc_strerror(rc)
    # pitch that is not a multiple of 8 elements
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(ctypes.c_void_p(X.data_ptr()), ctypes.c_void_p(D.data_ptr()), 128, 64, 1, 60, 128, 0, 0, 0, 0, 1.0, 0.0, stream)
    assert rc == -1
    # two matrices that would share one output (zero batch stride)
    X2 = torch.zeros(2, 128, 64, device=dev, dtype=torch.bfloat16)
    rc = fn(ctypes.c_void_p(X2.data_ptr()), ctypes.c_void_p(D.data_ptr()), 128, 64, 2, 64, 128, 128 * 64, 0, 0, 0, 1.0, 0.0, stream)
    assert rc == -1
    assert float(D.abs().sum()) == 0.0

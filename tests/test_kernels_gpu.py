"""sm_100a kernels against plain PyTorch fp32 references (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _ref_gemm(A, B, a_mn, b_mn, C, alpha, beta, diag):
    Af = A.float().transpose(-1, -2) if a_mn else A.float()
    Bf = B.float().transpose(-1, -2) if b_mn else B.float()
    D = alpha * Af @ Bf.transpose(-1, -2)
    if C is not None:
        D = D + beta * C.float()
    if diag:
        D = D + diag * torch.eye(D.shape[-2], D.shape[-1], device=D.device)
    return D


CASES = [
    # M, N, K, batch, a_mn, b_mn, bn, symmetric, dtype, out dtype, epilogue
    (128, 128, 64, 1, False, False, 128, False, torch.bfloat16, torch.bfloat16, False),
    (512, 768, 1024, 1, False, False, 256, False, torch.bfloat16, torch.bfloat16, False),
    (200, 300, 136, 1, False, False, 128, False, torch.bfloat16, torch.bfloat16, True),
    (256, 256, 512, 5, False, False, 128, False, torch.float16, torch.float16, False),
    (256, 512, 512, 2, False, False, 256, False, torch.bfloat16, torch.float32, True),
    (512, 512, 1024, 1, False, False, 128, True, torch.bfloat16, torch.bfloat16, True),
    (1152, 1152, 4304, 1, False, False, 256, True, torch.bfloat16, torch.bfloat16, False),
    (256, 512, 512, 1, False, True, 256, False, torch.bfloat16, torch.bfloat16, False),
    (256, 512, 512, 1, True, False, 256, False, torch.bfloat16, torch.bfloat16, False),
    (384, 512, 448, 1, True, True, 128, False, torch.bfloat16, torch.bfloat16, False),
    (512, 512, 1024, 2, True, True, 256, True, torch.bfloat16, torch.bfloat16, True),
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_gemm_matches_fp32(case):
    from dmuon_b200.ops import gemm as G

    M, N, K, batch, a_mn, b_mn, bn, sym, dt, odt, epi = case
    dev = _dev()
    torch.manual_seed(0)
    if sym:
        X = (torch.randn(batch, M, K, device=dev) * 0.1).to(dt)
        A = X.transpose(1, 2).contiguous() if a_mn else X
        B = X.transpose(1, 2).contiguous() if b_mn else X
    else:
        A = ((torch.randn(batch, K, M, device=dev) if a_mn else torch.randn(batch, M, K, device=dev)) * 0.1).to(dt)
        B = ((torch.randn(batch, K, N, device=dev) if b_mn else torch.randn(batch, N, K, device=dev)) * 0.1).to(dt)
    C = None
    alpha, beta, diag = 1.0, 0.0, 0.0
    if epi:
        C = torch.randn(batch, M, N, device=dev)
        if sym:
            C = C + C.transpose(1, 2)
        C = C.to(odt)
        alpha, beta, diag = 1.5, -0.5, (0.3 if M == N else 0.0)
    out = torch.full((batch, M, N), float("nan"), device=dev, dtype=odt)
    out2 = torch.full((batch, M, N), float("nan"), device=dev, dtype=torch.bfloat16) if odt == torch.float32 else None
    G.gemm(A, B, out, a_mn=a_mn, b_mn=b_mn, C=C, alpha=alpha, beta=beta, diag=diag, symmetric=sym, bn=bn, out2=out2)
    torch.cuda.synchronize()
    G.check_status(dev)
    ref = _ref_gemm(A, B, a_mn, b_mn, C, alpha, beta, diag)
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if odt != torch.float32 else 2e-3
    assert not torch.isnan(out.float()).any()
    assert (out.float() - ref).abs().max().item() / scale < tol
    if out2 is not None:
        assert (out2.float() - ref).abs().max().item() / scale < 2e-2


PAIR_CASES = [
    # M, N, K, batch, a_mn, b_mn, symmetric, out dtype, epilogue
    (256, 256, 64, 1, False, False, False, torch.bfloat16, False),
    (512, 768, 1024, 2, False, False, False, torch.bfloat16, True),
    (384, 640, 320, 1, False, False, False, torch.bfloat16, False),      # ragged in M and N
    (512, 1024, 512, 1, False, True, False, torch.float32, True),
    (512, 512, 512, 1, True, False, False, torch.bfloat16, False),
    (768, 512, 448, 1, True, True, False, torch.bfloat16, False),
    (1024, 1024, 512, 3, False, False, True, torch.bfloat16, True),
    (1152, 1152, 4304, 1, False, False, True, torch.bfloat16, False),
    (512, 512, 1024, 2, True, True, True, torch.float16, True),
]


@pytest.mark.parametrize("case", PAIR_CASES, ids=[f"pair{i}" for i in range(len(PAIR_CASES))])
def test_gemm_pair_kernel_matches_fp32(case):
    """CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 tiles)."""
    _run_cluster_case(case, 1)


QUAD_CASES = PAIR_CASES + [
    # one shared pair of tiles per row, K of a single block
    (256, 512, 64, 1, False, False, False, torch.bfloat16, False),
    # three column tiles per row: shared pairs plus unshared left-overs, odd total -> a filler tile
    (768, 768, 2368, 1, False, False, False, torch.bfloat16, True),
    # many k-blocks (several trips around the stage ring), both operand layouts, batch
    (512, 1024, 4096, 2, False, True, False, torch.bfloat16, False),
    (1024, 1024, 1472, 2, True, True, True, torch.bfloat16, True),
    # larger symmetric product, fp16 operands, batch 3
    (2048, 2048, 1024, 3, False, False, True, torch.float16, True),
]


@pytest.mark.parametrize("case", QUAD_CASES, ids=[f"quad{i}" for i in range(len(QUAD_CASES))])
def test_gemm_quad_kernel_matches_fp32(case):
    """CTA-quad kernel: two CTA pairs per cluster, A rows forwarded between the
    pairs through distributed shared memory."""
    from dmuon_b200.ops import gemm as G

    assert G.quad_max_clusters() > 0
    _run_cluster_case(case, 2)


def _run_cluster_case(case, two_cta):
    from dmuon_b200.ops import gemm as G

    M, N, K, batch, a_mn, b_mn, sym, odt, epi = case
    dt = torch.float16 if odt == torch.float16 else torch.bfloat16
    dev = _dev()
    torch.manual_seed(0)
    if sym:
        X = (torch.randn(batch, M, K, device=dev) * 0.1).to(dt)
        A = X.transpose(1, 2).contiguous() if a_mn else X
        B = X.transpose(1, 2).contiguous() if b_mn else X
    else:
        A = ((torch.randn(batch, K, M, device=dev) if a_mn else torch.randn(batch, M, K, device=dev)) * 0.1).to(dt)
        B = ((torch.randn(batch, K, N, device=dev) if b_mn else torch.randn(batch, N, K, device=dev)) * 0.1).to(dt)
    C = None
    alpha, beta, diag = 1.0, 0.0, 0.0
    if epi:
        C = torch.randn(batch, M, N, device=dev)
        if sym:
            C = C + C.transpose(1, 2)
        C = C.to(odt)
        alpha, beta, diag = 1.5, -0.5, (0.3 if M == N else 0.0)
    out = torch.full((batch, M, N), float("nan"), device=dev, dtype=odt)
    G.gemm(A, B, out, a_mn=a_mn, b_mn=b_mn, C=C, alpha=alpha, beta=beta, diag=diag, symmetric=sym, two_cta=two_cta)
    torch.cuda.synchronize()
    G.check_status(dev)
    ref = _ref_gemm(A, B, a_mn, b_mn, C, alpha, beta, diag)
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if odt != torch.float32 else 2e-3
    assert not torch.isnan(out.float()).any()
    assert (out.float() - ref).abs().max().item() / scale < tol


def test_gemm_alpha_vec_and_pointer_tables():
    from dmuon_b200.ops import gemm as G

    dev = _dev()
    torch.manual_seed(1)
    L, M, N, K = 3, 256, 384, 256
    A = (torch.randn(L, M, K, device=dev) * 0.1).bfloat16()
    B = (torch.randn(L, K, N, device=dev) * 0.1).bfloat16()
    s = torch.tensor([0.5, 2.0, -1.0], device=dev)
    masters = [torch.randn(M, N, device=dev) for _ in range(L)]
    before = [m.clone() for m in masters]
    pubs = [torch.zeros(M, N, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    tab = torch.tensor([m.data_ptr() for m in masters], dtype=torch.int64, device=dev)
    ptab = torch.tensor([p.data_ptr() for p in pubs], dtype=torch.int64, device=dev)
    G.gemm(A, B, None, b_mn=True, out_ptrs=tab, c_ptrs=tab, out_ld=N, out_dtype=torch.float32,
           out2_ptrs=ptab, out2_ld=N, alpha=-0.1, beta=0.9, alpha_vec=s)
    torch.cuda.synchronize()
    G.check_status(dev)
    for i in range(L):
        ref = 0.9 * before[i] + (-0.1 * s[i]) * (A[i].float() @ B[i].float())
        assert (masters[i] - ref).abs().max().item() < 2e-3
        assert (pubs[i].float() - ref).abs().max().item() < 3e-2


def test_muon_prologue_and_scales():
    from dmuon_b200.ops import multi_tensor as MT

    dev = _dev()
    torch.manual_seed(2)
    shapes = [(256, 512), (128, 100), (33, 7)]
    grads = [torch.randn(s, device=dev).bfloat16() for s in shapes]
    moms = [torch.randn(s, device=dev) for s in shapes]
    moms0 = [m.clone() for m in moms]
    xs = [torch.empty(s, device=dev, dtype=torch.bfloat16) for s in shapes]
    sumsq = torch.zeros(3, device=dev)
    gs = torch.tensor(0.5, device=dev)
    MT.muon_prologue(grads, moms, xs, [0, 1, 2], sumsq, 0.95, True, gs)
    scale, scale2 = torch.empty(3, device=dev), torch.empty(3, device=dev)
    MT.norm_scales(sumsq, scale, scale2, 1e-7)
    torch.cuda.synchronize()
    for i in range(3):
        g = grads[i].float() * 0.5
        m = 0.95 * moms0[i] + g
        u = g + 0.95 * m
        assert torch.allclose(moms[i], m, atol=1e-5)
        assert (xs[i].float() - u).abs().max().item() < 0.02 * u.abs().max().item()
        assert abs(sumsq[i].item() - (u * u).sum().item()) < 1e-3 * (u * u).sum().item()
        assert abs(scale[i].item() - 1.0 / (u.norm().item() + 1e-7)) < 1e-3 * scale[i].item()


@pytest.mark.parametrize("pdt,gdt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
def test_adamw_matches_formula(pdt, gdt):
    from dmuon_b200.ops import multi_tensor as MT

    dev = _dev()
    torch.manual_seed(3)
    shapes = [(1000,), (64, 129), (3,)]
    ps = [torch.randn(s, device=dev).to(pdt) for s in shapes]
    gs = [torch.randn(s, device=dev).to(gdt) for s in shapes]
    ms = [torch.zeros(s, device=dev) for s in shapes]
    vs = [torch.zeros(s, device=dev) for s in shapes]
    ref_p = [p.float().clone() for p in ps]
    ref_m = [m.clone() for m in ms]
    ref_v = [v.clone() for v in vs]
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    for t in (1, 2, 3):
        MT.adamw(ps, gs, ms, vs, [t, t + 1, t + 2], lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd)
        for i in range(3):
            tt = t + i
            g = gs[i].float()
            base = ps_prev = ref_p[i]
            if pdt != torch.float32:
                base = base.to(pdt).float()
            ref_m[i] = b1 * ref_m[i] + (1 - b1) * g
            ref_v[i] = b2 * ref_v[i] + (1 - b2) * g * g
            denom = ref_v[i].sqrt() / math.sqrt(1 - b2**tt) + eps
            ref_p[i] = base * (1 - lr * wd) - (lr / (1 - b1**tt)) * ref_m[i] / denom
    torch.cuda.synchronize()
    tol = 1e-5 if pdt == torch.float32 else 3e-2
    for i in range(3):
        assert (ps[i].float() - ref_p[i]).abs().max().item() < tol
        assert torch.allclose(ms[i], ref_m[i], atol=1e-5)


def test_clip_kernels():
    from dmuon_b200.ops import multi_tensor as MT

    dev = _dev()
    torch.manual_seed(4)
    ts = [torch.randn(1000, device=dev), torch.randn(77, 13, device=dev).bfloat16(), torch.randn(5, device=dev).half()]
    seg = [0, 1, 0]
    acc = torch.zeros(2, device=dev)
    MT.clip_sumsq(ts, seg, acc)
    ref0 = ts[0].float().pow(2).sum() + ts[2].float().pow(2).sum()
    ref1 = ts[1].float().pow(2).sum()
    assert abs(acc[0].item() - ref0.item()) < 1e-3 * ref0.item()
    assert abs(acc[1].item() - ref1.item()) < 1e-3 * ref1.item()
    before = [t.float().clone() for t in ts]
    MT.clip_scale(ts, seg, torch.tensor([0.5, 0.25], device=dev))
    for t, b, c in zip(ts, before, (0.5, 0.25, 0.5)):
        assert (t.float() - b * c).abs().max().item() < 1e-2


def _orth_err(O):
    m, n = O.shape
    X = O.float() if m <= n else O.float().T
    return (X @ X.T - torch.eye(X.shape[0], device=O.device)).abs().max().item()


@pytest.mark.parametrize("shape", [(512, 1024), (1024, 512), (256, 2048), (1152, 4304)])
@pytest.mark.parametrize("formulation,cdt", [("gram", torch.float16), ("gram", torch.bfloat16), ("direct", torch.bfloat16)])
def test_newton_schulz_kernels_vs_fp32(shape, formulation, cdt):
    from dmuon_b200.ops import ns_sm100
    from dmuon_b200.optim import newton_schulz as NS

    dev = _dev()
    torch.manual_seed(5)
    L = 3
    Gm = torch.randn(L, *shape, device=dev)
    coefs = list(NS.POLAR_EXPRESS_COEFFICIENTS)
    restarts = [2] if formulation == "gram" else []
    out = ns_sm100.newton_schulz_batched(Gm, coefs, restarts, 1e-7, formulation, cdt)
    torch.cuda.synchronize()
    from dmuon_b200.ops import gemm as G

    G.check_status(dev)
    for i in range(L):
        if formulation == "gram":
            ref = NS.gram_newton_schulz(Gm[i], coefficients=coefs, restart_iterations=restarts, deterministic=True,
                                        compute_dtype=torch.float32)
        else:
            ref = NS.direct_newton_schulz(Gm[i], coefficients=coefs, compute_dtype=torch.float32)
        assert (out[i] - ref).abs().max().item() < (0.03 if cdt == torch.float16 else 0.1)
        assert _orth_err(out[i]) < 0.35
        if cdt == torch.float16:
            # fp16 operands track the fp32 iteration closely
            assert _orth_err(out[i]) < _orth_err(ref) + 0.03
        cos = torch.nn.functional.cosine_similarity(out[i].flatten(), ref.flatten(), dim=0).item()
        assert cos > 0.995


@pytest.mark.parametrize("cdt", [torch.float16, torch.bfloat16])
def test_muon_update_batched_matches_reference_math(cdt):
    from dmuon_b200.ops import ns_sm100
    from dmuon_b200.optim import newton_schulz as NS

    dev = _dev()
    torch.manual_seed(6)
    L, m, n = 4, 512, 1536
    grads = [torch.randn(m, n, device=dev).bfloat16() * 1e-3 for _ in range(L)]
    moms = [torch.randn(m, n, device=dev) * 1e-3 for _ in range(L)]
    masters = [torch.randn(m, n, device=dev) * 0.02 for _ in range(L)]
    pubs = [torch.zeros(m, n, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    m0 = [x.clone() for x in moms]
    w0 = [x.clone() for x in masters]
    coefs, restarts = list(NS.POLAR_EXPRESS_COEFFICIENTS), [2]
    lr, wd, mu = 0.02, 0.1, 0.95
    scale = 0.2 * math.sqrt(max(m, n))
    ns_sm100.muon_update_batched(grads, moms, masters, mu=mu, nesterov=True, coefs=coefs, restarts=restarts,
                                 formulation="gram", lr=lr, weight_decay=wd, update_scale=scale, publish=pubs,
                                 compute_dtype=cdt)
    torch.cuda.synchronize()
    from dmuon_b200.ops import gemm as G

    G.check_status(dev)
    for i in range(L):
        g = grads[i].float()
        buf = mu * m0[i] + g
        u = g + mu * buf
        o = NS.gram_newton_schulz(u, coefficients=coefs, restart_iterations=restarts, deterministic=True,
                                  compute_dtype=torch.float32)
        ref = w0[i] * (1 - lr * wd) - lr * scale * o
        assert torch.allclose(moms[i], buf, atol=1e-6)
        upd_err = (masters[i] - ref).abs().max().item()
        assert upd_err < 0.1 * lr * scale, upd_err
        assert (pubs[i].float() - masters[i]).abs().max().item() < 1e-2 * masters[i].abs().max().item()


def test_muon_update_single_pass_operand_on_later_steps():
    """From the second step on the fp16 Gram operand is written by the prologue
    itself, scaled with the previous step's norm, and the products carry the
    exact correction.  Three steps whose gradient norms differ by factors of 5
    and 1/20 must still match fp32 math step by step."""
    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import ns_sm100
    from dmuon_b200.optim import newton_schulz as NS

    dev = _dev()
    torch.manual_seed(8)
    L, m, n = 3, 512, 1024
    moms = [torch.zeros(m, n, device=dev) for _ in range(L)]
    masters = [torch.randn(m, n, device=dev) * 0.02 for _ in range(L)]
    ref_m = [x.clone() for x in moms]
    ref_w = [x.clone() for x in masters]
    coefs, restarts = list(NS.POLAR_EXPRESS_COEFFICIENTS), [2]
    lr, wd, mu = 0.02, 0.1, 0.9
    scale = 0.2 * math.sqrt(max(m, n))
    ns_sm100.release_workspaces()
    for step, gmag in enumerate([1e-3, 5e-3, 2.5e-4]):
        grads = [(torch.randn(m, n, device=dev) * gmag).bfloat16() for _ in range(L)]
        ns_sm100.muon_update_batched(grads, moms, masters, mu=mu, nesterov=True, coefs=coefs, restarts=restarts,
                                     formulation="gram", lr=lr, weight_decay=wd, update_scale=scale)
        torch.cuda.synchronize()
        G.check_status(dev)
        assert (tuple(x.data_ptr() for x in moms) in ns_sm100._prescales) == ns_sm100.SINGLE_PASS_FP16
        for i in range(L):
            g = grads[i].float()
            ref_m[i] = mu * ref_m[i] + g
            u = g + mu * ref_m[i]
            o = NS.gram_newton_schulz(u, coefficients=coefs, restart_iterations=restarts, deterministic=True,
                                      compute_dtype=torch.float32)
            ref_w[i] = ref_w[i] * (1 - lr * wd) - lr * scale * o
            assert torch.allclose(moms[i], ref_m[i], atol=1e-6), step
            err = (masters[i] - ref_w[i]).abs().max().item()
            assert err < 0.1 * lr * scale * (step + 1), (step, err)
            ref_w[i] = masters[i].clone()        # compare each step on its own, not the accumulated drift


def test_newton_schulz_graph_replay_matches_eager(monkeypatch):
    """Stand-alone NS through the CUDA-graph cache: eager on the first call,
    captured on the second, replayed afterwards, same numbers as eager."""
    import dmuon_b200 as dmuon
    from dmuon_b200.optim import ns_graph

    dev = torch.device("cuda", 0)
    ns = dmuon.NewtonSchulz()
    torch.manual_seed(11)
    mats = [torch.randn(384, 1024, device=dev) for _ in range(4)]
    monkeypatch.setenv("DMUON_NS_CUDA_GRAPH", "0")
    eager = [ns.local(m, 5).clone() for m in mats]
    again = [ns.local(m, 5).clone() for m in mats]
    monkeypatch.setenv("DMUON_NS_CUDA_GRAPH", "1")
    ns_graph.cache().clear()
    base = ns_graph.cache().stats()
    got = [ns.local(m, 5).clone() for m in mats]
    torch.cuda.synchronize()
    st = ns_graph.cache().stats()
    assert st["failed"] == 0 and st["captures"] - base["captures"] == 1 and st["replays"] - base["replays"] == 3
    # The Frobenius norm is accumulated with atomics, so two runs of one input differ
    # in the last bit of the scale and the fp16 iteration amplifies that to a few
    # 1e-3; a replay that used a stale input or output would be off by about 1.4.
    # So: close to eager, no further from it than 2e-2, and just as orthogonal.
    eye = torch.eye(384, device=dev)
    for a, b, c in zip(got, eager, again):
        rel = ((a - b).norm() / b.norm()).item()
        spread = ((c - b).norm() / b.norm()).item()
        orth_a = ((a.float() @ a.float().T - eye).norm() / 384 ** 0.5).item()
        orth_b = ((b.float() @ b.float().T - eye).norm() / 384 ** 0.5).item()
        assert rel < 2e-2 and abs(orth_a - orth_b) < 0.01, (rel, spread, orth_a, orth_b)
    assert dmuon.get_backend_status()["cuda_graph_replay"] is True


@pytest.mark.parametrize("shape", [(512, 1536), (1536, 512)])
def test_gram_factors_on_kernels_reproduce_newton_schulz(shape):
    """The factor segments the tensor-parallel owner sends (computed on the
    tcgen05 GEMM) applied to column blocks of the matrix (again on the GEMM)
    give the same result as orthogonalising the whole matrix in fp32."""
    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import ns_sm100
    from dmuon_b200.optim.newton_schulz import (
        DEFAULT_COEFFICIENTS, DEFAULT_RESTART_ITERATIONS, apply_gram_factors, gram_newton_schulz_factors)

    dev = _dev()
    torch.manual_seed(5)
    U = torch.randn(*shape, device=dev)
    segs, transposed, norm = ns_sm100.gram_factors(U, DEFAULT_COEFFICIENTS, DEFAULT_RESTART_ITERATIONS)
    assert transposed == (shape[0] > shape[1]) and len(segs) == 2
    assert all(s.dtype == torch.float16 and s.shape == (512, 512) for s in segs)
    # fp32 PyTorch reference of the same schedule
    rsegs, rtr, rnorm = gram_newton_schulz_factors(U, compute_dtype=torch.float32, deterministic=True)
    assert rtr == transposed
    assert abs(float(norm) - float(rnorm)) < 1e-3 * float(rnorm)
    ref = apply_gram_factors(U, rsegs, rtr, rnorm)
    # apply to two halves along the dimension a tensor-parallel group would shard
    halves = U.chunk(2, dim=0 if transposed else 1)
    got = torch.cat([ns_sm100.apply_factors(h.contiguous(), segs, transposed, norm) for h in halves],
                    dim=0 if transposed else 1)
    torch.cuda.synchronize()
    G.check_status(dev)
    assert got.dtype == torch.float32 and got.shape == U.shape
    assert (got - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("shard_dim", [0, 1])
@pytest.mark.parametrize("cols", [256, 250])          # 250: narrow shards that are not a multiple of 8 wide
def test_tp_gather_prologue_and_apply_delta(shard_dim, cols):
    """The tensor-parallel kernels on one device (the shards of the "other
    ranks" are just other allocations): shards written into their place of the
    full matrix with momentum / Nesterov / cast / norm in the same pass, and the
    slice of a full update applied to a master shard."""
    from dmuon_b200.ops import tp_peer as TP

    dev = _dev()
    torch.manual_seed(13)
    T, rows, mu = 2, 192, 0.9
    full_g = (torch.randn(rows, cols, device=dev) * 1e-2).bfloat16()
    shards = [c.contiguous() for c in full_g.chunk(T, dim=shard_dim)]
    mom = torch.randn(rows, cols, device=dev) * 1e-2
    mom0 = mom.clone()
    x = torch.full((rows, cols), float("nan"), device=dev, dtype=torch.float16)
    sumsq = torch.zeros(2, device=dev)
    xscale = torch.tensor([1.0, 4.0], device=dev)
    jobs = []
    for t, s in enumerate(shards):
        r_off = t * s.shape[0] if shard_dim == 0 else 0
        c_off = t * s.shape[1] if shard_dim == 1 else 0
        jobs.append(TP.ShardJob(0, s.data_ptr(), s.shape[0], s.shape[1], r_off * cols + c_off, cols))
    TP.gather_prologue(jobs, torch.bfloat16, [mom], [x], [1], sumsq, mu=mu, nesterov=True, xscale=xscale)
    torch.cuda.synchronize()
    buf = mu * mom0 + full_g.float()
    u = full_g.float() + mu * buf
    assert torch.allclose(mom, buf, atol=1e-7)
    assert (x.float() - 4.0 * u).abs().max().item() < 2e-3 * (4.0 * u).abs().max().item()
    assert abs(float(sumsq[1]) - float((u * u).sum())) < 1e-3 * float((u * u).sum()) and float(sumsq[0]) == 0.0
    # scatter side: every "rank" applies its slice of the owner's full fp32 update to its master shard
    delta = torch.randn(rows, cols, device=dev) * 1e-3
    masters = [torch.randn_like(s, dtype=torch.float32) for s in shards]
    before = [m.clone() for m in masters]
    srcs = []
    for t, s in enumerate(shards):
        r_off = t * s.shape[0] if shard_dim == 0 else 0
        c_off = t * s.shape[1] if shard_dim == 1 else 0
        srcs.append(delta.data_ptr() + (r_off * cols + c_off) * 4)
    TP.apply_delta(srcs, [cols] * T, masters, [0.998] * T)
    torch.cuda.synchronize()
    for m, b, d in zip(masters, before, delta.chunk(T, dim=shard_dim)):
        assert torch.allclose(m, b * 0.998 + d, atol=1e-6)

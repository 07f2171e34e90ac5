"""Host-side logic without a process group: partition, policy, owner
coordinates, FSDP2 patch, Newton-Schulz math, clip semantics, symmetric tiles."""
import math

import pytest
import torch
import torch.nn as nn


class FakeMesh:
    def __init__(self, n, names=("dp",)):
        self._n, self.mesh_dim_names, self.ndim = n, names, 1

    def size(self):
        return self._n


class Layered(nn.Module):
    def __init__(self, n_layers=4, d=64, ffn=256):
        super().__init__()
        self.embed_tokens = nn.Embedding(100, d)
        self.layers = nn.ModuleList()
        for _ in range(n_layers):
            blk = nn.Module()
            blk.q_proj = nn.Linear(d, d, bias=False)
            blk.k_proj = nn.Linear(d, d // 4, bias=False)
            blk.v_proj = nn.Linear(d, d // 4, bias=False)
            blk.up_proj = nn.Linear(d, ffn, bias=False)
            blk.down_proj = nn.Linear(ffn, d, bias=False)
            blk.norm = nn.LayerNorm(d)
            self.layers.append(blk)


def _pred(n, p):
    return "proj" in n and p.ndim == 2


# ------------------------------------------------------------------ partition
def test_partition_is_balanced_deterministic_and_spreads_layers():
    from dmuon_b200.parallel.partition import compute_balanced_assignment, layer_key

    model = Layered()
    a = compute_balanced_assignment(model, FakeMesh(4), _pred)
    b = compute_balanced_assignment(model, FakeMesh(4), _pred)
    names = {p: n for n, p in model.named_parameters()}
    assert {names[p]: o for p, o in a.items()} == {names[p]: o for p, o in b.items()}
    assert all(isinstance(o, int) and 0 <= o < 4 for o in a.values())
    assert len(a) == 20
    # small same-layer parameters are packed: all five matrices of a layer are
    # below the threshold here, so each layer is one unit with one owner
    for i in range(4):
        owners = {a[p] for n, p in model.named_parameters() if n.startswith(f"layers.{i}.") and _pred(n, p)}
        assert len(owners) == 1
    assert a.packed_allocation_unit_count == 4
    assert sorted(set(a.values())) == [0, 1, 2, 3]
    assert layer_key("model.layers.3.mlp.up_proj.weight") == "model.layers.3"
    assert layer_key("visual.blocks.5.attn.qkv.weight") == "visual.blocks.5"
    assert layer_key("layers.2.x") == "_root.layers.2"
    assert layer_key("embed_tokens.weight") is None


def test_partition_unpacked_spreads_a_layer_over_owners_and_strategies():
    from dmuon_b200.parallel.partition import compute_balanced_assignment

    model = Layered()
    a = compute_balanced_assignment(model, FakeMesh(8), _pred, pack_small_params=False)
    for i in range(4):
        owners = [a[p] for n, p in model.named_parameters() if n.startswith(f"layers.{i}.") and _pred(n, p)]
        assert len(set(owners)) == 5          # same-layer rule: five matrices, five owners
    r0 = compute_balanced_assignment(model, FakeMesh(8), _pred, owner_strategy="rank0")
    assert set(r0.values()) == {0}
    rr = compute_balanced_assignment(model, FakeMesh(4), _pred, owner_strategy="round_robin", pack_small_params=False)
    assert [rr[p] for n, p in model.named_parameters() if _pred(n, p)][:5] == [0, 1, 2, 3, 0]
    capped = compute_balanced_assignment(model, FakeMesh(8), _pred, pack_small_params=False, max_owners_per_group=2)
    for i in range(4):
        owners = {capped[p] for n, p in model.named_parameters() if n.startswith(f"layers.{i}.") and _pred(n, p)}
        assert len(owners) <= 2
    with pytest.raises(ValueError):
        compute_balanced_assignment(model, FakeMesh(4), _pred, owner_strategy="nope")


def test_partition_hsdp_returns_coords_and_balances_columns():
    from dmuon_b200.parallel.partition import compute_balanced_assignment

    model = Layered(n_layers=8)
    a = compute_balanced_assignment(model, FakeMesh(2, ("shard",)), _pred, replicate_mesh=FakeMesh(2, ("replicate",)),
                                    pack_small_params=False)
    assert all(isinstance(o, tuple) and len(o) == 2 for o in a.values())
    col = [0, 0]
    for p, (s, r) in a.items():
        col[s] += p.numel()
    assert abs(col[0] - col[1]) / max(col) < 0.1
    assert {o for o in a.values()} == {(0, 0), (0, 1), (1, 0), (1, 1)}


def test_cost_model_orders_by_newton_schulz_work():
    from dmuon_b200.parallel.partition import optimizer_cost_units

    big = optimizer_cost_units("layers.0.mlp.down_proj.weight", (4096, 14336), 4096 * 14336)
    sq = optimizer_cost_units("layers.0.self_attn.q_proj.weight", (4096, 4096), 4096 * 4096)
    kv = optimizer_cost_units("layers.0.self_attn.k_proj.weight", (1024, 4096), 1024 * 4096)
    emb = optimizer_cost_units("embed_tokens.weight", (128256, 4096), 128256 * 4096)
    assert big > sq > kv
    assert emb == 128256 * 4096 // 1_000_000       # AdamW-routed by name: bytes only


# ------------------------------------------------------------------ owner coords / policy
def test_normalize_owner_rank():
    from dmuon_b200.parallel.topology import normalize_owner_rank

    assert normalize_owner_rank(3) == (3, 0)
    assert normalize_owner_rank((1, 2)) == (1, 2)
    for bad in (True, (1, True), (1,), (1, 2, 3), "1", 1.5):
        with pytest.raises((TypeError, ValueError)):
            normalize_owner_rank(bad)
    with pytest.raises(ValueError):
        normalize_owner_rank(-1)


def test_param_policy_resolution_order_and_validation():
    from dmuon_b200.policy import DMuonParamPolicy, resolve_param_policies

    model = Layered(n_layers=1)
    params = [p for n, p in model.named_parameters()]
    fqn = {p: n for n, p in model.named_parameters()}
    pol = resolve_param_policies(
        params=params, param_to_fqn=fqn,
        param_policy={
            "defaults": {"param_dtype": "bf16", "grad_dtype": "fp32"},
            "overrides": [
                {"contains": ["embed", "norm"], "set": {"route": "base", "param_dtype": None}},
                {"name": "embed", "set": {"route": "sharded"}},
            ],
        },
    )
    emb = pol[model.embed_tokens.weight]
    q = pol[model.layers[0].q_proj.weight]
    assert emb.route == "sharded_adamw" and emb.param_dtype is None and emb.matched_overrides == (0, 1)
    assert q.route is None and q.param_dtype == torch.bfloat16 and q.grad_dtype == torch.float32
    assert q.master_dtype == torch.float32 and q.optim_dtype == torch.float32
    fn = resolve_param_policies(params=params, param_to_fqn=fqn, compute_dtype=torch.bfloat16,
                                param_policy_fn=lambda n, p: {"route": "adamw"} if p.ndim < 2 else DMuonParamPolicy(route="muon"))
    assert fn[model.layers[0].norm.weight].route == "adamw"
    assert fn[model.layers[0].norm.weight].param_dtype == torch.bfloat16
    assert fn[model.layers[0].q_proj.weight].param_dtype is None     # a full policy object replaces the base
    with pytest.raises(ValueError):
        resolve_param_policies(params=params, param_to_fqn=fqn, param_policy={"defaults": {"bogus": 1}})
    with pytest.raises(ValueError):
        resolve_param_policies(params=params, param_to_fqn=fqn, param_policy={}, param_policy_fn=lambda n, p: None)
    with pytest.raises(ValueError):
        resolve_param_policies(params=params, param_to_fqn=fqn, route_hint_fn=lambda n, p: "x")
    legacy = resolve_param_policies(params=params, param_to_fqn=fqn, route_hint_fn=lambda n, p: "matrix_optimizer")
    assert all(v.route == "muon" for v in legacy.values())


# ------------------------------------------------------------------ FSDP2 patch
def test_fsdp_patch_filters_tagged_params_and_can_be_removed():
    from torch.distributed.fsdp._fully_shard import _fsdp_init

    import dmuon_b200
    from dmuon_b200.parallel import fsdp_patch

    assert fsdp_patch.is_installed()
    m = nn.Linear(4, 4)
    m.weight._dedicated_owner_rank = 0
    params, _ = _fsdp_init._get_managed_states([m])
    assert [id(p) for p in params] == [id(m.bias)]
    params, _ = _fsdp_init._get_managed_states([m], set())
    assert len(params) == 1
    fsdp_patch.uninstall_patch()
    assert not fsdp_patch.is_installed()
    assert len(_fsdp_init._get_managed_states([m])[0]) == 2
    assert dmuon_b200.install_patch() and fsdp_patch.is_installed()
    assert dmuon_b200.install_patch()          # idempotent


# ------------------------------------------------------------------ Newton-Schulz math
def _orth_err(O):
    X = O if O.shape[0] <= O.shape[1] else O.T
    return (X @ X.T - torch.eye(X.shape[0])).abs().max().item()


@pytest.mark.parametrize("shape", [(32, 96), (96, 32), (64, 64)])
def test_newton_schulz_orthogonalises_and_formulations_agree(shape):
    from dmuon_b200.optim import newton_schulz as NS

    torch.manual_seed(0)
    G = torch.randn(shape)
    gram = NS.gram_newton_schulz(G)
    direct = NS.direct_newton_schulz(G)
    assert _orth_err(gram) < 0.15 and _orth_err(direct) < 0.15
    assert (gram - direct).abs().max().item() < 1e-4       # same polynomial up to fp32 rounding
    assert torch.allclose(NS.gram_newton_schulz(G.T.contiguous()), gram.T, atol=1e-5)
    U, _, Vh = torch.linalg.svd(G, full_matrices=False)
    assert (gram - U @ Vh).abs().max().item() < 0.15
    segs, transposed, norm = NS.gram_newton_schulz_factors(G)
    assert len(segs) == 2 and transposed == (shape[0] > shape[1])
    assert torch.allclose(NS.apply_gram_factors(G, segs, transposed, norm), gram, atol=1e-5)
    no_restart = NS.gram_newton_schulz(G, restart_iterations=[])
    assert (no_restart - gram).abs().max().item() < 1e-4


def test_newton_schulz_config_object():
    from dmuon_b200.optim import newton_schulz as NS

    ns = NS.NewtonSchulz()
    assert ns.backend == "gram" and ns.resolved_restarts() == [2] and len(ns.resolved_coefficients(5)) == 5
    assert NS.NewtonSchulz("direct").resolved_restarts() == []
    assert NS.NewtonSchulz(kernel="cublas").deterministic
    assert NS.NewtonSchulz(kernel="quack").kernel == "tcgen05"
    with pytest.raises(ValueError):
        NS.NewtonSchulz(backend="x")
    with pytest.raises(ValueError):
        NS.NewtonSchulz(kernel="x")
    assert NS.get_ns_backend() in ("torch", "tcgen05")
    assert NS.get_backend_status()["arch"] == "sm_100a"
    a, b, c = NS.POLAR_EXPRESS_COEFFICIENTS[0]
    assert abs(a - 7.8926) < 1e-3 and abs(b + 20.383) < 1e-2 and abs(c - 13.555) < 1e-2


# ------------------------------------------------------------------ tiles
def test_symmetric_tile_lists_cover_every_element_exactly_once():
    from dmuon_b200.ops.gemm import symmetric_tiles

    for m, bn in [(512, 128), (1024, 256), (1152, 256), (200, 128), (384, 256)]:
        cover = torch.zeros(m, m, dtype=torch.int32)
        for i, j, mirror in symmetric_tiles(m, bn):
            r0, r1 = i * 128, min(m, i * 128 + 128)
            c0, c1 = j * bn, min(m, j * bn + bn)
            cover[r0:r1, c0:c1] += 1
            if mirror:
                cover[c0:c1, r0:r1] += 1
        assert int(cover.min()) == 1 and int(cover.max()) == 1, (m, bn)


# ------------------------------------------------------------------ clip
def test_bucket_clip_semantics_on_cpu():
    from dmuon_b200.fast_clip import GradClipBucket, clip_grad_norm_buckets_

    torch.manual_seed(1)
    a = [torch.randn(10), torch.randn(3, 4)]
    b = [torch.randn(7) * 1e-3]
    na = math.sqrt(sum(float(t.pow(2).sum()) for t in a))
    nb = float(b[0].norm())
    before_b = b[0].clone()
    res = clip_grad_norm_buckets_([GradClipBucket("big", a), GradClipBucket("small", b, reduce=False)], 1.0)
    st = res.stats_by_name
    assert abs(float(st["big"].total_norm) - na) < 1e-5 and abs(float(st["small"].total_norm) - nb) < 1e-8
    assert bool(st["big"].clipped) and not bool(st["small"].clipped)
    assert abs(math.sqrt(sum(float(t.pow(2).sum()) for t in a)) - 1.0) < 1e-4
    assert torch.equal(b[0], before_b)
    assert not res.fastpath and res.fallback_reason
    # stats-only and non-finite
    g = [torch.tensor([float("inf"), 1.0])]
    r2 = clip_grad_norm_buckets_([GradClipBucket("x", g)], None)
    assert bool(r2.bucket_stats[0].found_inf) and not bool(r2.bucket_stats[0].clipped)
    r3 = clip_grad_norm_buckets_([GradClipBucket("x", g)], 1.0)
    assert bool(r3.bucket_stats[0].found_inf) and not bool(r3.bucket_stats[0].clipped)


@pytest.mark.parametrize("m,n,sym", [(4096, 4096, True), (1152, 1152, True), (256, 256, True), (768, 1792, False),
                                     (4096, 14336, False), (300, 700, False), (2048, 2048, True)])
def test_quad_tile_list_covers_the_pair_tile_list_exactly(m, n, sym):
    """The two-tiles-per-entry list of the CTA-quad GEMM names every 256 x 256
    tile of the CTA-pair list exactly once, with the same mirror flags; entries
    marked as sharing rows do share them; at most one filler."""
    from dmuon_b200.ops import gemm as G

    want = G.symmetric_tiles(m, 256, 256) if sym else G.dense_tiles(m, n, 256, 256)
    got, fillers = [], 0
    for x, y, z, _ in G.quad_tile_list(m, n, sym):
        m0, m1, n0, n1 = x & 0xFFFF, x >> 16, y & 0xFFFF, y >> 16
        got.append((m0, n0, z & 1))
        if z & 8:
            fillers += 1
            assert (m1, n1) == (m0, n0) and not z & 4
        else:
            got.append((m1, n1, (z >> 1) & 1))
        if z & 4:
            assert m0 == m1 and n0 != n1
    assert fillers <= 1
    assert sorted(got) == sorted(want)


@pytest.mark.parametrize("shape", [(64, 128), (128, 64), (96, 96), (32, 256)])
@pytest.mark.parametrize("formulation", ["gram", "direct"])
def test_newton_schulz_against_svd_polar_factor_and_textbook_iteration(shape, formulation):
    """Pins the specification with two things the package did not write: the
    polar factor ``U V^T`` from an SVD (Newton-Schulz must share its singular
    vectors and push every singular value near 1) and a float64 textbook
    quintic iteration on the matrix itself (``tests/oracle.py``)."""
    from oracle import newton_schulz_reference

    from dmuon_b200.optim.newton_schulz import direct_newton_schulz, gram_newton_schulz

    torch.manual_seed(3)
    G = torch.randn(*shape)
    O = gram_newton_schulz(G) if formulation == "gram" else direct_newton_schulz(
        G, steps=5, compute_dtype=torch.float32)
    U, S, Vh = torch.linalg.svd(G.double(), full_matrices=False)
    core = U.T @ O.double() @ Vh.T              # diagonal iff O = U f(S) V^T
    diag = torch.diag(core)
    off = core - torch.diag(diag)
    assert off.abs().max().item() < 1e-4
    assert -1e-4 < diag.min().item() and diag.max().item() < 1.25      # singular values only move towards 1
    if shape[0] != shape[1]:
        # a rectangular Gaussian matrix is well conditioned: five steps bring every singular value near 1
        # (a square one has singular values near 0, which five steps cannot lift)
        assert diag.min().item() > 0.5
        small = O if shape[0] < shape[1] else O.T
        assert (small @ small.T - torch.eye(small.shape[0])).abs().max().item() < 0.3
    assert (O - newton_schulz_reference(G)).abs().max().item() < 2e-5


def test_ns_kernel_environment_variable_applies_only_to_auto(monkeypatch):
    """``DMUON_NS_KERNEL`` picks the implementation when the argument says
    "auto" and loses against an explicit argument; the reference's backend
    names are accepted, unknown names are rejected."""
    import dmuon_b200 as dmuon

    monkeypatch.delenv("DMUON_NS_KERNEL", raising=False)
    assert dmuon.NewtonSchulz().kernel == "tcgen05"
    monkeypatch.setenv("DMUON_NS_KERNEL", "cublas")
    assert dmuon.NewtonSchulz().kernel == "torch" and dmuon.NewtonSchulz().deterministic
    assert dmuon.NewtonSchulz(kernel="tcgen05").kernel == "tcgen05"
    monkeypatch.setenv("DMUON_NS_KERNEL", "quack")
    assert dmuon.NewtonSchulz().kernel == "tcgen05"
    monkeypatch.setenv("DMUON_NS_KERNEL", "nonsense")
    with pytest.raises(ValueError):
        dmuon.NewtonSchulz()


def test_old_partition_import_path_forwards_to_the_real_module():
    import dmuon_b200.partition as shim
    from dmuon_b200.parallel import partition as real
    from dmuon_b200.partition import SMALL_PARAM_THRESHOLD, AssignmentResult, compute_balanced_assignment

    assert compute_balanced_assignment is real.compute_balanced_assignment
    assert AssignmentResult is real.AssignmentResult and SMALL_PARAM_THRESHOLD == real.SMALL_PARAM_THRESHOLD
    assert "optimizer_cost_units" in dir(shim) and shim.optimizer_cost_units is real.optimizer_cost_units
    with pytest.raises(AttributeError):
        shim.no_such_name

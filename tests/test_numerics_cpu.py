"""Newton-Schulz properties, the sharded (all-reduce-Gram) iteration on gloo,
storage helpers and the CPU side of the CUDA-graph cache."""
import math

import pytest
import torch

from dist_utils import run_ranks


def _orth_err(U):
    m = min(U.shape)
    G = U @ U.T if U.shape[0] <= U.shape[1] else U.T @ U
    return ((G - torch.eye(m)).norm() / math.sqrt(m)).item()


@pytest.mark.parametrize("shape", [(48, 160), (160, 48), (64, 64)])
def test_factor_segments_reproduce_the_iteration(shape):
    from dmuon_b200.optim.newton_schulz import apply_gram_factors, gram_newton_schulz, gram_newton_schulz_factors

    torch.manual_seed(0)
    G = torch.randn(shape)
    full = gram_newton_schulz(G)
    segs, transposed, norm = gram_newton_schulz_factors(G)
    assert transposed == (shape[0] > shape[1]) and len(segs) == 2          # default restart at step 2 -> two windows
    again = apply_gram_factors(G, segs, transposed, norm)
    assert (again - full).abs().max().item() < 1e-5
    # column shards of the oriented matrix can be processed independently with the same factors
    Go = G.T if transposed else G
    halves = Go.chunk(2, dim=1)
    parts = [apply_gram_factors(h.T if transposed else h, segs, transposed, norm) for h in halves]
    glued = torch.cat(parts, dim=0 if transposed else 1)
    assert (glued - full).abs().max().item() < 1e-5


def test_tall_equals_transposed_wide_and_result_is_nearly_orthogonal():
    from dmuon_b200.optim.newton_schulz import direct_newton_schulz, gram_newton_schulz

    torch.manual_seed(1)
    G = torch.randn(40, 120)
    U = gram_newton_schulz(G)
    assert (gram_newton_schulz(G.T.contiguous()) - U.T).abs().max().item() < 1e-5
    assert (U @ U.T - torch.eye(40)).abs().max().item() < 0.15
    assert (direct_newton_schulz(G) - U).abs().max().item() < 0.1
    assert _orth_err(U) < 0.25


def test_restart_schedule_and_coefficient_tables():
    import dmuon_b200 as dmuon
    from dmuon_b200.optim.newton_schulz import CLASSIC_COEFFICIENTS, gram_newton_schulz

    torch.manual_seed(2)
    G = torch.randn(32, 96)
    base = gram_newton_schulz(G, restart_iterations=[])
    for restarts in ([2], [1, 3], [0, 2]):          # a restart only re-anchors the recurrence; 0 is ignored
        assert (gram_newton_schulz(G, restart_iterations=restarts) - base).abs().max().item() < 1e-4
    assert len(dmuon.POLAR_EXPRESS_COEFFICIENTS) == 5 and len(dmuon.YOU_COEFFICIENTS) == 5
    a, b, c = dmuon.POLAR_EXPRESS_COEFFICIENTS[0]
    assert abs(a - 8.28721201814563 / 1.05) < 1e-12 and abs(b + 23.595886519098837 / 1.05**3) < 1e-12
    assert _orth_err(gram_newton_schulz(G, coefficients=dmuon.YOU_COEFFICIENTS)) < 0.35
    assert _orth_err(gram_newton_schulz(G, coefficients=CLASSIC_COEFFICIENTS)) < 0.45


def _sharded_body(rank, world, transposed):
    import torch.distributed as dist

    from dmuon_b200.optim.newton_schulz import (
        gram_newton_schulz,
        gram_newton_schulz_distributed_local,
        gram_newton_schulz_distributed_local_batched,
    )

    torch.manual_seed(3)
    full = torch.randn(96, 24) if transposed else torch.randn(24, 96)
    ref = gram_newton_schulz(full)
    # shard along the long side: columns of the oriented (wide) matrix
    piece = full.chunk(world, dim=0 if transposed else 1)[rank].contiguous()
    out = gram_newton_schulz_distributed_local(piece, dist.group.WORLD, transposed=transposed)
    want = ref.chunk(world, dim=0 if transposed else 1)[rank]
    err1 = (out - want).abs().max().item()
    both = gram_newton_schulz_distributed_local_batched(torch.stack((piece, 2 * piece)), dist.group.WORLD, transposed=transposed)
    err2 = max((both[0] - want).abs().max().item(), (both[1] - want).abs().max().item())   # scale invariance
    return err1, err2


@pytest.mark.parametrize("transposed", [False, True])
def test_sharded_gram_iteration_equals_full_matrix_iteration(transposed):
    for err1, err2 in run_ranks(_sharded_body, 2, args=(transposed,)):
        assert err1 < 1e-4 and err2 < 1e-4


def test_storage_helpers_keep_views_alive_across_resize():
    from dmuon_b200.parallel.dparam import alloc_storage, free_storage

    buf = torch.arange(12, dtype=torch.float32)
    view = buf[4:10].view(2, 3)
    free_storage(buf)
    assert buf.untyped_storage().size() == 0 and view.shape == (2, 3)
    free_storage(buf)                                # idempotent
    alloc_storage(buf)
    alloc_storage(buf)
    assert buf.untyped_storage().size() == 48
    buf.copy_(torch.arange(12, dtype=torch.float32) * 2)
    assert torch.equal(view, torch.tensor([[8.0, 10.0, 12.0], [14.0, 16.0, 18.0]]))   # same storage object
    # the publish cast is a plain round-to-nearest-even copy, bit-identical to .to(bf16)
    src = [torch.randn(5, 7), torch.randn(3)]
    dst = [torch.empty(5, 7, dtype=torch.bfloat16), torch.empty(3, dtype=torch.bfloat16)]
    torch._foreach_copy_(dst, src)
    assert all(torch.equal(d, s.to(torch.bfloat16)) for d, s in zip(dst, src))


def test_graph_cache_is_transparent_on_cpu_and_counts_calls(monkeypatch):
    from dmuon_b200.optim import ns_graph

    c = ns_graph.NSGraphCache()
    calls = []

    def fn(x):
        calls.append(1)
        return x * 2

    x = torch.ones(3)
    for _ in range(3):
        assert torch.equal(c.run("k", fn, x), x * 2)
    assert len(calls) == 3 and c.stats() == {"keys": 1, "captures": 0, "replays": 0, "failed": 0}
    monkeypatch.delenv("DMUON_NS_CUDA_GRAPH", raising=False)
    assert ns_graph.enabled() is False
    monkeypatch.setenv("DMUON_NS_CUDA_GRAPH", "1")
    assert ns_graph.enabled() is True


def test_precision_study_runs_and_metrics_behave():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "ns_precision.py")
    spec = importlib.util.spec_from_file_location("ns_precision", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    G, nuclear = mod.make_matrix("uniform", 16, 48, seed=1)
    assert abs(nuclear - float(torch.linalg.svdvals(G.double()).sum())) < 1e-3 * nuclear     # the construction's spectrum
    Uo, _, Vh = torch.linalg.svd(G.double(), full_matrices=False)
    exact = mod.metrics((Uo @ Vh).float(), G, nuclear)                                      # the true polar factor
    assert exact["orth_err"] < 1e-5 and exact["sym_err"] < 1e-5 and abs(exact["dual_gap"]) < 1e-5
    rows = mod.run([(16, 48)], ["polar"], ["flat", "spike"], torch.device("cpu"))
    assert [r["variant"] for r in rows] == ["fp32", "fp32"] and all(r["vs_fp32"] == 0.0 for r in rows)
    assert all(r["orth_err"] < 0.35 and r["sym_err"] < 1e-3 and r["psd_violation"] < 1e-3 for r in rows)

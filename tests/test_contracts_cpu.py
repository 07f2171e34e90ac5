"""Host-side contracts pinned with fakes (no process group): the TP
distributed-Gram selection rule, clip strategies, diagnostics shape."""
from types import SimpleNamespace

import pytest
import torch

from dist_utils import run_ranks


def _fake_muon(backend="gram", policy="beneficial", ratio=0.5, restarts=(2,)):
    from dmuon_b200.optim.muon import Muon
    from dmuon_b200.optim.newton_schulz import NewtonSchulz

    ns = NewtonSchulz(backend=backend, restart_iterations=list(restarts), kernel="torch")
    fake = SimpleNamespace(
        ns=ns, ns_steps=5, tp_distributed_gram_policy=policy, tp_distributed_gram_max_factor_to_scatter_ratio=ratio,
    )
    fake._tp_gram_segment_count = lambda: Muon._tp_gram_segment_count(fake)
    return fake, Muon._tp_gram_rejection_reason


def _fake_dp(shape, shard_dim, tp=True, esize=4):
    return SimpleNamespace(
        tp_group=object() if tp else None, shard_dim=shard_dim, full_shape=torch.Size(shape),
        _owned_data=SimpleNamespace(element_size=lambda: esize),
    )


def test_tp_distributed_gram_selection_rule():
    fake, reason = _fake_muon()
    # wide matrix sharded by columns, tall matrix sharded by rows: the factors multiply from the left
    assert reason(fake, _fake_dp((1024, 8192), 1)) is None
    assert reason(fake, _fake_dp((8192, 1024), 0)) is None
    # the other orientations would need the factor on the sharded side
    assert reason(fake, _fake_dp((1024, 8192), 0)) == "unsupported_orientation"
    assert reason(fake, _fake_dp((8192, 1024), 1)) == "unsupported_orientation"
    assert reason(fake, _fake_dp((1024, 8192), 1, tp=False)) == "non_tp_param"
    assert reason(fake, _fake_dp((8192,), 0)) == "not_matrix"
    # two segments of 4096^2 fp16 against a 4096 x 4096 fp32 update: 2*2/4 = 1.0 -> not smaller
    assert reason(fake, _fake_dp((4096, 4096), 1)) == "factor_not_smaller"
    # 4096 x 14336 fp32: factors are 2*4096^2*2 / (4096*14336*4) = 0.286 of the update
    assert reason(fake, _fake_dp((4096, 14336), 1)) is None
    tight, reason2 = _fake_muon(ratio=0.25)
    assert reason2(tight, _fake_dp((4096, 14336), 1)) == "factor_ratio_too_high"
    off, reason3 = _fake_muon(policy="off")
    assert reason3(off, _fake_dp((1024, 8192), 1)) == "policy_disabled"
    force, reason4 = _fake_muon(policy="all")
    assert reason4(force, _fake_dp((4096, 4096), 1)) is None
    direct, reason5 = _fake_muon(backend="direct")
    assert reason5(direct, _fake_dp((1024, 8192), 1)) == "non_gram_backend"
    # one more restart window -> one more factor segment on the wire
    three, _ = _fake_muon(restarts=(2, 4))
    assert three._tp_gram_segment_count() == 3 and fake._tp_gram_segment_count() == 2


class _FakeOpt:
    """Just enough of Muon for the clip entry points."""

    def __init__(self, grads):
        self._grads = grads
        self._last_clip_stats = None
        self.device = torch.device("cpu")

    def _ensure_grads_ready(self, materialize=False):
        self.materialized = materialize

    def owned_muon_params(self):
        return [
            SimpleNamespace(fqn=f"w{i}", param_name=f"w{i}", _reduced_grad=g, _tp_full_grad=None, tp_group=None,
                            is_tp_owner=False, full_shape=g.shape, _orig_size=g.shape, _dmuon_route="muon")
            for i, g in enumerate(self._grads)
        ]


def test_clip_measures_scales_and_accepts_custom_strategies():
    import dmuon_b200 as dmuon
    from dmuon_b200 import grad_clip

    g = [torch.full((4, 4), 3.0), torch.full((2, 8), 4.0)]
    opt = _FakeOpt(g)
    ref = float(torch.cat([x.flatten() for x in g]).norm())
    stats = dmuon.clip_grad_norm_(opt, None)
    assert abs(float(stats.total_norm) - ref) < 1e-5 and not bool(stats.clipped) and opt.materialized
    assert float(g[0][0, 0]) == 3.0                                   # measuring never scales
    stats = dmuon.clip_grad_norm_(opt, ref / 4)
    assert bool(stats.clipped) and abs(float(stats.clip_coef) - 0.25) < 1e-4
    assert abs(float(g[0][0, 0]) - 0.75) < 1e-4 and stats.param_count == 2
    stats_inf = dmuon.clip_grad_norm_(opt, None, norm_type=float("inf"))
    assert abs(float(stats_inf.total_norm) - 1.0) < 1e-4
    seen = {}

    def halve(ctx):
        seen["names"] = [e.name for e in ctx.entries]
        for e in ctx.entries:
            e.grad.mul_(0.5)
        return grad_clip.MuonGradClipStats(
            total_norm=torch.tensor(0.0), max_norm=ctx.max_norm, norm_type=ctx.norm_type, clip_coef=0.5,
            clipped=True, param_count=len(ctx.entries), found_inf=torch.tensor(False), strategy="halve",
        )

    dmuon.register_muon_grad_clip_strategy("halve", halve)
    out = dmuon.clip_grad_norm_(opt, 1.0, strategy="halve")
    assert out.strategy == "halve" and seen["names"] == ["w0", "w1"] and opt._last_clip_stats is out
    assert abs(float(g[0][0, 0]) - 0.375) < 1e-4
    with pytest.raises(ValueError):
        dmuon.clip_grad_norm_(opt, 1.0, strategy="no-such-strategy")
    with pytest.raises(TypeError):
        dmuon.clip_grad_norm_(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1), 1.0)


def test_bucket_clip_handles_non_contiguous_and_non_finite_gradients():
    import dmuon_b200 as dmuon

    base = torch.arange(24, dtype=torch.float32).reshape(4, 6)
    strided = base.t()                                                # non-contiguous view
    other = torch.ones(5)
    res = dmuon.clip_grad_norm_buckets_(
        [dmuon.GradClipBucket("a", [strided], reduce=False), dmuon.GradClipBucket("b", [other], reduce=False)], 1.0
    )
    sa, sb = res.stats_by_name["a"], res.stats_by_name["b"]
    assert abs(float(base.norm()) - 1.0) < 1e-3 and bool(sa.clipped)          # scaled through the view
    assert abs(float(other.norm()) - 1.0) < 1e-3 and bool(sb.clipped)
    bad = torch.tensor([1.0, float("nan")])
    fine = torch.tensor([3.0, 4.0])
    res = dmuon.clip_grad_norm_buckets_(
        [dmuon.GradClipBucket("bad", [bad], reduce=False), dmuon.GradClipBucket("fine", [fine], reduce=False)], 10.0
    )
    assert bool(res.stats_by_name["bad"].found_inf) and not bool(res.stats_by_name["fine"].found_inf)
    assert not bool(res.stats_by_name["fine"].clipped) and float(fine[1]) == 4.0


def _diag_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import _build_model, _pred

    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
    model = _build_model()
    dmuon.dedicate_params(model, mesh["shard"], _pred, replicate_mesh=mesh["replicate"])
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, first_step_progress_log=False)
    pg = dmuon.summarize_param_groups(model, opt, max_rows=5)
    assert pg == dmuon.summarize_param_groups(opt, max_rows=5)            # single-argument form
    plan = dmuon.summarize_comm_plan(model, max_groups=2, max_params_per_group=3)
    owned_here = dmuon.get_owned_params(model)
    coord = (mesh["shard"].get_local_rank(), mesh["replicate"].get_local_rank())
    by_coord = dmuon.get_owned_params(model, coord)
    ctx = dmuon.get_comm_ctx(model)
    ctx.record_forward_unshard_counter("g", prefetch_hits=2)
    prof_keep = ctx.consume_forward_unshard_profile(clear=False)
    prof = dmuon.collect_forward_unshard_profile(model, clear=True, synchronize=False)
    dmuon.prepare_muon_grads(model, use_reduce_stream=False, coalesce_wait=False)
    import json

    json.dumps(pg), json.dumps(plan)                                       # JSON-friendly
    return pg, plan, [p.fqn for p in owned_here], [p.fqn for p in by_coord], prof_keep, prof, \
        len(list(dmuon.utils.iter_dedicated_states(model)))


def test_diagnostics_carry_the_reference_schema_and_signatures():
    """Code written against the reference's diagnostics keeps working: call
    forms, top-level keys, per-group and per-parameter keys, totals."""
    res = run_ranks(_diag_body, 4)
    pg, plan, owned_here, by_coord, prof_keep, prof, n_states = res[0]
    assert pg["available"] and pg["num_groups"] == 2 and pg["dedicated_param_count"] == 28
    assert len(pg["parameters"]) == 5 and pg["parameters_truncated"] == 23
    assert sum(r[0]["owned_dedicated_param_count"] for r in res) == 28      # every matrix has exactly one owner
    for key in ("group_index", "group_name", "semantic_group_name", "subgroup_type", "use_muon", "optimizer_param_count",
                "dedicated_param_count", "owned_dedicated_param_count", "dedicated_muon_param_count",
                "dedicated_adamw_param_count", "adamw_param_count", "route_param_counts"):
        assert key in pg["groups"][0], key
    for key in ("name", "param_name", "route", "param_dtype", "grad_dtype", "output_dtype", "master_dtype", "optim_dtype",
                "cast_forward_inputs", "matched_policy_overrides", "group_index", "group_name", "owner_rank", "is_owner",
                "is_dtensor", "uses_sharded_adamw", "numel", "shape"):
        assert key in pg["parameters"][0], key
    assert plan["available"] and plan["group_count"] == n_states == 4 and len(plan["groups"]) == 2 and plan["groups_truncated"] == 2
    g0 = plan["groups"][0]
    for key in ("group_index", "debug_name", "shard_rank", "replicate_rank", "param_count", "owner_bucket_count",
                "owner_bucket_bytes", "owner_bucket_bytes_in_order", "owner_buckets", "param_collectives",
                "param_collectives_truncated"):
        assert key in g0, key
    assert len(g0["param_collectives"]) == 3 and g0["param_collectives_truncated"] == g0["param_count"] - 3
    for key in ("param_index", "param_name", "owner_coord", "bytes", "route", "stage1_shard_reduce_root_global_rank",
                "stage2_replicate_axis_active_on_this_rank", "stage2_replicate_reduce_root_global_rank",
                "post_step_replicate_broadcast_root_global_rank"):
        assert key in g0["param_collectives"][0], key
    assert sum(g0["owner_bucket_bytes"]) == sum(b["bytes"] for b in g0["owner_buckets"])
    t = plan["totals"]
    for key in ("dedicated_local_bytes", "stage1_shard_reduce_tensor_bytes", "stage1_shard_reduce_ring_bytes_per_rank",
                "stage2_replicate_reduce_tensor_bytes_this_rank", "post_step_replicate_broadcast_tensor_bytes_this_rank",
                "owner_update_ring_bytes_per_rank", "same_payload_allreduce_ring_bytes_per_rank", "max_owner_bucket_bytes"):
        assert key in t, key
    # 28 fp32 matrices of the tiny decoder: 4 layers x (4 x 256x256 + 3 x 256x1024) x 4 bytes
    assert t["dedicated_local_bytes"] == 4 * (4 * 256 * 256 + 3 * 256 * 1024) * 4
    assert t["stage1_shard_reduce_ring_bytes_per_rank"] == t["dedicated_local_bytes"]      # 2 * (2 - 1) / 2
    # the replicate axis is active for the matrices whose owner column this rank sits in: both columns together cover all
    assert res[0][1]["totals"]["stage2_replicate_reduce_tensor_bytes_this_rank"] + \
        res[1][1]["totals"]["stage2_replicate_reduce_tensor_bytes_this_rank"] == t["dedicated_local_bytes"]
    assert owned_here == by_coord
    assert prof_keep["g"]["prefetch_hits"] == 2 and prof["g"]["prefetch_hits"] == 2

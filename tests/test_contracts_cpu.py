"""Host-side contracts pinned with fakes (no process group): the TP
distributed-Gram selection rule, clip strategies, diagnostics shape."""
from types import SimpleNamespace

import pytest
import torch


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

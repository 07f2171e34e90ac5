"""dmuon_b200 -- dedicated-ownership Muon for 8 x B200.

Every selected matrix parameter gets ONE owner rank.  The owner keeps the
fp32 master weights and the optimizer state and runs momentum + Newton-Schulz
for it; everybody else receives a published bf16 copy for forward/backward and
sends gradients back.  The remaining parameters stay with FSDP2 (or are
replicated) and get AdamW.

Typical use (``import dmuon_b200 as dmuon``)::

    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3)

Importing the package patches FSDP2 so ``fully_shard`` ignores dedicated
parameters.  The public names are those of the reference package
(dmuon/__init__.py:80-122).
"""
from __future__ import annotations

__version__ = "0.1.0"

from .parallel.fsdp_patch import install_patch, uninstall_patch

install_patch()

from .api import dedicate_params, dedicate_params_ddp, dedicate_params_ddp_tp  # noqa: E402
from .checkpoint import (  # noqa: E402
    get_model_state_dict,
    get_optimizer_state_dict,
    set_model_state_dict,
    set_optimizer_state_dict,
)
from .diagnostics import summarize_comm_plan, summarize_param_groups  # noqa: E402
from .fast_clip import (  # noqa: E402
    GradClipBucket,
    GradClipBucketStats,
    SegmentedGradClipResult,
    clip_grad_norm_buckets_,
    try_clip_optimizer_grad_norm_buckets_,
)
from .grad_clip import MuonGradClipStats, clip_grad_norm_, register_muon_grad_clip_strategy  # noqa: E402
from .optim.muon import Muon  # noqa: E402
from .optim.newton_schulz import (  # noqa: E402
    CLASSIC_COEFFICIENTS,
    POLAR_EXPRESS_COEFFICIENTS,
    YOU_COEFFICIENTS,
    NewtonSchulz,
    direct_newton_schulz,
    get_backend_status,
    get_ns_backend,
    gram_newton_schulz,
    gram_newton_schulz_factors,
    newton_schulz,
)
from .parallel.comm import DedicatedCommContext  # noqa: E402
from .parallel.ddp import replicate, replicate_tp  # noqa: E402
from .parallel.dgroup import DedicatedParamGroup, DedicatedParamGroupDDP  # noqa: E402
from .parallel.dparam import DedicatedParam, DedicatedParamDDP  # noqa: E402
from .parallel.partition import compute_balanced_assignment  # noqa: E402
from .policy import DMuonParamPolicy, resolve_param_policies  # noqa: E402
from .utils import (  # noqa: E402
    broadcast_all_updates,
    broadcast_all_updates_async,
    collect_forward_unshard_profile,
    get_comm_ctx,
    get_dedicated_params,
    get_owned_params,
    no_sync,
    prepare_muon_grads,
    wait_all_post_step_broadcasts,
    wait_all_reduces,
    wait_all_replicate_broadcasts,
)

__all__ = [
    "dedicate_params", "dedicate_params_ddp", "dedicate_params_ddp_tp", "replicate", "replicate_tp",
    "install_patch", "uninstall_patch", "Muon", "NewtonSchulz", "newton_schulz", "gram_newton_schulz",
    "direct_newton_schulz", "gram_newton_schulz_factors", "get_backend_status", "get_ns_backend",
    "get_comm_ctx", "get_dedicated_params", "get_owned_params", "DedicatedCommContext", "DMuonParamPolicy",
    "resolve_param_policies", "clip_grad_norm_", "clip_grad_norm_buckets_",
    "try_clip_optimizer_grad_norm_buckets_", "register_muon_grad_clip_strategy", "MuonGradClipStats",
    "GradClipBucket", "GradClipBucketStats", "SegmentedGradClipResult", "summarize_comm_plan",
    "summarize_param_groups", "no_sync", "prepare_muon_grads", "wait_all_reduces",
    "wait_all_replicate_broadcasts", "wait_all_post_step_broadcasts", "broadcast_all_updates",
    "broadcast_all_updates_async", "collect_forward_unshard_profile", "get_model_state_dict",
    "set_model_state_dict", "get_optimizer_state_dict", "set_optimizer_state_dict", "YOU_COEFFICIENTS",
    "POLAR_EXPRESS_COEFFICIENTS", "CLASSIC_COEFFICIENTS", "compute_balanced_assignment", "DedicatedParam",
    "DedicatedParamDDP", "DedicatedParamGroup", "DedicatedParamGroupDDP",
]

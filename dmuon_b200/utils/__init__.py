"""Model-level helpers: iterate dedicated state, drain or dispatch the
asynchronous phases of a step, gradient-accumulation context.

Same entry points as the reference's ``dmuon/utils.py`` (:28-64 iteration,
:89-204 gradient preparation, :238-438 post-step dispatch and drains, :441-484
debug fence, :487-530 ``no_sync``).
"""
from __future__ import annotations

import contextlib
import os
from typing import Iterator, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel.topology import is_isolated_process_group, isolated_process_groups, normalize_owner_rank  # noqa: F401


def get_comm_ctx(model: nn.Module):
    ctx = getattr(model, "_dedicated_comm_ctx", None)
    if ctx is None:
        raise RuntimeError(
            "model has no dedicated-parameter context: call dedicate_params "
            "(or dedicate_params_ddp / dedicate_params_ddp_tp) on it first"
        )
    return ctx


def iter_states(model: nn.Module) -> Iterator:
    ctx = getattr(model, "_dedicated_comm_ctx", None)
    if ctx is not None:
        yield from ctx.all_states


iter_dedicated_states = iter_states        # the reference's name (dmuon/utils.py:28)


def iter_groups(model: nn.Module) -> Iterator:
    """Groups in forward (module registration) order -- identical on every rank."""
    for st in iter_states(model):
        yield st.group


def get_dedicated_params(model: nn.Module) -> list:
    return [p for g in iter_groups(model) for p in g.params]


def get_owned_params(model: nn.Module, rank=None) -> list:
    """Dedicated parameters owned by this rank, or -- with ``rank`` (a shard
    index or a ``(shard, replicate)`` coordinate, as in the reference's
    ``get_owned_params(model, rank)``) -- by that owner coordinate."""
    if rank is None:
        return [p for p in get_dedicated_params(model) if p.is_owner]
    want = tuple(normalize_owner_rank(rank))
    return [p for p in get_dedicated_params(model) if tuple(p.owner_rank) == want]


# --------------------------------------------------------------------------- gradients
def prepare_group_muon_grads(group, use_reduce_lane: bool = True) -> None:
    """Queue everything the optimizer needs from this group: drain its reduce
    (owner gets ``_reduced_grad``) and start the tensor-parallel gather."""
    lane = group.comm_ctx.reduce_lane if use_reduce_lane else None
    if group.has_pending_reduce():
        group.wait_for_reduce(lane=lane)
    group.tp_gather_grads(lane=group.comm_ctx.reduce_lane)
    group._prepared_ticket = group.comm_ctx.reduce_lane.mark() if use_reduce_lane else None


def wait_group_muon_grads(group) -> None:
    t = getattr(group, "_prepared_ticket", None)
    if t is not None:
        t.wait_on_current()
        group._prepared_ticket = None
    group.materialize_tp_grads()


def prepare_muon_grads(model: nn.Module, coalesce_wait: bool = False, *, use_reduce_stream: Optional[bool] = None) -> None:
    """Make every owned gradient ready on the current stream.
    ``use_reduce_stream`` (keyword of the reference's function): ``False`` drains
    the reduces on the current stream instead of on the reduce lane; the default
    here is the lane, which is what the optimizer uses."""
    groups = list(iter_groups(model))
    on_lane = True if use_reduce_stream is None else bool(use_reduce_stream)
    for g in groups:
        prepare_group_muon_grads(g, use_reduce_lane=on_lane)
    if coalesce_wait and groups:
        # one aggregate wait on the lane instead of one per group
        groups[0].comm_ctx.reduce_lane.mark().wait_on_current()
        for g in groups:
            g._prepared_ticket = None
            g.materialize_tp_grads()
    else:
        for g in groups:
            wait_group_muon_grads(g)


def wait_all_reduces(model: nn.Module) -> None:
    prepare_muon_grads(model)


# --------------------------------------------------------------------------- post-step
def broadcast_all_updates(model: nn.Module) -> None:
    """Synchronous post-step publish for every group, in forward order."""
    broadcast_all_updates_async(model)
    wait_all_post_step_broadcasts(model)


def broadcast_all_updates_async(model: nn.Module) -> None:
    for g in iter_groups(model):
        g.post_step_publish_async()


def wait_all_replicate_broadcasts(model: nn.Module) -> None:
    """Drain asynchronous post-step publishes (required before reading master
    weights outside a forward pass, e.g. for a checkpoint)."""
    for g in iter_groups(model):
        g._pre_forward_wait()


wait_all_post_step_broadcasts = wait_all_replicate_broadcasts


def collect_forward_unshard_profile(model: nn.Module, *, clear: bool = True, synchronize: bool = False) -> dict:
    """Aggregated CUDA-event timings and counters of the forward publish
    (enabled with ``DMUON_RECORD_FORWARD_PROFILE=1``).  ``synchronize=True``
    waits for the device first, so that no timer is still pending;
    ``clear=False`` leaves the records in place for a later call."""
    ctx = get_comm_ctx(model)
    if synchronize and ctx.device.type == "cuda":
        torch.cuda.synchronize(ctx.device)
    return ctx.drain_profile("forward", clear=clear)


def collect_post_step_profile(model: nn.Module) -> dict:
    return get_comm_ctx(model).drain_profile("post_step")


def fence_isolated_process_groups(force: bool = False) -> None:
    """Optional step-end barrier on every cloned process group
    (``DMUON_ISOLATED_PG_BARRIER=1``); a debugging aid for collective-order
    problems."""
    raw = os.environ.get("DMUON_ISOLATED_PG_BARRIER", "0").strip().lower()
    if not force and raw in ("", "0", "false", "no", "off"):
        return
    if not (dist.is_available() and dist.is_initialized()):
        return
    for pg in isolated_process_groups():
        dist.barrier(group=pg)


@contextlib.contextmanager
def no_sync(model: nn.Module):
    """Skip gradient communication for the backward passes inside the context;
    gradients are kept locally and merged into the next synchronised backward.
    Also toggles FSDP2's and ``replicate``'s own synchronisation."""
    groups = list(iter_groups(model))
    prev = [g._no_sync for g in groups]
    fsdp_toggled = []
    for m in model.modules():
        setter = getattr(m, "set_requires_gradient_sync", None)
        if callable(setter):
            setter(False, recurse=False)
            fsdp_toggled.append(setter)
    rep = getattr(model, "_dmuon_replicated", None)
    if rep is not None:
        rep_prev = rep.require_sync
        rep.require_sync = False
    for g in groups:
        g._no_sync = True
    try:
        yield
    finally:
        for g, p in zip(groups, prev):
            g._no_sync = p
        for setter in fsdp_toggled:
            setter(True, recurse=False)
        if rep is not None:
            rep.require_sync = rep_prev

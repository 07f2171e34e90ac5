"""Gradient averaging for the parameters that are NOT dedicated, in the
replicated (DDP-style) placement.

``replicate(model, mesh)`` hooks every remaining trainable parameter: when
autograd has accumulated a gradient the parameter is queued, and one callback
at the end of the backward pass averages all queued gradients over the
data-parallel group, flattened into one buffer per dtype so a step costs one
collective per dtype.  ``replicate_tp`` does the same for DTensor parameters of
a tensor-parallel model (their local shards are averaged over the
data-parallel dimension only).  Reference: dmuon/_backends/ddp/replicate.py:146-279.
"""
from __future__ import annotations

from collections import defaultdict

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.autograd import Variable

from .dgroup import all_reduce_mean

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if DTensor is not None and isinstance(t, DTensor) else t


class _ReplicatedGroup:
    def __init__(self, params: list[nn.Parameter], group):
        self.params = params
        self.group = group
        self.require_sync = True
        self._queued: list[nn.Parameter] = []
        self._callback_queued = False
        self._handles = [p.register_post_accumulate_grad_hook(self._on_grad) for p in params]

    def _on_grad(self, p: nn.Parameter) -> None:
        if not self.require_sync:
            return
        self._queued.append(p)
        if not self._callback_queued:
            self._callback_queued = True
            Variable._execution_engine.queue_callback(self._flush)

    def _flush(self) -> None:
        self._callback_queued = False
        queued, self._queued = self._queued, []
        if not queued or self.group is None or self.group.size() <= 1:
            return
        buckets: dict[tuple, list[torch.Tensor]] = defaultdict(list)
        seen: set[int] = set()
        for p in queued:
            if id(p) in seen or p.grad is None:
                continue
            seen.add(id(p))
            g = _local(p.grad)
            buckets[(g.dtype, g.device)].append(g)
        with torch.no_grad():
            for (dtype, device), grads in buckets.items():
                flat = torch.empty(sum(g.numel() for g in grads), dtype=dtype, device=device)
                views, off = [], 0
                for g in grads:
                    views.append(flat[off : off + g.numel()].view_as(g))
                    off += g.numel()
                torch._foreach_copy_(views, grads)
                all_reduce_mean(flat, self.group)
                torch._foreach_copy_(grads, views)

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []


def _remaining_params(model: nn.Module) -> list[nn.Parameter]:
    out, seen = [], set()
    for p in model.parameters():
        if id(p) in seen or not p.requires_grad or hasattr(p, "_dedicated_owner_rank"):
            continue
        seen.add(id(p))
        out.append(p)
    return out


def _group_of(mesh_or_group):
    if mesh_or_group is None:
        return dist.group.WORLD if dist.is_initialized() else None
    if hasattr(mesh_or_group, "get_group"):
        return mesh_or_group.get_group()
    return mesh_or_group


def replicate(model: nn.Module, mesh=None) -> nn.Module:
    """Average the gradients of every non-dedicated parameter over ``mesh``
    (a 1-D DeviceMesh or a ProcessGroup; default: the world)."""
    params = _remaining_params(model)
    rep = _ReplicatedGroup(params, _group_of(mesh))
    model._dmuon_replicated = rep
    for p in params:
        p._dmuon_replicated = True
    return model


def replicate_tp(model: nn.Module, mesh=None, *, dp_mesh=None) -> nn.Module:
    """Tensor-parallel variant: ``mesh`` is the data-parallel sub-mesh (keyword
    ``dp_mesh`` is accepted as well); the gradients' local shards are averaged
    over it."""
    if mesh is None:
        mesh = dp_mesh
    if mesh is None:
        raise TypeError("replicate_tp needs the data-parallel mesh")
    return replicate(model, mesh)

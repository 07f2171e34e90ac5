"""Mesh-level facts: owner coordinates, tensor-parallel detection, group cloning.

Covers the roles of the reference's ``_core/owner_rank.py``, ``_core/tp.py``
and ``_core/process_groups.py``.
"""
from __future__ import annotations

import os
from typing import Optional

import torch.distributed as dist

try:  # DTensor is optional at import time (CPU-only unit tests use fakes)
    from torch.distributed.tensor import DTensor
    from torch.distributed.tensor.placement_types import Shard
except Exception:  # pragma: no cover
    DTensor = None
    Shard = None


# --------------------------------------------------------------------------- owner coords
def normalize_owner_rank(owner) -> tuple[int, int]:
    """``3 -> (3, 0)``; ``(s, r)`` is validated and returned as ints.

    Booleans are rejected explicitly: ``True`` is an ``int`` in Python and a
    predicate result stored by mistake would otherwise become rank 1
    (reference: dmuon/_core/owner_rank.py:19-50).
    """
    if isinstance(owner, bool):
        raise TypeError("owner rank must be an int or a (shard, replicate) pair, not bool")
    if isinstance(owner, int):
        if owner < 0:
            raise ValueError(f"owner rank must be non-negative, got {owner}")
        return (int(owner), 0)
    if isinstance(owner, (tuple, list)):
        if len(owner) != 2:
            raise ValueError(f"owner coordinate must have two entries, got {owner!r}")
        s, r = owner
        if isinstance(s, bool) or isinstance(r, bool) or not isinstance(s, int) or not isinstance(r, int):
            raise TypeError(f"owner coordinate entries must be ints, got {owner!r}")
        if s < 0 or r < 0:
            raise ValueError(f"owner coordinate entries must be non-negative, got {owner!r}")
        return (int(s), int(r))
    raise TypeError(f"owner rank must be an int or a (shard, replicate) pair, got {type(owner)!r}")


# --------------------------------------------------------------------------- tensor parallel
def _tp_dim_names(param, dp_dim_names: frozenset) -> list[str]:
    names = param.device_mesh.mesh_dim_names
    if names is None:
        raise ValueError(
            "tensor-parallel detection needs a named DeviceMesh; "
            "build it with init_device_mesh(..., mesh_dim_names=(...))"
        )
    return [n for n in names if n not in dp_dim_names]


def is_tp_sharded(param, dp_dim_names: frozenset) -> bool:
    """True when ``param`` is a DTensor with a ``Shard`` placement on a mesh
    dimension that is neither the shard nor the replicate axis and has more
    than one rank (reference: dmuon/_core/tp.py:41-77)."""
    if DTensor is None or not isinstance(param, DTensor):
        return False
    names = param.device_mesh.mesh_dim_names
    for name in _tp_dim_names(param, dp_dim_names):
        if param.device_mesh[name].size() <= 1:
            continue
        if isinstance(param.placements[names.index(name)], Shard):
            return True
    return False


def get_tp_mesh(param, dp_dim_names: frozenset):
    tp = _tp_dim_names(param, dp_dim_names)
    if len(tp) != 1:
        raise AssertionError(f"only one tensor-parallel mesh dimension is supported, found {tp}")
    return param.device_mesh[tp[0]]


def get_tp_shard_dim(param, dp_dim_names: frozenset) -> int:
    """0 for column-parallel weights (rows split), 1 for row-parallel ones."""
    names = param.device_mesh.mesh_dim_names
    tp = _tp_dim_names(param, dp_dim_names)[0]
    placement = param.placements[names.index(tp)]
    if not isinstance(placement, Shard):
        raise AssertionError(f"expected a Shard placement on mesh dim {tp!r}, got {placement}")
    return int(placement.dim)


# --------------------------------------------------------------------------- process groups
_PG_POLICIES = ("isolated", "shared")
_PG_ALIASES = {
    "default": "isolated",
    "isolate": "isolated",
    "dmuon": "isolated",
    "reuse": "shared",
    "caller": "shared",
    "mesh": "shared",
    "none": "shared",
}
_cloned: dict[tuple, object] = {}
_cloned_ids: set[int] = set()


def resolve_process_group_policy(policy: Optional[str] = None) -> str:
    raw = policy if policy is not None else os.environ.get("DMUON_PROCESS_GROUP_POLICY", "isolated")
    key = str(raw).strip().lower()
    key = _PG_ALIASES.get(key, key)
    if key not in _PG_POLICIES:
        raise ValueError(f"Unsupported process_group_policy={raw!r}; expected one of {', '.join(_PG_POLICIES)}.")
    return key


def maybe_isolate_process_group(group, *, policy: str, role: str):
    """Clone ``group`` so this library's collectives never share a communicator
    with the trainer's.

    Every rank learns all rank sets of this role through one world all-gather
    and then creates ALL of them in one deterministic order, which keeps the
    ``new_group`` calls aligned across ranks (reference:
    dmuon/_core/process_groups.py:46-110).
    """
    if group is None or policy == "shared":
        return group
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() <= 1:
        return group
    mine = tuple(int(r) for r in dist.get_process_group_ranks(group))
    key = (str(role), mine)
    if key in _cloned:
        return _cloned[key]
    everyone: list = [None] * dist.get_world_size()
    dist.all_gather_object(everyone, mine)
    partitions = sorted({tuple(int(r) for r in ranks) for ranks in everyone if ranks is not None})
    if mine not in partitions:
        raise RuntimeError(f"group cloning for role {role!r}: own rank set {mine} missing from the gathered sets")
    backend = dist.get_backend(group)
    clone = None
    for ranks in partitions:
        g = dist.new_group(ranks=list(ranks), backend=backend)
        if ranks == mine:
            clone = g
    if clone is None or clone == dist.GroupMember.NON_GROUP_MEMBER:
        raise RuntimeError(f"group cloning for role {role!r} produced no group for this rank")
    _cloned[key] = clone
    _cloned_ids.add(id(clone))
    return clone


def is_isolated_process_group(group) -> bool:
    if group is None or group == dist.GroupMember.NON_GROUP_MEMBER:
        return False
    return id(group) in _cloned_ids


def isolated_process_groups() -> list:
    return list(_cloned.values())

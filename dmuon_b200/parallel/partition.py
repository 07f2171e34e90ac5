"""Owner assignment: which rank runs the matrix optimizer for which parameter.

The assignment is a longest-processing-time-first greedy over "owner slots"
(the shard x replicate grid), with two structural rules that keep the
per-layer communication parallel:

* parameters of one layer prefer slots the layer has not used yet;
* small parameters of one layer travel together as one unit (one packed
  publish buffer, one owner).

The decision procedure (cost units, sort keys, tie-breaks) follows the
reference so that both frameworks place a given model identically
(dmuon/_core/partition.py:182-210 cost model, :379-396 ordering, :429-446
slot choice, :463-513 tensor-parallel owners).  The code is pure Python and
needs no process group: any object with ``size()`` and ``mesh_dim_names``
works as a mesh, which is what the unit tests use.
"""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Callable, Iterator, Optional, Union

import torch.nn as nn

from .topology import get_tp_mesh, is_tp_sharded

SMALL_PARAM_THRESHOLD = 5_000_000

OwnerCoord = tuple[int, int]
OwnerValue = Union[int, OwnerCoord]

_ADAMW_NAME_HINTS = ("embed", "embedding", "lm_head", "norm", "layernorm", "ln_", ".ln", "bias", "rope", "rotary")


@dataclass
class AssignmentResult:
    """Mapping ``param -> owner`` plus bookkeeping; behaves like ``dp_owners``."""

    dp_owners: dict = field(default_factory=dict)
    tp_owners: dict = field(default_factory=dict)
    allocation_unit_count: int = 0
    packed_allocation_unit_count: int = 0
    pack_small_params: bool = True

    def __getitem__(self, key):
        return self.dp_owners[key]

    def __contains__(self, key) -> bool:
        return key in self.dp_owners

    def __iter__(self) -> Iterator:
        return iter(self.dp_owners)

    def __len__(self) -> int:
        return len(self.dp_owners)

    def items(self):
        return self.dp_owners.items()

    def keys(self):
        return self.dp_owners.keys()

    def values(self):
        return self.dp_owners.values()

    def get(self, key, default=None):
        return self.dp_owners.get(key, default)


def layer_key(name: str) -> Optional[str]:
    """``a.layers.7.x.weight -> "a.layers.7"``; also ``blocks.N``; else None."""
    parts = name.split(".")
    for i in range(len(parts) - 1):
        if parts[i] in ("layers", "blocks"):
            head = ".".join(parts[:i]) or "_root"
            return f"{head}.{parts[i]}.{parts[i + 1]}"
    return None


def _local_numel(param) -> int:
    local = getattr(param, "_local_tensor", None)
    return int(local.numel()) if local is not None else int(param.numel())


def routes_to_adamw_by_name(name: str, shape: tuple[int, ...]) -> bool:
    if len(shape) < 2:
        return True
    low = name.lower()
    return any(tok in low for tok in _ADAMW_NAME_HINTS)


def optimizer_cost_units(name: str, shape: tuple[int, ...], numel: int) -> int:
    """Coarse owner-side work estimate: Newton-Schulz flops + a byte term."""
    numel = max(1, int(numel))
    if routes_to_adamw_by_name(name, shape):
        return max(1, numel // 1_000_000)
    rows = int(shape[0])
    cols = int(math.prod(shape[1:]))
    small, big = max(1, min(rows, cols)), max(rows, cols)
    flops = 5 * small * (rows * cols + 2 * big * small)
    return max(1, flops // 1_000_000_000) + max(1, numel // 4_000_000)


@dataclass
class _Unit:
    params: list
    group: Optional[str]
    numel: int
    cost: int
    first_order: int
    names: str


def compute_balanced_assignment(
    model: nn.Module,
    mesh,
    predicate: Callable[[str, nn.Parameter], bool],
    replicate_mesh=None,
    owner_strategy: str = "lpt",
    tp_owner_strategy: str = "lpt",
    assignment_group_key_fn: Optional[Callable[[str, nn.Parameter], Optional[str]]] = None,
    max_owners_per_group: Optional[int] = None,
    owner_cost_model: str = "optimizer",
    hsdp_column_balance: bool = True,
    pack_small_params: bool = True,
) -> AssignmentResult:
    if owner_strategy not in ("lpt", "round_robin", "rank0"):
        raise ValueError(f"Unsupported owner_strategy: {owner_strategy!r}; expected 'lpt', 'round_robin', or 'rank0'.")
    if tp_owner_strategy != "lpt":
        raise ValueError(f"Unsupported tp_owner_strategy: {tp_owner_strategy!r}; only 'lpt' is supported.")
    if max_owners_per_group is not None and max_owners_per_group <= 0:
        raise ValueError("max_owners_per_group must be positive when set")
    if owner_cost_model not in ("optimizer", "numel"):
        raise ValueError(f"Unsupported owner_cost_model: {owner_cost_model!r}; expected 'optimizer' or 'numel'.")

    n_shard = mesh.size()
    n_rep = replicate_mesh.size() if replicate_mesh is not None else 1
    hsdp = replicate_mesh is not None
    slots: list[OwnerCoord] = [(s, r) for s in range(n_shard) for r in range(n_rep)]

    dp_dims: set[str] = set(mesh.mesh_dim_names or ())
    if replicate_mesh is not None:
        dp_dims |= set(replicate_mesh.mesh_dim_names or ())
    dp_dims_f = frozenset(dp_dims)

    def cost_of(name: str, p) -> int:
        if owner_cost_model == "numel":
            return int(p.numel()) if is_tp_sharded(p, dp_dims_f) else _local_numel(p)
        return optimizer_cost_units(name, tuple(int(d) for d in p.shape), int(p.numel()))

    names: dict = {}
    by_group: dict[Optional[str], list[tuple]] = defaultdict(list)
    for order, (name, p) in enumerate(model.named_parameters()):
        if not predicate(name, p):
            continue
        names[p] = name
        gkey = assignment_group_key_fn(name, p) if assignment_group_key_fn is not None else layer_key(name)
        tp = is_tp_sharded(p, dp_dims_f)
        numel = int(p.numel()) if tp else _local_numel(p)
        by_group[gkey].append((p, name, numel, cost_of(name, p), order, tp))

    units: list[_Unit] = []
    packed_units = 0
    for gkey, members in by_group.items():
        if not pack_small_params:
            units += [_Unit([p], gkey, n, c, o, nm) for p, nm, n, c, o, _ in members]
            continue
        standalone = [m for m in members if m[5]]                       # TP-sharded: never packed
        standalone += [m for m in members if not m[5] and m[2] >= SMALL_PARAM_THRESHOLD]
        small = [m for m in members if not m[5] and m[2] < SMALL_PARAM_THRESHOLD]
        units += [_Unit([p], gkey, n, c, o, nm) for p, nm, n, c, o, _ in standalone]
        if small:
            units.append(
                _Unit(
                    [m[0] for m in small],
                    gkey,
                    sum(m[2] for m in small),
                    sum(m[3] for m in small),
                    min(m[4] for m in small),
                    ",".join(m[1] for m in small),
                )
            )
            packed_units += len(small) > 1

    if owner_strategy == "lpt":
        units.sort(key=lambda u: (-u.cost, -u.numel, "" if u.group is None else str(u.group), u.names))
    else:
        units.sort(key=lambda u: u.first_order)

    load_numel = {s: 0 for s in slots}
    load_cost = {s: 0 for s in slots}
    col_numel = [0] * n_shard
    col_cost = [0] * n_shard
    used_by_group: dict[Optional[str], set] = defaultdict(set)
    placed: dict = {}
    rr = 0
    column_first = hsdp and hsdp_column_balance
    for u in units:
        used = used_by_group[u.group]
        cands = slots
        if max_owners_per_group is not None and len(used) >= max_owners_per_group:
            cands = sorted(used)
        if owner_strategy == "rank0":
            pick = slots[0]
        elif owner_strategy == "round_robin":
            pick = cands[rr % len(cands)]
            rr += 1
        else:
            pick = min(
                cands,
                key=lambda s: (
                    s in used,
                    col_cost[s[0]] if column_first else 0,
                    load_cost[s],
                    col_numel[s[0]] if column_first else 0,
                    load_numel[s],
                ),
            )
        for p in u.params:
            placed[p] = pick
        load_numel[pick] += u.numel
        load_cost[pick] += u.cost
        col_numel[pick[0]] += u.numel
        col_cost[pick[0]] += u.cost
        used.add(pick)

    dp_owners = dict(placed) if hsdp else {p: c[0] for p, c in placed.items()}

    # Tensor-parallel owners: a separate LPT inside every DP-owner bucket, with
    # the tie-break rotated by the bucket so equal shapes do not pile up on TP
    # rank 0.
    tp_owners: dict = {}
    buckets: dict = defaultdict(list)
    for p, owner in dp_owners.items():
        if is_tp_sharded(p, dp_dims_f):
            buckets[owner].append(p)

    def tp_cost(p) -> int:
        if owner_cost_model == "numel":
            return int(p.numel())
        return optimizer_cost_units(names.get(p, ""), tuple(int(d) for d in p.shape), int(p.numel()))

    for owner, plist in buckets.items():
        tp_size = get_tp_mesh(plist[0], dp_dims_f).size()
        rot = (owner[0] * n_rep + owner[1]) % tp_size if isinstance(owner, tuple) else int(owner) % tp_size
        c_load = [0] * tp_size
        n_load = [0] * tp_size
        for p in sorted(plist, key=lambda q: (-tp_cost(q), -int(q.numel()), names.get(q, ""))):
            t = min(range(tp_size), key=lambda i: (c_load[i], n_load[i], (i - rot) % tp_size))
            tp_owners[p] = t
            c_load[t] += tp_cost(p)
            n_load[t] += int(p.numel())

    return AssignmentResult(
        dp_owners=dp_owners,
        tp_owners=tp_owners,
        allocation_unit_count=len(units),
        packed_allocation_unit_count=int(packed_units),
        pack_small_params=pack_small_params,
    )


def imbalance(loads: list[int]) -> float:
    """(max - mean) / mean of a load vector; 0 for an empty or all-zero one."""
    if not loads:
        return 0.0
    mean = sum(loads) / len(loads)
    return (max(loads) - mean) / mean if mean > 0 else 0.0

"""JSON-friendly, collective-free summaries of how a model was set up.

``summarize_param_groups`` lists every optimizer group with its dedicated and
ordinary parameters; ``summarize_comm_plan`` lists every communication group
with the bytes each step moves for it and per-owner load.  Neither function
communicates or synchronises, so they can be called on any subset of ranks
(reference: dmuon/diagnostics.py:130-247, :250-395).
"""
from __future__ import annotations

from collections import defaultdict
from typing import Any

import torch

from .utils import iter_groups


def _dtype(d) -> str:
    return str(d).replace("torch.", "") if d is not None else "none"


def _esize(d: torch.dtype) -> int:
    return torch.empty((), dtype=d).element_size()


def _dp_entry(dp) -> dict[str, Any]:
    return {
        "name": dp.fqn,
        "shape": list(dp._orig_size),
        "full_shape": list(dp.full_shape),
        "numel": int(dp.numel),
        "owner": list(dp.owner_rank),
        "is_owner": bool(dp.is_owner),
        "route": dp._dmuon_route,
        "param_dtype": _dtype(dp._param_dtype),
        "grad_dtype": _dtype(dp._grad_dtype),
        "master_dtype": _dtype(dp._master_dtype),
        "optim_dtype": _dtype(dp._optim_dtype),
        "tp_sharded": dp.tp_group is not None,
        "is_tp_owner": bool(dp.is_tp_owner),
        "mode": dp.mode,
    }


def summarize_param_groups(optimizer) -> list[dict[str, Any]]:
    out = []
    for i, pg in enumerate(optimizer.param_groups):
        all_dps = optimizer._bucket_all_dps.get(i, [])
        owned = optimizer._bucket_dps.get(i, [])
        plain = optimizer._bucket_plain.get(i, [])
        hp = {k: (list(v) if isinstance(v, tuple) else v) for k, v in pg.items() if k != "params"}
        out.append(
            {
                "index": i,
                "group_name": pg.get("group_name"),
                "semantic_group_name": pg.get("semantic_group_name"),
                "subgroup_type": pg.get("subgroup_type"),
                "use_muon": bool(pg.get("use_muon")),
                "hyperparameters": hp,
                "dedicated_param_count": len(all_dps),
                "owned_dedicated_param_count": len(owned),
                "owned_dedicated_numel": int(sum(dp.numel for dp in owned)),
                "plain_param_count": len(plain),
                "plain_local_numel": int(sum(getattr(p, "_local_tensor", p).numel() for p in plain)),
                "dedicated_params": [_dp_entry(dp) for dp in all_dps],
            }
        )
    return out


def summarize_comm_plan(model) -> dict[str, Any]:
    """Per-group byte estimates.  A broadcast or reduce of ``B`` bytes over ``N``
    ranks is counted as ``B * (N - 1) / N`` per rank (ring / switch volume)."""
    groups = []
    owner_numel: dict[tuple, int] = defaultdict(int)
    totals = defaultdict(float)
    for g in iter_groups(model):
        n, r = g.shard_size, g.replicate_size
        pub = sum(p.numel * _esize(p._param_dtype) for p in g.bcast_params)
        red = sum(p.numel * _esize(p._grad_dtype or p._param_dtype) for p in g.bcast_params)
        flat = sum(p._flat_shard_numel * n * _esize(p._param_dtype) for p in g.flat_params)
        rep = sum(p.numel * _esize(p._master_dtype) for p in g.bcast_params) if r > 1 else 0
        publishes = 1 if (g.mode == "ddp" or not g.reshard_after_forward) else 2
        factor = (n - 1) / n if n > 1 else 0.0
        rfactor = (r - 1) / r if r > 1 else 0.0
        entry = {
            "name": g.name,
            "mode": g.mode,
            "reshard_after_forward": bool(g.reshard_after_forward),
            "param_count": len(g.params),
            "owners": sorted({list(p.owner_rank)[0] for p in g.bcast_params}),
            "owner_coords": sorted({tuple(p.owner_rank) for p in g.bcast_params}),
            "publish_bytes": int(pub),
            "publishes_per_step": publishes if g.mode == "fsdp" else 0,
            "reduce_bytes": int(red),
            "sharded_adamw_bytes": int(flat),
            "replicate_publish_bytes": int(rep),
            "tp_param_count": len(g.tp_params),
            "est_bytes_per_rank_per_step": int(
                (pub * publishes * factor if g.mode == "fsdp" else pub * factor)
                + red * factor
                + 2 * flat * factor
                + (rep + red) * rfactor
            ),
        }
        groups.append(entry)
        for p in g.bcast_params:
            owner_numel[tuple(p.owner_rank)] += p.numel
        totals["publish_bytes"] += pub
        totals["reduce_bytes"] += red
        totals["est_bytes_per_rank_per_step"] += entry["est_bytes_per_rank_per_step"]
    loads = list(owner_numel.values())
    mean = sum(loads) / len(loads) if loads else 0.0
    return {
        "groups": groups,
        "totals": {k: int(v) for k, v in totals.items()},
        "owner_numel": {f"{s},{r}": int(v) for (s, r), v in sorted(owner_numel.items())},
        "owner_imbalance": (max(loads) - mean) / mean if mean > 0 else 0.0,
    }

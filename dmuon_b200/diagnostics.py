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


def _data_plane(model) -> dict[str, Any]:
    """Which mechanism moves the dedicated parameters, with the memory it holds
    and what one step costs this rank over NVLink (estimates from sizes)."""
    ctx = getattr(model, "_dedicated_comm_ctx", None)
    rt = getattr(ctx, "peer_runtime", None)
    out: dict[str, Any] = {"kind": "collective (torch.distributed)"}
    if rt is not None:
        esz_p, esz_g = rt.pub.element_size(), rt.grad.element_size()
        own_elems = max(rt.own_hi - rt.own_lo, 0)
        total = rt.payload_end - rt.guard
        others = max(total - own_elems, 0)
        out = {
            "kind": "peer memory",
            "copy_mode": rt.copy_mode,
            "reduce_via": rt.reduce_via,
            "publish_via": rt.publish_via,
            "ranks": rt.world,
            "publish_arena_bytes": int(rt.total * esz_p),
            "gradient_arena_bytes": int(rt.total * esz_g),
            "owned_span_bytes": int(own_elems * esz_g),
            # what the owner keeps besides the arenas: gathered peer slices ("ce") or one reduced copy ("nvls")
            "staging_bytes": int(rt.stage.numel() * esz_g) if rt.stage is not None else 0,
            "reduced_copy_bytes": int(rt.reduced.numel() * esz_g) if rt.reduced is not None else 0,
            "multicast_mapped": bool(rt.pub_mc and rt.grad_mc),
            # per step and rank: weights of other owners arrive, gradients of other owners' spans leave
            "publish_ingress_bytes": int(others * esz_p),
            "publish_egress_bytes": int(own_elems * esz_p * (1 if rt.publish_via == "nvls" else max(rt.world - 1, 0))),
            "reduce_egress_bytes": int(others * esz_g),
            "reduce_ingress_bytes": int(own_elems * esz_g * (1 if rt.reduce_via == "nvls" else max(rt.world - 1, 0))),
            "fused_forward_publish": bool(rt.fused_forward),
            "replicated_placement": bool(getattr(ctx, "ddp_on_peer_plane", False)),
        }
    ex = getattr(ctx, "tp_exchanges", None) or {}
    if ex:
        out["tensor_parallel_exchange"] = [
            {
                "ranks": e.world,
                "gradient_shard_buffer_bytes": int(e.grad_total * e.grad.element_size()),
                "update_buffer_bytes": int(e.delta_total * 4),
                "params": len(e.params),
            }
            for e in ex.values()
        ]
    return out


def summarize_comm_plan(model, *, max_groups: int = 64, max_params_per_group: int = 128) -> dict[str, Any]:
    """Per-group byte estimates.  A broadcast or reduce of ``B`` bytes over ``N``
    ranks is counted as ``B * (N - 1) / N`` per rank (ring / switch volume).
    Every group lists its owner buckets (what one owner publishes and receives
    for this group, with the global rank that is the root) and, up to
    ``max_params_per_group``, its parameters; ``data_plane`` says which mechanism
    carries the bytes.  At most ``max_groups`` groups are listed (totals cover all)."""
    groups = []
    owner_numel: dict[tuple, int] = defaultdict(int)
    totals = defaultdict(float)
    max_bucket = 0
    for gi, g in enumerate(iter_groups(model)):
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
        buckets: dict[tuple, list] = defaultdict(list)
        for p in g.bcast_params:
            buckets[tuple(p.owner_rank)].append(p)
        entry["owner_buckets"] = []
        for coord, plist in sorted(buckets.items()):
            b = sum(p.numel * _esize(p._param_dtype) for p in plist)
            max_bucket = max(max_bucket, b)
            root = None
            try:
                root = int(g._global_rank(g.dp_group, coord[0]))
            except Exception:
                pass
            entry["owner_buckets"].append({
                "owner_coord": list(coord), "publish_bytes": int(b),
                "reduce_bytes": int(sum(p.numel * _esize(p._grad_dtype or p._param_dtype) for p in plist)),
                "param_count": len(plist), "root_global_rank": root,
            })
        entry["params"] = [
            {"name": p.fqn, "numel": int(p.numel), "owner": list(p.owner_rank), "route": p._dmuon_route,
             "tp_owner_local_rank": (int(p._tp_owner_local_rank) if p.tp_group is not None else None)}
            for p in g.params[:max_params_per_group]
        ]
        entry["params_truncated"] = max(0, len(g.params) - max_params_per_group)
        if gi < max_groups:
            groups.append(entry)
        for p in g.bcast_params:
            owner_numel[tuple(p.owner_rank)] += p.numel
        totals["publish_bytes"] += pub
        totals["reduce_bytes"] += red
        totals["est_bytes_per_rank_per_step"] += entry["est_bytes_per_rank_per_step"]
    loads = list(owner_numel.values())
    mean = sum(loads) / len(loads) if loads else 0.0
    totals["max_owner_bucket_bytes"] = max_bucket
    n_groups = sum(1 for _ in iter_groups(model))
    return {
        "groups": groups,
        "groups_truncated": max(0, n_groups - max_groups),
        "data_plane": _data_plane(model),
        "totals": {k: int(v) for k, v in totals.items()},
        "owner_numel": {f"{s},{r}": int(v) for (s, r), v in sorted(owner_numel.items())},
        "owner_imbalance": (max(loads) - mean) / mean if mean > 0 else 0.0,
    }

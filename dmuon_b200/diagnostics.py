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


def _owner_list(owner) -> list:
    try:
        return [int(x) for x in owner]
    except TypeError:
        return [int(owner), 0]


def summarize_param_groups(model, optimizer=None, *, max_rows: int = 128) -> dict[str, Any]:
    """How ``Muon`` routed the trainable parameters: one entry per optimizer
    group under ``groups`` and one row per dedicated parameter under
    ``parameters`` (at most ``max_rows``; ``parameters_truncated`` counts the
    rest).  Counts are facts of this rank unless the key says otherwise.  Call
    as ``summarize_param_groups(model, optimizer)`` (the reference's signature,
    dmuon/diagnostics.py:130) or ``summarize_param_groups(optimizer)``."""
    if optimizer is None:
        optimizer = model                      # single-argument form: the optimizer knows its model
    param_groups = list(getattr(optimizer, "param_groups", []) or [])
    groups = []
    group_of: dict[int, int] = {}
    for i, pg in enumerate(param_groups):
        all_dps = optimizer._bucket_all_dps.get(i, [])
        owned = optimizer._bucket_dps.get(i, [])
        plain = optimizer._bucket_plain.get(i, [])
        for dp in all_dps:
            group_of[id(dp)] = i
        routes: dict[str, int] = defaultdict(int)
        for dp in all_dps:
            routes[str(dp._dmuon_route)] += 1
        hp = {k: (list(v) if isinstance(v, tuple) else v) for k, v in pg.items() if k != "params"}
        name = pg.get("group_name")
        params = pg.get("params", [])
        groups.append(
            {
                "group_index": i,
                "index": i,
                "group_name": str(name) if name is not None else f"group_{i}",
                "semantic_group_name": str(pg.get("semantic_group_name", name if name is not None else f"group_{i}")),
                "subgroup_type": str(pg.get("subgroup_type") or ""),
                "use_muon": bool(pg.get("use_muon")),
                "hyperparameters": hp,
                "optimizer_param_count": len(list(params)) if not isinstance(params, torch.Tensor) else 1,
                "dedicated_param_count": len(all_dps),
                "owned_dedicated_param_count": len(owned),
                "owned_dedicated_numel": int(sum(dp.numel for dp in owned)),
                "dedicated_muon_param_count": sum(1 for dp in all_dps if dp._dmuon_route == "muon"),
                "dedicated_adamw_param_count": sum(1 for dp in all_dps if dp._dmuon_route != "muon"),
                "adamw_param_count": len(plain),
                "plain_param_count": len(plain),
                "plain_local_numel": int(sum(getattr(p, "_local_tensor", p).numel() for p in plain)),
                "route_param_counts": dict(routes),
                "dedicated_params": [_dp_entry(dp) for dp in all_dps],
            }
        )
    all_dedicated = list(getattr(optimizer, "_all_dedicated", []) or [])
    rows = []
    for dp in all_dedicated[:max_rows]:
        gi = group_of.get(id(dp))
        pol = getattr(dp, "policy", None)
        rows.append(
            {
                "name": dp.fqn,
                "param_name": str(getattr(dp, "param_name", dp.fqn)),
                "route": str(dp._dmuon_route),
                "param_dtype": _dtype(dp._param_dtype),
                "grad_dtype": _dtype(dp._grad_dtype),
                "output_dtype": _dtype(getattr(dp, "_output_dtype", None)),
                "master_dtype": _dtype(dp._master_dtype),
                "optim_dtype": _dtype(dp._optim_dtype),
                "cast_forward_inputs": bool(getattr(dp, "_cast_forward_inputs", False)),
                "matched_policy_overrides": list(getattr(pol, "matched_overrides", ()) or ()),
                "group_index": gi,
                "group_name": groups[gi]["group_name"] if gi is not None else None,
                "owner_rank": _owner_list(dp.owner_rank),
                "is_owner": bool(dp.is_owner),
                "is_dtensor": bool(getattr(dp, "is_dtensor", False)),
                "uses_sharded_adamw": dp._dmuon_route == "sharded_adamw",
                "numel": int(dp.numel),
                "shape": [int(x) for x in dp.full_shape],
            }
        )
    return {
        "available": True,
        "num_groups": len(param_groups),
        "dedicated_param_count": len(all_dedicated),
        "owned_dedicated_param_count": sum(1 for dp in all_dedicated if dp.is_owner),
        "groups": groups,
        "parameters": rows,
        "parameters_truncated": max(0, len(all_dedicated) - len(rows)),
    }


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


def _group_rank(group) -> Any:
    try:
        return int(group.rank()) if group is not None else None
    except Exception:
        return None


def summarize_comm_plan(model, *, max_groups: int = 64, max_params_per_group: int = 128) -> dict[str, Any]:
    """Per-group byte estimates (planned tensor sizes and roots, not measured
    times).  A broadcast or reduce of ``B`` bytes over ``N`` ranks is counted as
    ``B * (N - 1) / N`` per rank (ring / switch volume).  Every group lists its
    owner buckets (what one owner publishes and receives for this group, with
    the global rank that is the root) and, up to ``max_params_per_group``, its
    parameters with the roots of the collectives they take part in;
    ``data_plane`` says which mechanism carries the bytes.  At most
    ``max_groups`` groups are listed (totals cover all).  The keys of the
    reference's summary (dmuon/diagnostics.py:250-395: ``group_count``,
    ``debug_name``, ``owner_bucket_bytes``, ``param_collectives``, the
    ``stage1_* / stage2_* / post_step_*`` totals) are present with the same
    meaning, next to this package's own."""
    groups = []
    owner_numel: dict[tuple, int] = defaultdict(int)
    totals = defaultdict(float)
    for key in ("dedicated_local_bytes", "stage1_shard_reduce_tensor_bytes", "stage1_shard_reduce_ring_bytes_per_rank",
                "stage2_replicate_reduce_tensor_bytes_this_rank", "post_step_replicate_broadcast_tensor_bytes_this_rank",
                "owner_update_ring_bytes_per_rank", "same_payload_allreduce_ring_bytes_per_rank"):
        totals[key] = 0
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
            "group_index": gi,
            "name": g.name,
            "debug_name": g.name,
            "mode": g.mode,
            "shard_rank": int(g.shard_rank),
            "replicate_rank": int(g.replicate_rank) if r > 1 else None,
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
        for bi, (coord, plist) in enumerate(sorted(buckets.items())):
            b = sum(p.numel * _esize(p._param_dtype) for p in plist)
            max_bucket = max(max_bucket, b)
            root = None
            try:
                root = int(g._global_rank(g.dp_group, coord[0]))
            except Exception:
                pass
            entry["owner_buckets"].append({
                "bucket_index": bi, "owner_coord": list(coord), "bytes": int(b), "publish_bytes": int(b),
                "reduce_bytes": int(sum(p.numel * _esize(p._grad_dtype or p._param_dtype) for p in plist)),
                "param_count": len(plist), "root_global_rank": root, "stage1_shard_reduce_root_global_rank": root,
            })
        entry["owner_bucket_count"] = len(entry["owner_buckets"])
        entry["owner_bucket_bytes"] = [b["bytes"] for b in entry["owner_buckets"]]
        entry["owner_bucket_bytes_in_order"] = list(entry["owner_bucket_bytes"])
        # replicate axis: only the ranks of the owner's shard column take part in stage 2 and in the post-step publish
        stage2 = 0
        collectives = []
        for pi, p in enumerate(g.params):
            pbytes = int(p.numel * _esize(p._param_dtype))
            active = bool(r > 1 and p._dmuon_route != "sharded_adamw" and p.in_owner_column)
            if active:
                stage2 += pbytes
            if pi < max_params_per_group:
                rep_root = None
                if r > 1:
                    try:
                        rep_root = int(g._global_rank(g.replicate_group, p.owner_replicate))
                    except Exception:
                        pass
                s1_root = None
                try:
                    s1_root = int(g._global_rank(g.dp_group, p.owner_shard))
                except Exception:
                    pass
                collectives.append({
                    "param_index": pi, "param_name": p.fqn, "name": p.fqn, "owner_coord": list(p.owner_rank),
                    "owner": list(p.owner_rank), "bytes": pbytes, "numel": int(p.numel), "route": p._dmuon_route,
                    "param_dtype": _dtype(p._param_dtype), "grad_dtype": _dtype(p._grad_dtype),
                    "stage1_shard_reduce_root_global_rank": s1_root,
                    "stage2_replicate_axis_active_on_this_rank": active,
                    "stage2_replicate_reduce_root_global_rank": rep_root,
                    "post_step_replicate_broadcast_root_global_rank": rep_root,
                    "tp_owner_local_rank": (int(p._tp_owner_local_rank) if p.tp_group is not None else None),
                })
        entry["param_collectives"] = collectives
        entry["params"] = collectives
        entry["param_collectives_truncated"] = max(0, len(g.params) - max_params_per_group)
        entry["params_truncated"] = entry["param_collectives_truncated"]
        if gi < max_groups:
            groups.append(entry)
        for p in g.bcast_params:
            owner_numel[tuple(p.owner_rank)] += p.numel
        local = sum(int(p.numel * _esize(p._param_dtype)) for p in g.params)
        bucket_bytes = sum(entry["owner_bucket_bytes"])
        totals["publish_bytes"] += pub
        totals["reduce_bytes"] += red
        totals["est_bytes_per_rank_per_step"] += entry["est_bytes_per_rank_per_step"]
        totals["dedicated_local_bytes"] += local
        totals["stage1_shard_reduce_tensor_bytes"] += local
        totals["stage1_shard_reduce_ring_bytes_per_rank"] += round(local * 2 * factor)
        totals["stage2_replicate_reduce_tensor_bytes_this_rank"] += stage2
        totals["post_step_replicate_broadcast_tensor_bytes_this_rank"] += stage2
        totals["owner_update_ring_bytes_per_rank"] += bucket_bytes
        totals["same_payload_allreduce_ring_bytes_per_rank"] += round(bucket_bytes * 2 * factor)
    loads = list(owner_numel.values())
    mean = sum(loads) / len(loads) if loads else 0.0
    totals["max_owner_bucket_bytes"] = max_bucket
    n_groups = sum(1 for _ in iter_groups(model))
    return {
        "available": True,
        "group_count": n_groups,
        "groups": groups,
        "groups_truncated": max(0, n_groups - max_groups),
        "data_plane": _data_plane(model),
        "totals": {k: int(v) for k, v in totals.items()},
        "owner_numel": {f"{s},{r}": int(v) for (s, r), v in sorted(owner_numel.items())},
        "owner_imbalance": (max(loads) - mean) / mean if mean > 0 else 0.0,
    }

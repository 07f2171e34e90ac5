"""Full (unsharded) state dicts for models and optimizers with dedicated
parameters.

Layouts (identical to the reference, dmuon/checkpoint.py:422-509, :597-756):

model      ``{fqn: full tensor}`` in each parameter's original dtype -- the
           same keys and shapes as the single-GPU ``model.state_dict()``
optimizer  ``{"fsdp":            {fqn: {"step", "exp_avg", "exp_avg_sq"}},
             "dedicated":       {fqn: {"momentum_buffer": (rows, rest) matrix}},
             "dedicated_adamw": {fqn: {"step", "exp_avg", "exp_avg_sq"}},
             "param_groups":    [group options without "params"]}``

Every rank takes part in the gathers; with ``rank0_only`` only rank 0 keeps the
tensors.  Asynchronous post-step publishes are drained before anything is
read.  Loading expects the same parallel layout the state was saved from.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .utils import get_dedicated_params, wait_all_replicate_broadcasts

try:
    from torch.distributed.tensor import DTensor, distribute_tensor
except Exception:  # pragma: no cover
    DTensor = None
    distribute_tensor = None


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _keep(t: torch.Tensor, cpu_offload: bool, rank0_only: bool) -> Optional[torch.Tensor]:
    if rank0_only and _rank() != 0:
        return None
    t = t.detach()
    # .cpu() of a CPU tensor is the tensor itself: always hand out a private copy
    return t.cpu() if (cpu_offload and t.device.type != "cpu") else t.clone()


def _bcast(t: torch.Tensor, group, src_local: int) -> None:
    if group is not None and group.size() > 1:
        dist.broadcast(t, src=dist.get_global_rank(group, src_local), group=group)


def _staged_broadcast(dp, value: Optional[torch.Tensor], shape, dtype, *, from_tp_owner: bool) -> torch.Tensor:
    """Bring a tensor that lives on the owner (optionally on the TP owner only)
    to every rank: TP group, then replicate axis, then shard axis."""
    buf = value.to(dtype).contiguous() if value is not None else torch.empty(shape, dtype=dtype, device=dp.device)
    if from_tp_owner and dp.tp_group is not None and dp.is_owner:
        _bcast(buf, dp.tp_group, dp._tp_owner_local_rank)
    if dp.in_owner_column:
        _bcast(buf, dp.replicate_group, dp.owner_replicate)
    _bcast(buf, dp.dp_group, dp.owner_shard)
    return buf


def _tp_assemble(dp, local: torch.Tensor) -> torch.Tensor:
    """Concatenate the TP shards of a tensor every TP peer holds a slice of."""
    if dp.tp_group is None or dp.tp_group.size() == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(dp.tp_group.size())]
    dist.all_gather(parts, local.contiguous(), group=dp.tp_group)
    return torch.cat(parts, dim=dp.shard_dim)


def _tp_slice(dp, full: torch.Tensor) -> torch.Tensor:
    if dp.tp_group is None:
        return full
    ext = dp._orig_size[dp.shard_dim]
    return full.narrow(dp.shard_dim, dp.tp_group.rank() * ext, ext)


def _full_dedicated_value(dp) -> torch.Tensor:
    """Current full-precision value of a dedicated parameter on every rank."""
    if dp._dmuon_route == "sharded_adamw":
        shard = dp._sharded_adamw_data
        if dp.shard_size > 1:
            full = torch.empty(shard.numel() * dp.shard_size, dtype=shard.dtype, device=shard.device)
            dist.all_gather_into_tensor(full, shard, group=dp.dp_group)
        else:
            full = shard
        local = full[: dp.numel].view(dp._orig_size)
    elif dp.mode == "ddp":
        local = dp._owned_data
    else:
        local = dp._owned_data if dp.in_owner_column else torch.empty(
            dp._orig_size, dtype=dp._master_dtype, device=dp.device
        )
        _bcast(local, dp.dp_group, dp.owner_shard)
    return _tp_assemble(dp, local)


def _full_plain(p: torch.Tensor) -> torch.Tensor:
    if DTensor is not None and isinstance(p, DTensor):
        return p.detach().full_tensor()
    return p.detach()


def _dedicated_by_ref(model: nn.Module) -> dict[int, Any]:
    out = {}
    for dp in get_dedicated_params(model):
        for ref in (dp._original_param, dp._placeholder, dp._unsharded_param):
            if ref is not None:
                out[id(ref)] = dp
    return out


# --------------------------------------------------------------------------- model
@torch.no_grad()
def get_model_state_dict(model: nn.Module, cpu_offload: bool = True, rank0_only: bool = True) -> dict[str, torch.Tensor]:
    wait_all_replicate_broadcasts(model)
    by_ref = _dedicated_by_ref(model)
    out: dict[str, torch.Tensor] = {}
    cache: dict[int, Optional[torch.Tensor]] = {}
    for name, p in model.named_parameters(remove_duplicate=False):
        dp = by_ref.get(id(p))
        key = id(dp) if dp is not None else id(p)
        if key not in cache:
            full = _full_dedicated_value(dp).to(dp._orig_dtype) if dp is not None else _full_plain(p)
            cache[key] = _keep(full, cpu_offload, rank0_only)
        if cache[key] is not None:
            out[name] = cache[key]
    for name, b in model.named_buffers(remove_duplicate=False):
        mod_name, _, leaf = name.rpartition(".")
        owner = model.get_submodule(mod_name) if mod_name else model
        if leaf in owner._non_persistent_buffers_set:
            continue
        kept = _keep(_full_plain(b), cpu_offload, rank0_only)
        if kept is not None:
            out[name] = kept
    return out


def _load_plain(p: torch.Tensor, full: torch.Tensor) -> None:
    if DTensor is not None and isinstance(p, DTensor):
        src = distribute_tensor(full.to(device=p._local_tensor.device, dtype=p.dtype), p.device_mesh, p.placements)
        p._local_tensor.copy_(src._local_tensor)
    else:
        p.copy_(full.to(device=p.device, dtype=p.dtype))


def _load_dedicated(dp, full: torch.Tensor) -> None:
    local = _tp_slice(dp, full.to(dp.device))
    if dp._dmuon_route == "sharded_adamw":
        per = dp._flat_shard_numel
        flat = local.reshape(-1)
        lo = min(dp.numel, dp.shard_rank * per)
        hi = min(dp.numel, lo + per)
        dp._sharded_adamw_data.zero_()
        dp._sharded_adamw_data[: hi - lo].copy_(flat[lo:hi])
        return
    if dp._owned_data is not None:
        dp._owned_data.copy_(local)
        dp._publish_fresh = False
    if dp._sharded_muon_data is not None:
        per = dp._flat_shard_numel
        flat = local.reshape(-1)
        lo = min(dp.numel, dp.shard_rank * per)
        hi = min(dp.numel, lo + per)
        dp._sharded_muon_data.zero_()
        dp._sharded_muon_data[: hi - lo].copy_(flat[lo:hi])
    if dp.mode == "ddp":
        dp.copy_owned_to_live()


@torch.no_grad()
def set_model_state_dict(
    model: nn.Module, state_dict: dict[str, torch.Tensor], strict: bool = True, broadcast_from_rank0: bool = False
) -> None:
    """Load a full state dict (for example one saved from a single GPU).  With
    ``broadcast_from_rank0`` only rank 0 needs to hold the tensors."""
    wait_all_replicate_broadcasts(model)
    by_ref = _dedicated_by_ref(model)
    done: set[int] = set()
    missing = []
    device = getattr(getattr(model, "_dedicated_comm_ctx", None), "device", torch.device("cpu"))

    bcast = broadcast_from_rank0 and _dist_on()
    present: Optional[dict[str, bool]] = None
    if bcast:
        # rank 0 tells everybody which names it holds, so that all ranks skip the same ones and no rank is
        # left waiting in a broadcast that rank 0 never enters
        names = [n for n, _ in model.named_parameters(remove_duplicate=False)]
        names += [n for n, _ in model.named_buffers(remove_duplicate=False)]
        mask = torch.tensor([1 if (_rank() == 0 and n in state_dict) else 0 for n in names], dtype=torch.int32,
                            device=device)
        dist.broadcast(mask, src=0)
        present = {n: bool(v) for n, v in zip(names, mask.tolist())}

    def fetch(name: str, shape, dtype) -> Optional[torch.Tensor]:
        if not bcast:
            return state_dict.get(name)
        if not present.get(name, False):
            return None
        t = state_dict[name].to(device=device, dtype=dtype) if _rank() == 0 else torch.empty(shape, dtype=dtype, device=device)
        dist.broadcast(t, src=0)
        return t

    for name, p in model.named_parameters(remove_duplicate=False):
        dp = by_ref.get(id(p))
        key = id(dp) if dp is not None else id(p)
        if key in done:
            continue
        shape = dp.full_shape if dp is not None else p.shape
        dtype = dp._orig_dtype if dp is not None else p.dtype
        full = fetch(name, shape, dtype)
        if full is None:
            missing.append(name)
            continue
        done.add(key)
        if dp is not None:
            _load_dedicated(dp, full)
        else:
            _load_plain(p, full)
    seen_buffers: set[int] = set()
    for name, b in model.named_buffers(remove_duplicate=False):
        if id(b) in seen_buffers:
            continue
        full = fetch(name, b.shape, b.dtype)
        if full is not None:
            seen_buffers.add(id(b))
            _load_plain(b, full)
    if strict and missing:
        raise KeyError(f"set_model_state_dict: missing keys {missing[:8]}")
    # peer data plane: readers hold pulled copies of the OLD weights; publish a new epoch
    # (every rank is inside this call, so the flag protocol lines up)
    rt = getattr(getattr(model, "_dedicated_comm_ctx", None), "peer_runtime", None)
    if rt is not None:
        rt.before_owner_writes()
        rt.publish_owned()


# --------------------------------------------------------------------------- optimizer
_GROUP_STRUCT_KEYS = ("use_muon", "group_name", "semantic_group_name", "subgroup_type")


def _plain_fqns(model: nn.Module, optimizer) -> dict[int, str]:
    ids = {id(p) for p in optimizer._plain_params}
    return {id(p): n for n, p in model.named_parameters() if id(p) in ids}


def _any_rank_has(flags: list[bool], device) -> list[bool]:
    """Element-wise OR over ranks of a list of booleans (one all-reduce)."""
    if not flags:
        return []
    t = torch.tensor([1 if f else 0 for f in flags], dtype=torch.int32, device=device)
    if _dist_on():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [bool(v) for v in t.tolist()]


def _full_like_param(p: torch.Tensor, local_state: torch.Tensor) -> torch.Tensor:
    if DTensor is not None and isinstance(p, DTensor):
        d = DTensor.from_local(
            local_state, device_mesh=p.device_mesh, placements=p.placements, run_check=False,
            shape=p.shape, stride=p.stride(),
        )
        return d.full_tensor()
    return local_state


@torch.no_grad()
def get_optimizer_state_dict(
    model: nn.Module, optimizer, cpu_offload: bool = True, rank0_only: bool = True
) -> dict[str, Any]:
    wait_all_replicate_broadcasts(model)
    device = optimizer.device
    dps = list(optimizer._all_dedicated)
    state = optimizer.state

    # Muon momentum: lives on the owner (TP owner for TP matrices), full-matrix shape
    muon = [dp for dp in dps if dp._dmuon_route == "muon"]
    have = _any_rank_has([("momentum_buffer" in state.get(id(dp), {})) for dp in muon], device)
    dedicated: dict[str, dict] = {}
    for dp, present in zip(muon, have):
        if not present:
            continue
        rows = int(dp.full_shape[0])
        shape = (rows, int(dp.full_shape.numel() // rows))
        holder = dp.is_owner and (dp.tp_group is None or dp.is_tp_owner)
        val = state[id(dp)]["momentum_buffer"].reshape(shape) if holder and "momentum_buffer" in state.get(id(dp), {}) else None
        buf = _staged_broadcast(dp, val, shape, torch.float32, from_tp_owner=True)
        kept = _keep(buf, cpu_offload, rank0_only)
        if kept is not None:
            dedicated[dp.fqn] = {"momentum_buffer": kept}

    # dedicated AdamW: on the owner (each TP peer holds its shard) or flat shards
    ad = [dp for dp in dps if dp._dmuon_route != "muon"]
    have = _any_rank_has([("exp_avg" in state.get(id(dp), {})) for dp in ad], device)
    dedicated_adamw: dict[str, dict] = {}
    for dp, present in zip(ad, have):
        if not present:
            continue
        st = state.get(id(dp), {})
        step = torch.tensor([int(st.get("step", 0))], dtype=torch.int64, device=device)
        if _dist_on():
            dist.all_reduce(step, op=dist.ReduceOp.MAX)
        entry: dict[str, Any] = {"step": int(step.item())}
        for key in ("exp_avg", "exp_avg_sq"):
            if dp._dmuon_route == "sharded_adamw":
                shard = st[key].float()
                full = torch.empty(shard.numel() * dp.shard_size, dtype=torch.float32, device=device)
                if dp.shard_size > 1:
                    dist.all_gather_into_tensor(full, shard.contiguous(), group=dp.dp_group)
                else:
                    full.copy_(shard)
                local = full[: dp.numel].view(dp._orig_size)
            else:
                val = st[key] if (dp.is_owner and key in st) else None
                local = _staged_broadcast(dp, val, dp._orig_size, torch.float32, from_tp_owner=False)
            kept = _keep(_tp_assemble(dp, local), cpu_offload, rank0_only)
            if kept is not None:
                entry[key] = kept
        if not rank0_only or _rank() == 0:
            dedicated_adamw[dp.fqn] = entry

    # AdamW of the non-dedicated parameters (FSDP2 shards or replicas)
    fqns = _plain_fqns(model, optimizer)
    fsdp: dict[str, dict] = {}
    for p in optimizer._plain_params:
        st = state.get(p, {})
        has = _any_rank_has(["exp_avg" in st], device)[0]
        if not has:
            continue
        entry = {"step": int(st.get("step", 0))}
        for key in ("exp_avg", "exp_avg_sq"):
            local = st[key] if key in st else torch.zeros_like(getattr(p, "_local_tensor", p), dtype=torch.float32)
            kept = _keep(_full_like_param(p, local), cpu_offload, rank0_only)
            if kept is not None:
                entry[key] = kept
        if not rank0_only or _rank() == 0:
            fsdp[fqns[id(p)]] = entry

    groups = [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
    if rank0_only and _rank() != 0:
        return {"fsdp": {}, "dedicated": {}, "dedicated_adamw": {}, "param_groups": groups}
    return {"fsdp": fsdp, "dedicated": dedicated, "dedicated_adamw": dedicated_adamw, "param_groups": groups}


def _shard_like_param(p: torch.Tensor, full: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if DTensor is not None and isinstance(p, DTensor):
        d = distribute_tensor(full.to(device=p._local_tensor.device, dtype=dtype), p.device_mesh, p.placements)
        return d._local_tensor.clone()
    return full.to(device=p.device, dtype=dtype).clone()


@torch.no_grad()
def set_optimizer_state_dict(model: nn.Module, optimizer, state_dict: dict[str, Any]) -> None:
    """Restore optimizer state saved by :func:`get_optimizer_state_dict`; every
    rank passes the full dict.  The param-group structure must match."""
    wait_all_replicate_broadcasts(model)
    saved = state_dict.get("param_groups", [])
    if len(saved) != len(optimizer.param_groups):
        raise ValueError(
            f"optimizer state has {len(saved)} param groups, the optimizer has {len(optimizer.param_groups)}"
        )
    for i, (sg, og) in enumerate(zip(saved, optimizer.param_groups)):
        for k in _GROUP_STRUCT_KEYS:
            if sg.get(k) != og.get(k):
                raise ValueError(f"param group {i}: structure key {k!r} differs ({sg.get(k)!r} vs {og.get(k)!r})")
        for k, v in sg.items():
            if k not in _GROUP_STRUCT_KEYS:
                og[k] = v
    state = optimizer.state
    by_fqn = {dp.fqn: dp for dp in optimizer._all_dedicated}
    for fqn, entry in state_dict.get("dedicated", {}).items():
        dp = by_fqn.get(fqn)
        if dp is None:
            raise KeyError(f"optimizer state names unknown dedicated parameter {fqn!r}")
        buf = entry["momentum_buffer"]
        if dp.is_owner and (dp.tp_group is None or dp.is_tp_owner):
            state[id(dp)]["momentum_buffer"] = buf.to(device=dp.device, dtype=dp._optim_dtype).clone()
        if dp.tp_group is not None and dp.is_owner:
            # this rank's part of the (rows, rest) momentum MATRIX, the shape the distributed-Gram step adds
            # its 2-D local gradient to (parameters with more than two dimensions included)
            rows = int(dp.full_shape[0])
            full = buf.to(dp.device).reshape(rows, -1)
            tp_rank, tp_size = dp.tp_group.rank(), dp.tp_group.size()
            if dp.shard_dim == 0:
                per = rows // tp_size
                local = full.narrow(0, tp_rank * per, per)
            else:
                per = full.shape[1] // tp_size
                local = full.narrow(1, tp_rank * per, per)
            state[id(dp)]["tp_local_momentum_buffer"] = local.to(dp._optim_dtype).contiguous().clone()
    for fqn, entry in state_dict.get("dedicated_adamw", {}).items():
        dp = by_fqn.get(fqn)
        if dp is None:
            raise KeyError(f"optimizer state names unknown dedicated parameter {fqn!r}")
        if not optimizer._updates_here(dp):
            continue
        st = state[id(dp)]
        st["step"] = int(entry["step"])
        for key in ("exp_avg", "exp_avg_sq"):
            local = _tp_slice(dp, entry[key].to(dp.device).view(dp.full_shape))
            if dp._dmuon_route == "sharded_adamw":
                per = dp._flat_shard_numel
                flat = local.reshape(-1)
                lo = min(dp.numel, dp.shard_rank * per)
                hi = min(dp.numel, lo + per)
                shard = torch.zeros(per, dtype=dp._optim_dtype, device=dp.device)
                shard[: hi - lo].copy_(flat[lo:hi])
                st[key] = shard
            else:
                st[key] = local.to(dp._optim_dtype).clone()
    plain = {n: p for n, p in model.named_parameters() if id(p) in {id(q) for q in optimizer._plain_params}}
    for fqn, entry in state_dict.get("fsdp", {}).items():
        p = plain.get(fqn)
        if p is None:
            raise KeyError(f"optimizer state names unknown parameter {fqn!r}")
        st = state[p]
        st["step"] = int(entry["step"])
        for key in ("exp_avg", "exp_avg_sq"):
            st[key] = _shard_like_param(p, entry[key], torch.float32)

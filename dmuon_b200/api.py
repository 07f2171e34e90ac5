"""Setup entry points: give every selected parameter one owner rank and wire
the model for dedicated-ownership training.

``dedicate_params`` is called BEFORE ``fully_shard``: it moves the selected
parameters out of FSDP2's sight (zero-size tagged placeholders), keeps a master
copy on the owner, and registers the publish/reduce hooks at per-layer
boundaries.  ``fully_shard`` then shards only what is left, and
``Muon(model, ...)`` finds everything through ``model._dedicated_comm_ctx``.

Signatures and return values match the reference (dmuon/api.py:392-416,
:754-950, :953-1137): the returned mapping is ``param -> owner`` with ints on a
1-D mesh and ``(shard, replicate)`` pairs when ``replicate_mesh`` is given.
"""
from __future__ import annotations

import logging
import os
from collections import defaultdict
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .parallel.comm import DedicatedCommContext
from .parallel.dgroup import DedicatedParamGroup, DedicatedParamGroupDDP
from .parallel.dparam import DedicatedParam
from .parallel.hooks import DedicatedState
from .parallel.partition import compute_balanced_assignment, imbalance
from .parallel.topology import (
    get_tp_mesh,
    get_tp_shard_dim,
    is_tp_sharded,
    maybe_isolate_process_group,
    normalize_owner_rank,
    resolve_process_group_policy,
)
from .policy import resolve_param_policies

log = logging.getLogger(__name__)


# --------------------------------------------------------------------------- env helpers
def _env_bool(name: str, default: bool) -> bool:
    raw = os.environ.get(name)
    if raw is None or raw == "":
        return default
    key = raw.strip().lower()
    if key in ("1", "true", "yes", "on"):
        return True
    if key in ("0", "false", "no", "off"):
        return False
    raise ValueError(f"{name} must be a boolean flag, got {raw!r}")


def _pick(value, env: str, default: str, allowed: tuple[str, ...], what: str) -> str:
    out = value or os.environ.get(env, default)
    if out not in allowed:
        raise ValueError(f"Unsupported {what}: {out!r}; expected one of {allowed}.")
    return out


# --------------------------------------------------------------------------- model index
class _ModelIndex:
    """Parameter -> (module, attribute) sites and module -> dotted name, built
    in one walk so setup stays linear in model size."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.module_fqn: dict[int, str] = {}
        self.sites: dict[int, list[tuple[nn.Module, str]]] = defaultdict(list)
        self.site_fqns: dict[int, list[str]] = defaultdict(list)
        self.module_order: dict[int, int] = {}
        for i, (mname, mod) in enumerate(model.named_modules()):
            self.module_fqn[id(mod)] = mname
            self.module_order[id(mod)] = i
            for pname, p in mod.named_parameters(recurse=False):
                self.sites[id(p)].append((mod, pname))
                self.site_fqns[id(p)].append(f"{mname}.{pname}" if mname else pname)

    def parent(self, p: nn.Parameter) -> tuple[nn.Module, str]:
        sites = self.sites.get(id(p))
        if not sites:
            raise ValueError(f"Parameter not found in model: {tuple(p.shape)}")
        return sites[0]

    def ancestors(self, module: nn.Module):
        """``module`` and its ancestors, innermost first."""
        parts = self.module_fqn[id(module)].split(".") if self.module_fqn[id(module)] else []
        for depth in range(len(parts), -1, -1):
            path = ".".join(parts[:depth])
            yield self.model.get_submodule(path) if path else self.model

    def layer_module(self, p: nn.Parameter) -> nn.Module:
        """The ``layers.N`` / ``blocks.N`` / ``h.N`` / ``layer.N`` ancestor (the
        usual names of a model's repeated block list), else the direct parent."""
        parent, _ = self.parent(p)
        fqn = self.module_fqn[id(parent)]
        parts = fqn.split(".") if fqn else []
        for i in range(len(parts) - 1):
            if parts[i] in ("layers", "blocks", "h", "layer") and parts[i + 1].isdigit():
                try:
                    return self.model.get_submodule(".".join(parts[: i + 2]))
                except AttributeError:
                    break
        return parent

    def common_ancestor(self, modules: list[nn.Module]) -> nn.Module:
        paths = [self.module_fqn[id(m)].split(".") if self.module_fqn[id(m)] else [] for m in modules]
        common: list[str] = []
        for col in zip(*paths):
            if all(c == col[0] for c in col):
                common.append(col[0])
            else:
                break
        # a pure container (ModuleList, ModuleDict, ...) is never called, so hooks on it
        # would never fire: climb to the first ancestor that has a forward of its own
        while common:
            mod = self.model.get_submodule(".".join(common))
            if type(mod).forward is not nn.Module.forward:
                return mod
            common.pop()
        return self.model


def _resolve_hook_module(index: _ModelIndex, p, fqn, predicate, resolver, strict) -> nn.Module:
    if resolver is not None:
        mod = resolver(fqn, p)
        if mod is not None:
            return mod
        if strict:
            raise ValueError(
                f"{fqn}: hook_boundary_resolver returned None. Extend the resolver to cover this "
                "parameter or exclude it via the dedicate_params predicate."
            )
        return index.parent(p)[0]
    if predicate is not None:
        parent = index.parent(p)[0]
        for mod in index.ancestors(parent):
            if predicate(mod):
                return mod
        if strict:
            raise ValueError(
                f"{fqn}: no ancestor matched hook_boundary_predicate. Extend the predicate to cover "
                "this module, or exclude the param via the dedicate_params `predicate` arg."
            )
        return parent
    return index.layer_module(p)


def _check_activation_casts(groups: dict, index: _ModelIndex) -> None:
    """Two groups on one module that both cast activations must agree."""
    per_module: dict[int, list] = defaultdict(list)
    for (module, _key), dparams in groups.items():
        per_module[id(module)].append((module, dparams[0]))
    for entries in per_module.values():
        in_casts = {d._param_dtype for _, d in entries if d._cast_forward_inputs}
        out_casts = {d._output_dtype for _, d in entries if d._output_dtype is not None}
        if len(in_casts) > 1 or len(out_casts) > 1:
            name = index.module_fqn[id(entries[0][0])] or "<root>"
            raise ValueError(
                f"hook boundary {name!r} has parameter policies with conflicting activation casts "
                f"(inputs {sorted(map(str, in_casts))}, outputs {sorted(map(str, out_casts))}); "
                "give them separate hook boundaries or one activation dtype"
            )


def _link_forward_order(index: _ModelIndex, states: list[DedicatedState], ctx: DedicatedCommContext) -> None:
    ordered = sorted(states, key=lambda s: index.module_order.get(id(s.module), 1 << 30))
    for i, st in enumerate(ordered):
        st.next_states = ordered[i + 1 :]
        st.group.next_forward_groups = [s.group for s in ordered[i + 1 :]]
    ctx.all_states[:] = ordered


def _log_balance(assignment, params, names, n_shard, n_rep, what: str) -> None:
    loads: dict = defaultdict(int)
    for p in params:
        loads[normalize_owner_rank(assignment[p])] += int(p.numel())
    vec = [loads.get((s, r), 0) for s in range(n_shard) for r in range(n_rep)]
    log.info(
        "%s: %d parameters over %d owner slots, %d allocation units (%d packed), "
        "load min/max %.1fM/%.1fM elements, imbalance %.1f%%",
        what,
        len(params),
        len(vec),
        assignment.allocation_unit_count,
        assignment.packed_allocation_unit_count,
        min(vec) / 1e6,
        max(vec) / 1e6,
        100.0 * imbalance(vec),
    )


def _device_of(model: nn.Module) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _dp_dim_names(mesh, replicate_mesh) -> frozenset:
    names = set(mesh.mesh_dim_names or ())
    if replicate_mesh is not None:
        names |= set(replicate_mesh.mesh_dim_names or ())
    return frozenset(names)


# --------------------------------------------------------------------------- single-node HSDP on the peer plane
class _FlatMesh:
    """Stand-in for a 1-D mesh over every rank of a replicate x shard grid."""

    def __init__(self, size: int, dim_names: tuple):
        self._size, self.mesh_dim_names = int(size), tuple(dim_names)

    def size(self) -> int:
        return self._size

    def get_group(self):
        return dist.group.WORLD


def _maybe_flatten_hsdp(model, mesh, replicate_mesh, predicate, comm_backend, policy_kwargs) -> Optional[_FlatMesh]:
    """On one NVSwitch domain the two axes of an HSDP grid are the same kind of
    link, so dedicated ownership can treat the grid as ONE data-parallel axis:
    every rank writes its gradients into its arena, the owner gathers from all
    R x S peers and averages once (= the two-stage mean), and every rank pulls
    the published weights from the owner.  That is exactly the 1-D peer data
    plane over the flattened group, so this returns a flat mesh when the peer
    plane can take the job (all ranks of the job, at most 8, on one host, no
    tensor parallelism, no sharded routes) and None otherwise (collective
    two-stage implementation).  FSDP2 keeps its own 2-D mesh for everything
    that is not dedicated."""
    from .parallel import peer as peer_mod

    want = (comm_backend or peer_mod.peer_backend_requested()).lower()
    if want not in ("auto", "peer") or not (dist.is_available() and dist.is_initialized()):
        return None
    if _device_of(model).type != "cuda":
        return None
    world = dist.get_world_size()
    if world != mesh.size() * replicate_mesh.size() or world > peer_mod.MAX_PEERS:
        return None
    if int(os.environ.get("LOCAL_WORLD_SIZE", str(torch.cuda.device_count()))) < world:
        return None           # the grid spans hosts: the replicate axis is not NVLink
    dp_dims = _dp_dim_names(mesh, replicate_mesh)
    cand, names = [], {}
    seen: set[int] = set()
    for name, p in model.named_parameters():
        if id(p) not in seen and predicate(name, p):
            seen.add(id(p))
            cand.append(p)
            names[p] = name
    if not cand or any(is_tp_sharded(p, dp_dims) for p in cand):
        return None
    pols = resolve_param_policies(params=cand, param_to_fqn=names, **policy_kwargs)
    for p in cand:
        pol = pols[p]
        if (pol.route or "") == "sharded_adamw" or (pol.muon_forward_unshard or "broadcast") != "broadcast":
            return None
    return _FlatMesh(world, tuple(dp_dims))


# --------------------------------------------------------------------------- shared setup
def _setup(
    model,
    mesh,
    predicate,
    *,
    mode: str,
    compute_dtype=None,
    reshard_after_forward=True,
    replicate_mesh=None,
    hook_boundary_predicate=None,
    hook_boundary_strict=True,
    hook_boundary_resolver=None,
    assignment_group_key_fn=None,
    route_hint_fn=None,
    max_owners_per_group=None,
    owner_strategy=None,
    owner_cost_model=None,
    hsdp_column_balance=None,
    pack_small_params=None,
    tp_buffer_reuse=False,
    replicate_broadcast_bucket_mb=0.0,
    muon_forward_unshard="broadcast",
    delay_stage2_to_optimizer=True,
    param_policy=None,
    param_policy_fn=None,
    process_group_policy=None,
    allow_tp=True,
    comm_backend=None,
):
    owner_strategy = _pick(owner_strategy, "DMUON_OWNER_STRATEGY", "lpt", ("lpt", "round_robin", "rank0"), "owner_strategy")
    owner_cost_model = _pick(owner_cost_model, "DMUON_OWNER_COST_MODEL", "optimizer", ("optimizer", "numel"), "owner_cost_model")
    if hsdp_column_balance is None:
        hsdp_column_balance = _env_bool("DMUON_HSDP_COLUMN_BALANCE", True)
    if pack_small_params is None:
        pack_small_params = _env_bool("DMUON_OWNER_PACK_SMALL_PARAMS", True)
    pg_policy = resolve_process_group_policy(process_group_policy)
    if muon_forward_unshard not in ("broadcast", "all_gather"):
        raise ValueError("muon_forward_unshard must be 'broadcast' or 'all_gather'")

    # single-node HSDP: one flattened ownership axis on the peer plane when possible
    hsdp_coords = None
    user_mesh, user_replicate_mesh = mesh, replicate_mesh
    if mode == "fsdp" and replicate_mesh is not None and replicate_mesh.size() > 1:
        flat = _maybe_flatten_hsdp(
            model, mesh, replicate_mesh, predicate, comm_backend,
            dict(compute_dtype=compute_dtype, route_hint_fn=route_hint_fn, param_policy=param_policy,
                 param_policy_fn=param_policy_fn, default_muon_forward_unshard=muon_forward_unshard),
        )
        if flat is not None:
            hsdp_coords = [None] * dist.get_world_size()
            dist.all_gather_object(hsdp_coords, (mesh.get_local_rank(), replicate_mesh.get_local_rank()))
            mesh, replicate_mesh = flat, None

    assignment = compute_balanced_assignment(
        model,
        mesh,
        predicate,
        replicate_mesh=replicate_mesh,
        owner_strategy=owner_strategy,
        assignment_group_key_fn=assignment_group_key_fn,
        max_owners_per_group=max_owners_per_group,
        owner_cost_model=owner_cost_model,
        hsdp_column_balance=hsdp_column_balance,
        pack_small_params=pack_small_params,
    )
    index = _ModelIndex(model)
    selected: list[nn.Parameter] = []
    fqn_of: dict = {}
    seen: set[int] = set()
    for name, p in model.named_parameters():
        if p in assignment and id(p) not in seen:
            seen.add(id(p))
            selected.append(p)
            fqn_of[p] = name
    if not selected:
        raise ValueError("dedicate_params: the predicate selected no parameter")
    n_shard = mesh.size()
    n_rep = replicate_mesh.size() if replicate_mesh is not None else 1
    _log_balance(assignment, selected, fqn_of, n_shard, n_rep, f"dedicate_params[{mode}]")

    dp_dims = _dp_dim_names(user_mesh, user_replicate_mesh)
    if not allow_tp:
        bad = [fqn_of[p] for p in selected if is_tp_sharded(p, dp_dims)]
        if bad:
            raise ValueError(
                f"dedicate_params_ddp does not take tensor-parallel parameters ({bad[:3]}...); "
                "use dedicate_params_ddp_tp"
            )

    for p in selected:
        p._dedicated_owner_rank = assignment[p]

    dp_group = maybe_isolate_process_group(mesh.get_group(), policy=pg_policy, role="dp")
    rep_group = None
    if replicate_mesh is not None:
        rep_group = maybe_isolate_process_group(replicate_mesh.get_group(), policy=pg_policy, role="replicate")
    tp_groups: dict[int, object] = {}

    device = _device_of(model)
    ctx = DedicatedCommContext(
        device,
        replicate_group=rep_group,
        tp_buffer_reuse=tp_buffer_reuse,
        replicate_broadcast_bucket_mb=replicate_broadcast_bucket_mb,
    )
    ctx.dp_group = dp_group
    ctx.mode = mode
    ctx.process_group_policy = pg_policy

    policies = resolve_param_policies(
        params=selected,
        param_to_fqn=fqn_of,
        compute_dtype=compute_dtype,
        route_hint_fn=route_hint_fn,
        param_policy=param_policy,
        param_policy_fn=param_policy_fn,
        default_muon_forward_unshard=muon_forward_unshard,
    )

    # Replicated placement on one NVSwitch domain: the dedicated matrices take the peer-memory plane in
    # its FSDP form (bf16 copies in every rank's publish arena, masters and momentum on the owner only, the
    # owner's update stored to all ranks, gradients reduced from the arenas); ``replicate`` keeps averaging
    # the other parameters.  What a replicated placement promises -- every rank holds the whole weight for
    # forward and backward, one owner updates it -- holds unchanged; the fp32 post-step broadcast
    # (reference dmuon/_backends/ddp/group.py:565-603) has nothing left to send.
    ddp_on_peer = False
    if mode == "ddp":
        from .parallel import peer as peer_mod0

        want0 = (comm_backend or peer_mod0.peer_backend_requested()).lower()
        if want0 in ("auto", "peer"):
            why0 = peer_mod0.peer_backend_possible_from_policies(
                device, dp_group, rep_group, selected, policies, lambda q: is_tp_sharded(q, dp_dims))
            if why0 is None:
                ddp_on_peer, mode, reshard_after_forward = True, "fsdp", False
            elif want0 == "peer":
                raise RuntimeError(f"comm_backend='peer' is not possible here: {why0}")

    grouped: dict[tuple, list[DedicatedParam]] = defaultdict(list)
    for p in selected:
        sites = index.sites[id(p)]
        fqn = fqn_of[p]
        hook_mod = _resolve_hook_module(
            index, p, fqn, hook_boundary_predicate, hook_boundary_resolver, hook_boundary_strict
        )
        if len(sites) > 1 and mode == "fsdp" and reshard_after_forward:
            # a tied parameter is read at several places: the boundary has to
            # span all of them when the published copy is dropped after forward
            hook_mod = index.common_ancestor([hook_mod] + [m for m, _ in sites])
        tp_group = None
        tp_owner = 0
        tp_dim = None
        if is_tp_sharded(p, dp_dims):
            tp_mesh = get_tp_mesh(p, dp_dims)
            raw = tp_mesh.get_group()
            tp_group = tp_groups.get(id(raw))
            if tp_group is None:
                tp_group = maybe_isolate_process_group(raw, policy=pg_policy, role="tp")
                tp_groups[id(raw)] = tp_group
            tp_owner = assignment.tp_owners.get(p, 0)
            tp_dim = get_tp_shard_dim(p, dp_dims)
        dparam = DedicatedParam(
            p,
            sites[0][0],
            sites[0][1],
            assignment[p],
            dp_group,
            device,
            policy=policies[p],
            replicate_group=rep_group,
            tp_group=tp_group,
            tp_owner_local_rank=tp_owner,
            tp_shard_dim=tp_dim,
            fqn=fqn,
            mode=mode,
            alias_sites=sites,
        )
        dparam.alias_fqns = list(index.site_fqns[id(p)])
        grouped[(hook_mod, policies[p].group_key())].append(dparam)

    _check_activation_casts(grouped, index)

    states: list[DedicatedState] = []
    group_cls = DedicatedParamGroup if mode == "fsdp" else DedicatedParamGroupDDP
    # data plane: peer-memory kernels where the placement allows it, else collectives
    from .parallel import peer as peer_mod

    want = (comm_backend or peer_mod.peer_backend_requested()).lower()
    if want not in ("auto", "peer", "nccl", "collective"):
        raise ValueError(f"comm_backend must be 'auto', 'peer' or 'nccl', got {want!r}")
    use_peer = False
    if mode == "fsdp" and want in ("auto", "peer"):
        why_not = peer_mod.peer_backend_possible(device, dp_group, rep_group, [d for v in grouped.values() for d in v])
        if why_not is None:
            use_peer = True
        elif want == "peer":
            raise RuntimeError(f"comm_backend='peer' is not possible here: {why_not}")
        else:
            log.info("dedicate_params: collective data plane (%s)", why_not)
    if use_peer:
        group_cls = peer_mod.PeerParamGroup
    for (hook_mod, _key), dparams in grouped.items():
        gname = index.module_fqn.get(id(hook_mod), "") or type(hook_mod).__name__
        group = group_cls(
            dparams,
            hook_mod,
            ctx,
            dp_group,
            reshard_after_forward=reshard_after_forward,
            name=gname,
            delay_stage2_to_optimizer=delay_stage2_to_optimizer,
        )
        states.append(DedicatedState(hook_mod, group, ctx))
    _link_forward_order(index, states, ctx)
    ctx.peer_runtime = None
    if use_peer:
        ctx.peer_runtime = peer_mod.PeerRuntime(ctx, dp_group, [st.group for st in ctx.all_states])
    model._dedicated_comm_ctx = ctx
    # tensor-parallel gather / scatter over peer memory, one exchange per TP group (all its ranks are here)
    ctx.tp_exchanges = {}
    if tp_groups and want != "nccl" and want != "collective":
        from .parallel import tp_peer as tp_peer_mod

        if tp_peer_mod.tp_peer_requested():
            all_dparams = [d for st in ctx.all_states for d in st.group.params]
            for tpg in tp_groups.values():
                why_not = tp_peer_mod.tp_peer_possible(device, tpg)
                if why_not is None:
                    mine = [d for d in all_dparams if d.tp_group is tpg]
                    ctx.tp_exchanges[id(tpg)] = tp_peer_mod.TPPeerExchange(ctx, tpg, mine)
                else:
                    log.info("dedicate_params: collective tensor-parallel gather/scatter (%s)", why_not)
    ctx.ddp_on_peer_plane = ddp_on_peer
    if ddp_on_peer:
        ctx.mode = "ddp"
        for st in ctx.all_states:
            for dpar in st.group.params:
                dpar._unsharded_param._dedicated_mode = "ddp"
                dpar._placeholder._dedicated_mode = "ddp"
    ctx.tp_groups = list(tp_groups.values())
    ctx.hsdp_flattened = hsdp_coords is not None
    if hsdp_coords is not None:
        # the caller asked for a replicate x shard grid: report owners as (shard, replicate) coordinates
        return {p: tuple(hsdp_coords[int(o)]) for p, o in assignment.dp_owners.items()}
    return dict(assignment.dp_owners)


# --------------------------------------------------------------------------- public API
def dedicate_params(
    model: nn.Module,
    mesh,
    predicate: Callable[[str, nn.Parameter], bool],
    compute_dtype: Optional[torch.dtype] = None,
    reshard_after_forward: bool = True,
    replicate_mesh=None,
    hook_boundary_predicate: Optional[Callable[[nn.Module], bool]] = None,
    hook_boundary_strict: bool = True,
    hook_boundary_resolver: Optional[Callable[[str, nn.Parameter], Optional[nn.Module]]] = None,
    assignment_group_key_fn: Optional[Callable[[str, nn.Parameter], Optional[str]]] = None,
    route_hint_fn: Optional[Callable[[str, nn.Parameter], Optional[str]]] = None,
    max_owners_per_group: Optional[int] = None,
    owner_strategy: Optional[str] = None,
    owner_cost_model: Optional[str] = None,
    hsdp_column_balance: Optional[bool] = None,
    pack_small_params: Optional[bool] = None,
    tp_buffer_reuse: bool | str = False,
    replicate_broadcast_bucket_mb: float = 0.0,
    muon_forward_unshard: str = "broadcast",
    delay_stage2_to_optimizer: bool = True,
    param_policy=None,
    param_policy_fn=None,
    process_group_policy: Optional[str] = None,
    comm_backend: Optional[str] = None,
) -> dict:
    """Dedicated ownership on top of FSDP2 (call before ``fully_shard``).

    ``reshard_after_forward=True`` drops the published copy after forward and
    publishes again for backward (three transfers of the dedicated parameters
    per step); ``False`` keeps it until backward is done (two transfers, more
    memory).  With ``replicate_mesh`` the owner is a ``(shard, replicate)``
    coordinate: gradients are averaged over the shard axis, then the replicate
    axis, and the owner's update is copied to the other replicate rows after
    the step.

    ``comm_backend`` (not in the reference): ``"peer"`` moves dedicated data with
    peer-memory kernels over NVLink (one shard axis of at most 8 GPUs, no tensor
    parallelism), ``"nccl"`` uses collectives, ``"auto"`` (default, also
    ``DMUON_COMM_BACKEND``) picks peer memory where it is possible.
    """
    if getattr(mesh, "ndim", 1) != 1 or (replicate_mesh is not None and getattr(replicate_mesh, "ndim", 1) != 1):
        raise ValueError("dedicate_params expects 1-D meshes for the shard and the replicate axis")
    return _setup(
        model,
        mesh,
        predicate,
        mode="fsdp",
        compute_dtype=compute_dtype,
        reshard_after_forward=reshard_after_forward,
        replicate_mesh=replicate_mesh,
        hook_boundary_predicate=hook_boundary_predicate,
        hook_boundary_strict=hook_boundary_strict,
        hook_boundary_resolver=hook_boundary_resolver,
        assignment_group_key_fn=assignment_group_key_fn,
        route_hint_fn=route_hint_fn,
        max_owners_per_group=max_owners_per_group,
        owner_strategy=owner_strategy,
        owner_cost_model=owner_cost_model,
        hsdp_column_balance=hsdp_column_balance,
        pack_small_params=pack_small_params,
        tp_buffer_reuse=tp_buffer_reuse,
        replicate_broadcast_bucket_mb=replicate_broadcast_bucket_mb,
        muon_forward_unshard=muon_forward_unshard,
        delay_stage2_to_optimizer=delay_stage2_to_optimizer,
        param_policy=param_policy,
        param_policy_fn=param_policy_fn,
        process_group_policy=process_group_policy,
        comm_backend=comm_backend,
    )


def dedicate_params_ddp(
    model: nn.Module,
    mesh,
    predicate: Callable[[str, nn.Parameter], bool],
    compute_dtype: Optional[torch.dtype] = None,
    hook_boundary_predicate=None,
    hook_boundary_strict: bool = True,
    hook_boundary_resolver=None,
    assignment_group_key_fn=None,
    max_owners_per_group: Optional[int] = None,
    owner_strategy: Optional[str] = None,
    owner_cost_model: Optional[str] = None,
    pack_small_params: Optional[bool] = None,
    param_policy=None,
    param_policy_fn=None,
    process_group_policy: Optional[str] = None,
    comm_backend: Optional[str] = None,
    route_hint_fn=None,
) -> dict:
    """Replicated (DDP-style) placement: every rank keeps the live parameter,
    gradients are reduced to the owner, the owner's update is broadcast after
    the step.  Use together with :func:`replicate` for the other parameters.

    ``comm_backend`` (``auto`` / ``peer`` / ``nccl``, default from
    ``DMUON_COMM_BACKEND``): on one NVSwitch domain the dedicated matrices use
    the peer-memory data plane -- every rank holds the bf16 weights in its
    publish arena, the owner's update kernel stores the new weights to all of
    them and gradients are reduced out of the ranks' arenas -- instead of NCCL
    reduce / broadcast."""
    if getattr(mesh, "ndim", 1) != 1:
        raise ValueError("dedicate_params_ddp expects a 1-D data-parallel mesh")
    return _setup(
        model,
        mesh,
        predicate,
        mode="ddp",
        compute_dtype=compute_dtype,
        reshard_after_forward=False,
        hook_boundary_predicate=hook_boundary_predicate,
        hook_boundary_strict=hook_boundary_strict,
        hook_boundary_resolver=hook_boundary_resolver,
        assignment_group_key_fn=assignment_group_key_fn,
        route_hint_fn=route_hint_fn,
        max_owners_per_group=max_owners_per_group,
        owner_strategy=owner_strategy,
        owner_cost_model=owner_cost_model,
        pack_small_params=pack_small_params,
        param_policy=param_policy,
        param_policy_fn=param_policy_fn,
        process_group_policy=process_group_policy,
        allow_tp=False,
        comm_backend=comm_backend,
    )


def dedicate_params_ddp_tp(
    model: nn.Module,
    mesh,
    predicate: Callable[[str, nn.Parameter], bool],
    compute_dtype: Optional[torch.dtype] = None,
    hook_boundary_predicate=None,
    hook_boundary_strict: bool = True,
    hook_boundary_resolver=None,
    assignment_group_key_fn=None,
    max_owners_per_group: Optional[int] = None,
    owner_strategy: Optional[str] = None,
    owner_cost_model: Optional[str] = None,
    pack_small_params: Optional[bool] = None,
    tp_buffer_reuse: bool | str = False,
    param_policy=None,
    param_policy_fn=None,
    process_group_policy: Optional[str] = None,
    route_hint_fn=None,
) -> dict:
    """Replicated placement for models whose matrices are DTensors sharded on a
    tensor-parallel mesh dimension (``mesh`` is the data-parallel dimension)."""
    if getattr(mesh, "ndim", 1) != 1:
        raise ValueError("dedicate_params_ddp_tp expects the 1-D data-parallel sub-mesh")
    out = _setup(
        model,
        mesh,
        predicate,
        mode="ddp",
        compute_dtype=compute_dtype,
        reshard_after_forward=False,
        hook_boundary_predicate=hook_boundary_predicate,
        hook_boundary_strict=hook_boundary_strict,
        hook_boundary_resolver=hook_boundary_resolver,
        assignment_group_key_fn=assignment_group_key_fn,
        route_hint_fn=route_hint_fn,
        max_owners_per_group=max_owners_per_group,
        owner_strategy=owner_strategy,
        owner_cost_model=owner_cost_model,
        pack_small_params=pack_small_params,
        tp_buffer_reuse=tp_buffer_reuse,
        param_policy=param_policy,
        param_policy_fn=param_policy_fn,
        process_group_policy=process_group_policy,
    )
    for st in model._dedicated_comm_ctx.all_states:
        for p in st.group.params:
            p._unsharded_param._dedicated_mode = "ddp_tp"
    model._dedicated_comm_ctx.mode = "ddp_tp"
    return out

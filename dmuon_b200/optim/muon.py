"""Muon for dedicated matrices, AdamW for everything else.

``Muon(model, lr, ns_steps, adamw_lr, ...)`` finds the dedicated parameters
through ``model._dedicated_comm_ctx`` and the remaining ones through
``model.parameters()`` (FSDP2 shards or replicated tensors).  Each rank updates
only what it owns:

* owned matrices on the ``muon`` route: momentum, Nesterov, Newton-Schulz and
  the scaled update ``W <- (1 - lr wd) W - lr 0.2 sqrt(max(m, n)) NS(u)``.  On a
  B200 all owned matrices of one shape go through the tcgen05 kernels as one
  batch and the last product writes the fp32 master weights directly;
* owned tensors on the ``adamw`` / ``sharded_adamw`` routes and all
  non-dedicated parameters: AdamW with per-tensor step counts, one fused
  multi-tensor launch per dtype combination on a GPU.

Constructor arguments, per-group keys, group names (``<name>/muon``,
``<name>/adamw``) and the update rules follow the reference
(dmuon/optim/muon.py:127-153, :473-510, :598-638, :1674-1740, :1862-1916).

``group_prepare_ahead`` (default on) pipelines the step over blocks of
communication groups whenever something travels after the update (replicate-axis
publish, tensor-parallel scatter, DDP broadcast): the next block's gradient
waits and tensor-parallel gathers are queued before the current block's
Newton-Schulz products, and each block's publish is dispatched as soon as the
block is updated (``DMUON_GROUP_PIPELINE_BLOCKS``, default 4; the reference
pipelines per group, dmuon/optim/muon.py:1446-1546).  Results are bit-identical
to the unpipelined order.  ``post_step_prefetch_groups``,
``forward_prefetch_depth``, ``replicate_async`` and the ``tp_distributed_gram*``
arguments do what their names say.  Accepted for signature parity only:
``post_step_prefetch_sharded_adamw`` and
``sharded_adamw_unshard_separate_stream`` (sharded-AdamW all-gathers share the
publish lane).
"""
from __future__ import annotations

import logging
import math
import os
import time
from collections import defaultdict
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..policy import normalize_route
from ..utils import (
    fence_isolated_process_groups,
    iter_groups,
    prepare_group_muon_grads,
    prepare_muon_grads,
    wait_group_muon_grads,
)
from .newton_schulz import NewtonSchulz, apply_gram_factors, gram_newton_schulz_factors

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None

log = logging.getLogger(__name__)

_ROUTE_KEYS = ("dmuon_route", "dmuon_optimizer", "matrix_optimizer")


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if DTensor is not None and isinstance(t, DTensor) else t


def muon_update_scale(shape) -> float:
    rows = int(shape[0])
    cols = int(math.prod(shape[1:])) if len(shape) > 1 else 1
    return 0.2 * math.sqrt(max(rows, cols))


class _StepProfile:
    """Per-phase timers of one optimizer step (CUDA events on a GPU, host
    clock on CPU); read back lazily so recording never forces a sync."""

    def __init__(self, device: torch.device, enabled: bool):
        self.device, self.enabled = device, enabled
        self.records: list[tuple[str, Any, Any]] = []

    def phase(self, name: str):
        return _Phase(self, name)

    def summary(self) -> dict[str, float]:
        out: dict[str, float] = defaultdict(float)
        for name, a, b in self.records:
            if isinstance(a, float):
                out[f"{name}_ms"] += (b - a) * 1e3
            else:
                b.synchronize()
                out[f"{name}_ms"] += a.elapsed_time(b)
        return dict(out)


class _Phase:
    def __init__(self, prof: _StepProfile, name: str):
        self.prof, self.name = prof, name

    def __enter__(self):
        if self.prof.enabled:
            if self.prof.device.type == "cuda":
                self.a = torch.cuda.Event(enable_timing=True)
                self.a.record()
            else:
                self.a = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.prof.enabled:
            if self.prof.device.type == "cuda":
                b = torch.cuda.Event(enable_timing=True)
                b.record()
            else:
                b = time.perf_counter()
            self.prof.records.append((self.name, self.a, b))
        return False


class Muon(torch.optim.Optimizer):
    def __init__(
        self,
        model: nn.Module,
        lr: float = 0.02,
        momentum: float = 0.95,
        weight_decay: float = 0.0,
        ns_steps: int = 5,
        adamw_lr: float = 1e-3,
        adamw_betas: tuple[float, float] = (0.9, 0.999),
        adamw_weight_decay: float = 0.01,
        adamw_eps: float = 1e-8,
        param_groups: Optional[list[dict]] = None,
        ns_backend: str | NewtonSchulz = "gram",
        nesterov: bool = True,
        replicate_async: bool = True,
        record_step_profile: bool = False,
        group_prepare_ahead: bool = True,
        tp_distributed_gram: bool = False,
        tp_distributed_gram_policy: str = "beneficial",
        tp_distributed_gram_max_factor_to_scatter_ratio: float = 0.5,
        post_step_prefetch_groups: int = 0,
        post_step_prefetch_sharded_adamw: bool = False,
        sharded_adamw_unshard_separate_stream: bool = False,
        forward_prefetch_depth: int = 1,
        first_step_progress_log: bool = True,
        first_step_progress_log_limit: int = 8,
    ):
        ctx = getattr(model, "_dedicated_comm_ctx", None)
        if ctx is None:
            raise RuntimeError(
                "Muon needs a model prepared with dedicate_params (or dedicate_params_ddp / "
                "dedicate_params_ddp_tp): model._dedicated_comm_ctx is missing"
            )
        self.model = model
        self.comm_ctx = ctx
        self.device = ctx.device
        self.ns = ns_backend if isinstance(ns_backend, NewtonSchulz) else NewtonSchulz(backend=str(ns_backend))
        self.ns_steps = int(ns_steps)
        self.nesterov = bool(nesterov)
        self.replicate_async = bool(replicate_async)
        self.record_step_profile = bool(record_step_profile)
        self.group_prepare_ahead = bool(group_prepare_ahead)
        self.tp_distributed_gram = bool(tp_distributed_gram)
        self.tp_distributed_gram_policy = tp_distributed_gram_policy
        self.tp_distributed_gram_max_factor_to_scatter_ratio = float(tp_distributed_gram_max_factor_to_scatter_ratio)
        self.post_step_prefetch_groups = int(post_step_prefetch_groups)
        self.post_step_prefetch_sharded_adamw = bool(post_step_prefetch_sharded_adamw)
        self.first_step_progress_log = bool(first_step_progress_log)
        self.first_step_progress_log_limit = int(first_step_progress_log_limit)
        ctx.forward_prefetch_depth = int(forward_prefetch_depth)
        ctx.sharded_adamw_unshard_separate_stream_enabled = bool(sharded_adamw_unshard_separate_stream)

        self._comm_groups = list(iter_groups(model))
        self._all_dedicated = [p for g in self._comm_groups for p in g.params]
        self._has_tp = any(p.tp_group is not None for p in self._all_dedicated)
        self._plain_params = self._collect_plain_params(model)
        self._dummy_params: list[nn.Parameter] = []
        self._bucket_dps: dict[int, list] = {}        # optimizer group index -> owned dedicated params
        self._bucket_all_dps: dict[int, list] = {}
        self._bucket_plain: dict[int, list] = {}
        self._last_profile: Optional[_StepProfile] = None
        self._last_clip_stats = None
        self._pending_gscale: Optional[torch.Tensor] = None
        self._step_count = 0
        self._first_step_shapes_logged = 0

        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay)
        groups = self._lower_param_groups(
            param_groups,
            lr=lr,
            momentum=momentum,
            weight_decay=weight_decay,
            adamw_lr=adamw_lr,
            adamw_betas=tuple(adamw_betas),
            adamw_weight_decay=adamw_weight_decay,
            adamw_eps=adamw_eps,
        )
        super().__init__(groups, defaults)
        if self.first_step_progress_log:
            self._log_setup()

    # ------------------------------------------------------------------ discovery
    def _collect_plain_params(self, model: nn.Module) -> list[nn.Parameter]:
        plain, seen, unmanaged = [], set(), []
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        for name, p in model.named_parameters():
            if id(p) in seen or hasattr(p, "_dedicated_owner_rank") or not p.requires_grad:
                continue
            seen.add(id(p))
            plain.append(p)
            managed = (DTensor is not None and isinstance(p, DTensor)) or getattr(p, "_dmuon_replicated", False)
            if world > 1 and not managed:
                unmanaged.append(name)
        if unmanaged:
            raise RuntimeError(
                "Muon: trainable parameters that are neither dedicated nor covered by fully_shard / "
                f"replicate would silently diverge across ranks: {', '.join(unmanaged[:8])}"
                + (" ..." if len(unmanaged) > 8 else "")
            )
        return plain

    def _dummy(self) -> nn.Parameter:
        d = nn.Parameter(torch.zeros(1, device=self.device), requires_grad=False)
        self._dummy_params.append(d)
        return d

    @staticmethod
    def _ref_of(dp) -> torch.Tensor:
        return dp._placeholder if dp._placeholder is not None else dp._unsharded_param

    @staticmethod
    def _refs_of(dp) -> list[torch.Tensor]:
        refs = [dp._original_param]
        if dp._placeholder is not None:
            refs.append(dp._placeholder)
        if dp._unsharded_param is not None:
            refs.append(dp._unsharded_param)
        return refs

    @staticmethod
    def _updates_here(dp) -> bool:
        if dp._dmuon_route == "sharded_adamw":
            return dp._sharded_adamw_data is not None
        return dp.is_owner

    # ------------------------------------------------------------------ param groups
    @staticmethod
    def _pick(group: dict, first: str, second: Optional[str], default):
        if first in group:
            return group[first]
        if second is not None and second in group:
            return group[second]
        return default

    def _add_bucket_pair(self, out: list[dict], name: str, muon_dps, adamw_dps, plain, hp: dict) -> None:
        """Append the ``<name>/muon`` and ``<name>/adamw`` optimizer groups."""
        mi = len(out)
        refs = [self._ref_of(dp) for dp in muon_dps if dp.is_owner]
        out.append(
            {
                "params": refs or [self._dummy()],
                "lr": hp["muon_lr"],
                "momentum": hp["momentum"],
                "weight_decay": hp["muon_wd"],
                "use_muon": True,
                "group_name": f"{name}/muon",
                "semantic_group_name": name,
                "subgroup_type": "muon",
            }
        )
        self._bucket_all_dps[mi] = list(muon_dps)
        self._bucket_dps[mi] = [dp for dp in muon_dps if dp.is_owner]
        ai = len(out)
        arefs = list(plain) + [self._ref_of(dp) for dp in adamw_dps]
        out.append(
            {
                "params": arefs or [self._dummy()],
                "lr": hp["adamw_lr"],
                "betas": tuple(hp["betas"]),
                "weight_decay": hp["adamw_wd"],
                "eps": hp["eps"],
                "use_muon": False,
                "group_name": f"{name}/adamw",
                "semantic_group_name": name,
                "subgroup_type": "adamw",
            }
        )
        self._bucket_all_dps[ai] = list(adamw_dps)
        self._bucket_dps[ai] = [dp for dp in adamw_dps if self._updates_here(dp)]
        self._bucket_plain[ai] = list(plain)

    def _lower_param_groups(self, user_groups, *, lr, momentum, weight_decay, adamw_lr, adamw_betas,
                            adamw_weight_decay, adamw_eps) -> list[dict]:
        base = dict(muon_lr=lr, momentum=momentum, muon_wd=weight_decay, adamw_lr=adamw_lr, betas=adamw_betas,
                    adamw_wd=adamw_weight_decay, eps=adamw_eps)
        out: list[dict] = []
        if user_groups is None:
            muon_dps, adamw_dps = [], []
            for dp in self._all_dedicated:
                route = normalize_route(dp._dmuon_route) or "muon"
                if route == "sharded_adamw" and dp._sharded_adamw_data is None:
                    raise RuntimeError(
                        f"{dp.fqn}: routed to sharded_adamw but built without shard storage; "
                        "give the route to dedicate_params (route_hint_fn / param_policy)"
                    )
                (muon_dps if route == "muon" else adamw_dps).append(dp)
            self._add_bucket_pair(out, "default", muon_dps, adamw_dps, self._plain_params, base)
            return out

        if isinstance(user_groups, dict):
            raise TypeError("Muon param_groups must be a list of dicts, not a dict")
        user_groups = list(user_groups)
        if not user_groups:
            raise ValueError("Muon param_groups must not be empty")
        dp_of: dict[int, Any] = {}
        for dp in self._all_dedicated:
            for ref in self._refs_of(dp):
                dp_of[id(ref)] = dp
        plain_of = {id(p): p for p in self._plain_params}
        names = {id(p): n for n, p in self.model.named_parameters()}
        taken: dict[tuple, str] = {}
        for gi, ug in enumerate(user_groups):
            if not isinstance(ug, dict):
                raise TypeError(f"Muon param_groups[{gi}] must be a dict")
            if "params" not in ug:
                raise ValueError(f"Muon param_groups[{gi}] is missing 'params'")
            gname = str(ug.get("group_name", ug.get("name", f"group_{gi}")))
            raw = ug["params"]
            raw = [raw] if isinstance(raw, torch.Tensor) else list(raw)
            override = None
            if any(k in ug for k in _ROUTE_KEYS):
                override = normalize_route(next(ug[k] for k in _ROUTE_KEYS if k in ug))
            muon_dps, adamw_dps, plain = [], [], []
            for t in raw:
                if not isinstance(t, torch.Tensor):
                    raise TypeError(f"Muon param_groups[{gi}] contains {type(t).__name__}, expected Tensor")
                if not t.requires_grad:
                    continue
                if id(t) in dp_of:
                    dp = dp_of[id(t)]
                    key = ("dedicated", id(dp))
                    route = override or normalize_route(dp._dmuon_route) or "muon"
                    if dp._sharded_adamw_data is not None and route != "sharded_adamw":
                        raise RuntimeError(
                            f"{dp.fqn}: built on the sharded_adamw route; a param group cannot move it to {route!r}"
                        )
                    if route == "sharded_adamw" and dp._sharded_adamw_data is None:
                        raise RuntimeError(
                            f"{dp.fqn}: assigned to sharded_adamw but built without shard storage; "
                            "give the route to dedicate_params"
                        )
                    dp._dmuon_route = route
                    (muon_dps if route == "muon" else adamw_dps).append(dp)
                elif id(t) in plain_of:
                    key = ("plain", id(t))
                    plain.append(plain_of[id(t)])
                else:
                    raise RuntimeError(
                        "Muon param_groups contains a trainable parameter this optimizer does not manage: "
                        f"{names.get(id(t), '<not in current model>')}. Build param_groups from the wrapped model."
                    )
                if key in taken:
                    raise ValueError(f"trainable parameter appears in multiple param_groups: {taken[key]} and {gname}")
                taken[key] = gname
            hp = dict(
                muon_lr=self._pick(ug, "muon_lr", "lr", lr),
                momentum=self._pick(ug, "momentum", None, momentum),
                muon_wd=self._pick(ug, "muon_weight_decay", "weight_decay", weight_decay),
                adamw_lr=self._pick(ug, "adamw_lr", "lr", adamw_lr),
                betas=self._pick(ug, "adamw_betas", None, adamw_betas),
                adamw_wd=self._pick(ug, "adamw_weight_decay", "weight_decay", adamw_weight_decay),
                eps=self._pick(ug, "adamw_eps", None, adamw_eps),
            )
            self._add_bucket_pair(out, gname, muon_dps, adamw_dps, plain, hp)
        missing = [dp.fqn for dp in self._all_dedicated if dp._requires_grad and ("dedicated", id(dp)) not in taken]
        missing += [names.get(id(p), "?") for p in self._plain_params if ("plain", id(p)) not in taken]
        if missing:
            raise RuntimeError("Muon param_groups omitted trainable model parameters: " + ", ".join(missing[:8]))
        return out

    def _log_setup(self) -> None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        owned = sum(len(v) for i, v in self._bucket_dps.items() if self.param_groups[i]["use_muon"])
        if rank < self.first_step_progress_log_limit:
            kern = "tcgen05 sm_100a kernels" if self.device.type == "cuda" and not self.ns.deterministic else "PyTorch"
            log.info(
                "[rank %d] Muon: %d owned matrices, %d dedicated tensors in total, %d other parameters; "
                "Newton-Schulz %s via %s", rank, owned, len(self._all_dedicated), len(self._plain_params),
                self.ns.backend, kern,
            )

    # ------------------------------------------------------------------ first-step progress
    def _first_step_log(self, message: str) -> None:
        """Rank-tagged progress line of the FIRST optimizer step (stdout,
        flushed): on a large job that step also loads the kernel library and
        builds every per-shape workspace, so a user watching the log sees where
        it is (the reference prints the same kind of lines around its one-time
        kernel selection, dmuon/optim/muon.py:325-442)."""
        if not self.first_step_progress_log:
            return
        if dist.is_available() and dist.is_initialized():
            rank, world = dist.get_rank(), dist.get_world_size()
        else:
            rank, world = 0, 1
        print(f"[dmuon_b200][rank={rank}/{world}] {message}", flush=True)

    def _first_step_begin(self) -> Optional[float]:
        if self._step_count != 1:
            return None
        self._first_step_shapes_logged = 0
        muon = self.owned_muon_params()
        adamw = self.owned_adamw_params()
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if rank == 0 or muon or adamw:
            shapes = {tuple(int(d) for d in dp.full_shape) for dp in muon}
            kern = "tcgen05 sm_100a kernels" if self.device.type == "cuda" and not self.ns.deterministic else "PyTorch"
            self._first_step_log(
                "first optimizer step started; the kernel library is loaded and per-shape workspaces are "
                f"allocated now (owned_muon_params={len(muon)}, owned_adamw_params={len(adamw)}, "
                f"unique_muon_shapes={len(shapes)}, ns_backend={self.ns.backend}, ns_kernel={kern}, "
                f"replicate_async={self.replicate_async})"
            )
        return time.perf_counter()

    def _first_step_shape(self, rows: int, cols: int, count: int, path: str) -> None:
        if self._step_count != 1 or self._first_step_shapes_logged >= self.first_step_progress_log_limit:
            return
        self._first_step_shapes_logged += 1
        self._first_step_log(
            f"first optimizer step: Newton-Schulz ({self.ns.backend}) on {count} matrices of shape "
            f"{rows} x {cols}, gram_dim={min(rows, cols)}, path={path}"
        )

    def _first_step_end(self, started: Optional[float], failed: bool = False) -> None:
        if started is None:
            return
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if rank == 0 or self.owned_muon_params() or self.owned_adamw_params():
            what = "failed" if failed else "queued"
            self._first_step_log(
                f"first optimizer step {what} after {time.perf_counter() - started:.3f} s of host time"
                + ("" if failed else "; later steps reuse what was set up now")
            )

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], Any]] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step_count += 1
        self._raise_if_a_kernel_wait_ran_out()
        started = self._first_step_begin()
        try:
            self._step_impl()
        except BaseException:
            self._first_step_end(started, failed=True)
            raise
        self._first_step_end(started)
        self._poll_kernel_status()
        return loss

    # ------------------------------------------------------------------ device status word
    def _status_watch_enabled(self) -> bool:
        if self.device.type != "cuda":
            return False
        return os.environ.get("DMUON_STATUS_WATCH", "1").strip().lower() not in ("0", "false", "no", "off")

    def _poll_kernel_status(self) -> None:
        """Queue a 16-byte copy of the device's status word (where kernels record
        a bounded wait that ran out) into pinned host memory, behind this step.
        Nothing waits for it: the NEXT step looks at it if the copy has landed."""
        if getattr(self, "_status_watch_broken", False) or not self._status_watch_enabled() or not _kernels_ok():
            return
        from ..ops import gemm as G

        try:
            if getattr(self, "_status_host", None) is None:
                self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
                self._status_event = torch.cuda.Event()
            self._status_host.copy_(G.status_buffer(self.device), non_blocking=True)
            self._status_event.record(torch.cuda.current_stream(self.device))
            self._status_polled = True
        except Exception as exc:      # a watch that cannot be set up (no pinned memory, stream capture) must not stop training
            self._status_watch_broken = True
            self._status_polled = False
            log.warning("dmuon_b200: kernel status watch switched off (%s); call check_kernel_status() by hand", exc)

    def _raise_if_a_kernel_wait_ran_out(self) -> None:
        """Report, one step late and without synchronising, that a kernel gave up
        waiting (a peer that never signalled, a stalled pipeline): training on
        after that would use stale weights or gradients."""
        if not getattr(self, "_status_polled", False):
            return
        try:
            if not self._status_event.query():
                return
            code = int(self._status_host[0])
        except Exception as exc:
            self._status_watch_broken, self._status_polled = True, False
            log.warning("dmuon_b200: kernel status watch switched off (%s); call check_kernel_status() by hand", exc)
            return
        self._status_polled = False
        if code != 0:
            from ..ops import gemm as G

            G.status_buffer(self.device).zero_()
            raise G.KernelTimeout(
                f"dmuon_b200 kernel wait ran out during the previous step (code {code}: {G.describe_status(code)})")

    def check_kernel_status(self) -> None:
        """Synchronising form of the same check (end of training, before a
        checkpoint is trusted)."""
        if self.device.type == "cuda" and _kernels_ok():
            from ..ops import gemm as G

            G.check_status(self.device)

    # ------------------------------------------------------------------ group pipeline
    def _has_post_step_traffic(self, g) -> bool:
        """Does this group send anything after the update (replicate-axis
        publish, tensor-parallel scatter, sharded-Muon scatter, DDP broadcast)?"""
        if getattr(g, "uses_peer_memory", False):
            return False
        if g.mode != "fsdp":
            return True
        rep = getattr(g, "replicate_group", None)
        if rep is not None and rep.size() > 1:
            return True
        return any(p.tp_group is not None or p._sharded_muon_data is not None for p in g.params)

    def _pipeline_blocks(self) -> list[list]:
        """Consecutive blocks of communication groups (forward order) that the
        step works through one after the other: while block *k* runs its
        Newton-Schulz products, block *k+1*'s gradient waits and tensor-parallel
        gathers are already queued on the reduce lane and block *k-1*'s post-step
        publish is in flight on the publish lanes.  The reference pipelines per
        group (dmuon/optim/muon.py:1446-1546); blocks of several layers keep the
        per-shape batches large enough for the kernels.  One block (no
        pipelining) when nothing travels after the update, when
        ``group_prepare_ahead`` is off, or on the peer-memory plane, where the
        update kernels themselves publish."""
        groups = self._comm_groups
        if not groups or not self.group_prepare_ahead or not any(self._has_post_step_traffic(g) for g in groups):
            return [list(groups)]
        try:
            want = int(os.environ.get("DMUON_GROUP_PIPELINE_BLOCKS", "4"))
        except ValueError:
            want = 4
        n = max(1, min(want, len(groups)))
        per = (len(groups) + n - 1) // n
        return [list(groups[i : i + per]) for i in range(0, len(groups), per)]

    def _step_impl(self) -> None:
        prof = _StepProfile(self.device, self.record_step_profile)
        groups = self._comm_groups
        gscale, self._pending_gscale = self._pending_gscale, None

        rt = getattr(self.comm_ctx, "peer_runtime", None)
        blocks = self._pipeline_blocks()
        with prof.phase("prepare_muon_grads"):
            if len(blocks) == 1:
                self._ensure_grads_ready()
            else:
                for g in blocks[0]:
                    prepare_group_muon_grads(g, use_reduce_lane=True)
            if rt is not None:
                rt.before_owner_writes()
        # a published copy that survived until here (evaluation forward, no
        # backward) would be stale after the update below
        for g in groups:
            if g.mode == "fsdp" and (g._is_unsharded or g._unshard_ticket is not None):
                g.reshard()
            if g.mode == "fsdp":
                g.stage_publish_targets()

        for bi, block in enumerate(blocks):
            only = None
            if len(blocks) > 1:
                with prof.phase("group_pipeline"):
                    # queue the next block's waits and gathers before this block's compute is issued
                    if bi + 1 < len(blocks):
                        for g in blocks[bi + 1]:
                            prepare_group_muon_grads(g, use_reduce_lane=True)
                    for g in block:
                        wait_group_muon_grads(g)
                only = {id(p) for g in block for p in g.params}
            with prof.phase("muon"):
                for gi, pg in enumerate(self.param_groups):
                    if pg["use_muon"]:
                        self._step_muon_bucket(gi, pg, gscale, prof, only)
            with prof.phase("dedicated_adamw"):
                for gi, pg in enumerate(self.param_groups):
                    if not pg["use_muon"]:
                        self._step_dedicated_adamw(gi, pg, gscale, only)
            if len(blocks) > 1:
                with prof.phase("post_step_publish"):
                    for g in block:
                        g.post_step_publish_async()
        with prof.phase("post_step_publish"):
            if rt is not None:
                rt.after_optimizer_consumed()
                rt.publish_owned()
            for ex in (getattr(self.comm_ctx, "tp_exchanges", None) or {}).values():
                ex.after_step()
            if len(blocks) == 1:
                for g in groups:
                    g.post_step_publish_async()
            if not self.replicate_async or self._has_tp:
                for g in groups:
                    g._pre_forward_wait()
        with prof.phase("adamw"):
            for gi, pg in enumerate(self.param_groups):
                if not pg["use_muon"]:
                    self._step_plain_adamw(gi, pg, gscale)
        if self.post_step_prefetch_groups > 0:
            for g in groups[: self.post_step_prefetch_groups]:
                if g.mode == "fsdp":
                    g._pre_forward_wait()
                    g.unshard(prefetch=True)
        fence_isolated_process_groups()
        self._last_profile = prof if self.record_step_profile else None

    def _ensure_grads_ready(self, materialize: bool = False) -> None:
        prepare_muon_grads(self.model, coalesce_wait=True)
        rt = getattr(self.comm_ctx, "peer_runtime", None)
        if rt is not None:
            rt.announce_grads()
            if materialize:
                rt.materialize([dp for dp in self._all_dedicated if dp.is_owner])
        if materialize:
            for dp in self._all_dedicated:
                if hasattr(dp._tp_full_grad, "materialize"):
                    dp._tp_full_grad.materialize()

    # ------------------------------------------------------------------ Muon
    def _momentum_of(self, dp, shape, device) -> torch.Tensor:
        st = self.state[id(dp)]
        buf = st.get("momentum_buffer")
        if buf is None:
            buf = torch.zeros(shape, dtype=dp._optim_dtype, device=device)
            st["momentum_buffer"] = buf
        return buf

    def _step_muon_bucket(self, gi: int, pg: dict, gscale, prof: _StepProfile, only: Optional[set] = None) -> None:
        """Muon update of the owned matrices of optimizer group ``gi``; with
        ``only`` (ids of dedicated parameters) restricted to one pipeline block."""
        lr, mu, wd = float(pg["lr"]), float(pg["momentum"]), float(pg["weight_decay"])
        # every TP peer learns the decay factor locally (the update itself arrives by scatter)
        for dp in self._bucket_all_dps.get(gi, ()):
            if dp.tp_group is not None and (only is None or id(dp) in only):
                dp._tp_wd_factor = 1.0 - lr * wd
        bucket = [dp for dp in self._bucket_dps.get(gi, ()) if only is None or id(dp) in only]
        gram_ids: set[int] = set()
        if self.tp_distributed_gram:
            gram_dps = [
                dp for dp in bucket
                if dp.tp_group is not None and dp._reduced_grad is not None and self._tp_gram_rejection_reason(dp) is None
            ]
            if gram_dps:
                with prof.phase("tp_distributed_gram"):
                    self._step_tp_distributed_gram(gram_dps, lr, mu, wd, gscale)
                gram_ids = {id(dp) for dp in gram_dps}
        work = []
        for dp in bucket:
            if id(dp) in gram_ids:
                continue
            if dp.tp_group is not None:
                if not dp.is_tp_owner or dp._tp_full_grad is None:
                    continue
                grad = dp._tp_full_grad
            else:
                if dp._reduced_grad is None and not getattr(dp, "_peer_grad_pending", False):
                    continue
                grad = dp._reduced_grad      # None: still in the peers' arenas
            work.append((dp, grad))
        if not work:
            return
        use_kernels = self.device.type == "cuda" and self.ns.uses_kernels(work[0][0]._owned_data)
        if not use_kernels and any(g is None for _, g in work):
            rt = self.comm_ctx.peer_runtime
            rt.materialize([dp for dp, g in work if g is None])
            work = [(dp, dp._reduced_grad) for dp, _ in work]
        if not use_kernels:
            work = [(dp, g.materialize() if hasattr(g, "materialize") else g) for dp, g in work]
        if use_kernels:
            self._step_muon_kernels(work, lr, mu, wd, gscale)
        else:
            for dp, grad in work:
                rows = int(grad.shape[0])
                self._first_step_shape(rows, grad.numel() // rows, 1, f"PyTorch, {dp.fqn}")
                self._step_muon_torch(dp, grad, lr, mu, wd, gscale)
        for dp, _ in work:
            if dp.tp_group is None:
                dp._reduced_grad = None

    def _step_muon_torch(self, dp, grad, lr, mu, wd, gscale) -> None:
        rows = int(grad.shape[0])
        g2 = grad.reshape(rows, -1)
        buf = self._momentum_of(dp, g2.shape, g2.device)
        g = g2.to(buf.dtype)
        if gscale is not None:
            g = g * gscale.to(g.dtype)
        buf.mul_(mu).add_(g)
        u = g.add(buf, alpha=mu) if self.nesterov else buf
        upd = self.ns.local(u, self.ns_steps)
        scale = muon_update_scale(g2.shape)
        if dp.tp_group is not None:
            dp._tp_full_delta = (upd.float() * (-lr * scale)).reshape(dp.full_shape)
            return
        w = dp._owned_data.view(rows, -1)
        if wd > 0:
            w.mul_(1.0 - lr * wd)
        w.add_(upd.to(w.dtype), alpha=-lr * scale)

    # ------------------------------------------------------------------ TP distributed Gram
    def _tp_gram_segment_count(self) -> int:
        coefs = self.ns.resolved_coefficients(self.ns_steps)
        return 1 + sum(1 for i in self.ns.resolved_restarts() if i != 0 and 0 <= i < len(coefs))

    def _tp_gram_wire_dtype(self) -> torch.dtype:
        return torch.float16 if self.device.type == "cuda" else torch.float32

    def _tp_gram_rejection_reason(self, dp) -> Optional[str]:
        """Why a parameter keeps the gather -> NS -> scatter route (None: it
        takes the factor-broadcast route).  Same rules as the reference
        (``dmuon/optim/muon.py:1035-1078``): Gram formulation only, the shard
        must lie along the columns of the oriented (wide) matrix so that the
        factors multiply from the left, and under the default policy the
        factors must be clearly cheaper to send than the full update."""
        if self.ns.backend != "gram":
            return "non_gram_backend"
        if dp.tp_group is None:
            return "non_tp_param"
        if dp.shard_dim not in (0, 1):
            return "unsupported_shard_dim"
        if len(dp.full_shape) < 2:
            return "not_matrix"
        rows = int(dp.full_shape[0])
        cols = int(math.prod(dp.full_shape[1:]))
        transposed = rows > cols
        if (1 - dp.shard_dim if transposed else dp.shard_dim) != 1:
            return "unsupported_orientation"
        policy = str(self.tp_distributed_gram_policy).lower()
        if policy in ("all", "force", "always"):
            return None
        if policy in ("0", "false", "no", "off", "none"):
            return "policy_disabled"
        factor_dim = cols if transposed else rows
        scatter_bytes = rows * cols * dp._owned_data.element_size()
        factor_bytes = self._tp_gram_segment_count() * factor_dim * factor_dim * 2
        ratio = self.tp_distributed_gram_max_factor_to_scatter_ratio
        if ratio <= 0:
            return "ratio_threshold_disabled"
        if factor_bytes >= scatter_bytes:
            return "factor_not_smaller"
        if factor_bytes / scatter_bytes > ratio:
            return "factor_ratio_too_high"
        return None

    def _step_tp_distributed_gram(self, dps, lr, mu, wd, gscale) -> None:
        """TP owners turn the gathered full matrix into left-factor segments
        and broadcast them (plus the normaliser); every TP rank keeps momentum
        for its own shard and applies the factors to it, so the full update is
        never scattered (reference ``dmuon/optim/muon.py:1097-1278``)."""
        nseg, wire = self._tp_gram_segment_count(), self._tp_gram_wire_dtype()
        on_kernels = self.device.type == "cuda" and _kernels_ok() and not self.ns.deterministic
        if on_kernels:
            from ..ops import ns_sm100
        pending = []
        for dp in dps:
            st = self.state[id(dp)]
            rows = int(dp.full_shape[0])
            cols = int(math.prod(dp.full_shape[1:]))
            transposed = rows > cols
            fdim = cols if transposed else rows
            lg = _local(dp._reduced_grad)
            lg = lg.reshape(lg.shape[0], -1).to(dp._optim_dtype)
            if gscale is not None:
                lg = lg * gscale.to(lg.dtype)
            lbuf = st.get("tp_local_momentum_buffer")
            if lbuf is None:
                lbuf = st["tp_local_momentum_buffer"] = torch.zeros_like(lg)
            lbuf.mul_(mu).add_(lg)
            local_u = lg.add(lbuf, alpha=mu) if self.nesterov else lbuf
            if dp.is_tp_owner:
                if dp._tp_full_grad is None:
                    raise RuntimeError(f"{dp.param_name}: the TP gather did not deliver the full gradient to its TP owner")
                full = dp._tp_full_grad
                if hasattr(full, "materialize"):
                    full = full.materialize()       # shards still in the TP peers' buffers
                fg = full.reshape(rows, cols).to(dp._optim_dtype)
                if gscale is not None:
                    fg = fg * gscale.to(fg.dtype)
                fbuf = self._momentum_of(dp, (rows, cols), fg.device)
                fbuf.mul_(mu).add_(fg)
                full_u = fg.add(fbuf, alpha=mu) if self.nesterov else fbuf
                if on_kernels:
                    # every product of the factor computation on the tcgen05 kernels
                    segs, tr, norm = ns_sm100.gram_factors(
                        full_u, self.ns.resolved_coefficients(self.ns_steps), self.ns.resolved_restarts())
                else:
                    segs, tr, norm = gram_newton_schulz_factors(
                        full_u, steps=self.ns_steps, coefficients=self.ns.coefficients,
                        restart_iterations=self.ns.restart_iterations, compute_dtype=wire,
                    )
                assert tr == transposed and len(segs) == nseg
                segs = [s.to(wire).contiguous() for s in segs]
                norm = norm.reshape(()).float()
            else:
                segs = [torch.empty(fdim, fdim, dtype=wire, device=self.device) for _ in range(nseg)]
                norm = torch.empty((), dtype=torch.float32, device=self.device)
            pending.append((dp, segs, norm, local_u, transposed, rows, cols))
        # one pass of broadcasts per TP group, in parameter order (identical on every TP rank)
        for dp, segs, norm, *_ in pending:
            dist.broadcast(norm, src=dp._tp_owner_global_rank, group=dp.tp_group)
            for s in segs:
                dist.broadcast(s, src=dp._tp_owner_global_rank, group=dp.tp_group)
        for dp, segs, norm, local_u, transposed, rows, cols in pending:
            if on_kernels and ns_sm100.factors_supported(int(local_u.shape[0]), int(local_u.shape[1])):
                upd = ns_sm100.apply_factors(local_u, segs, transposed, norm)
            else:
                upd = apply_gram_factors(local_u.float(), segs, transposed, norm)
            w = dp._owned_data
            if wd > 0:
                w.mul_(1.0 - lr * wd)
            w.add_(upd.reshape(w.shape).to(w.dtype), alpha=-lr * muon_update_scale((rows, cols)))
            dp._tp_full_grad = dp._tp_full_delta = dp._reduced_grad = None
            dp._tp_gathered = False
            dp._tp_wd_factor = 1.0

    def _step_muon_kernels(self, work, lr, mu, wd, gscale) -> None:
        from ..ops import ns_sm100

        by_shape: dict[tuple, list] = defaultdict(list)
        rt = getattr(self.comm_ctx, "peer_runtime", None)
        for dp, grad in work:
            shape = grad.shape if grad is not None else dp._orig_size
            rows = int(shape[0])
            numel = grad.numel() if grad is not None else dp.numel
            gdt = grad.dtype if grad is not None else "peer"
            # parameters with and without a publish slot never share a batch: the update kernel writes
            # the bf16 copies for all matrices of a batch or for none
            key = (rows, numel // rows, gdt, dp._optim_dtype, dp._owned_data.dtype, dp.tp_group is not None,
                   getattr(dp, "_publish_view", None) is not None)
            by_shape[key].append((dp, grad))
        coefs = self.ns.resolved_coefficients(self.ns_steps)
        restarts = self.ns.resolved_restarts()
        for (rows, cols, gdt, _od, _md, is_tp, _has_pub), items in by_shape.items():
            cap = ns_sm100.max_batch(rows, cols)
            self._first_step_shape(rows, cols, len(items), "sm_100a kernels, batched by shape")
            for lo in range(0, len(items), cap):
                chunk = items[lo : lo + cap]
                moms = [self._momentum_of(dp, (rows, cols), self.device) for dp, _ in chunk]
                if gdt == "peer":
                    # reduce-to-owner happens inside the prologue kernel
                    grads = None
                    peer = rt.source_for([dp for dp, _ in chunk])
                elif gdt == "tp_peer":
                    # tensor-parallel gather happens inside the prologue kernel
                    from ..parallel.tp_peer import TPGatherSource

                    grads = None
                    peer = TPGatherSource([g for _, g in chunk])
                else:
                    peer = None
                    grads = [g.reshape(rows, cols) if g.is_contiguous() else g.reshape(rows, cols).contiguous() for _, g in chunk]
                common = dict(
                    mu=mu, nesterov=self.nesterov, coefs=coefs, restarts=restarts, formulation=self.ns.backend,
                    lr=lr, weight_decay=wd, update_scale=muon_update_scale((rows, cols)),
                    compute_dtype=self.ns.compute_dtype, gscale=gscale, peer=peer,
                )
                if is_tp:
                    exchanges = getattr(self.comm_ctx, "tp_exchanges", None) or {}
                    deltas = []
                    for dp, _ in chunk:
                        ex = exchanges.get(id(dp.tp_group))
                        if ex is not None:
                            # written where the TP peers will pull their slices from
                            ex.before_delta_writes()
                            deltas.append(ex.delta_view(dp))
                        else:
                            deltas.append(torch.empty(dp.full_shape, dtype=torch.float32, device=self.device))
                    ns_sm100.muon_update_batched(grads, moms, None, deltas=deltas, **common)
                    for (dp, _), d in zip(chunk, deltas):
                        dp._tp_full_delta = d
                else:
                    masters = [dp._owned_data for dp, _ in chunk]
                    publish = [getattr(dp, "_publish_view", None) for dp, _ in chunk]
                    multicast = None
                    nvls = rt is not None and rt.publish_via == "nvls" and all(p is not None for p in publish)
                    if nvls and rt.nvls_publish == "epilogue":
                        if cols % 8 == 0:
                            # the last product stores the bf16 weights through the NVSwitch multicast
                            # mapping of the publish arena: they land on every rank while it runs
                            esz = rt.pub.element_size()
                            multicast = [rt.pub_mc + dp._arena_offset * esz for dp, _ in chunk]
                        else:
                            publish = [None] * len(chunk)       # published (cast + multicast) after the step
                    wrote = ns_sm100.muon_update_batched(grads, moms, masters, publish=publish,
                                                         publish_multicast=multicast, **common)
                    if nvls and wrote and multicast is None:
                        # the last product wrote the local slots: replicate them to all ranks on the
                        # publish lane while the next batch is orthogonalised
                        rt.multicast_publish_async([dp for dp, _ in chunk])
                    for dp, _ in chunk:
                        dp._publish_fresh = bool(wrote)

    # ------------------------------------------------------------------ AdamW
    def _adamw_state(self, key, like: torch.Tensor, dtype: torch.dtype) -> dict:
        st = self.state[key]
        if "exp_avg" not in st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(like, dtype=dtype)
            st["exp_avg_sq"] = torch.zeros_like(like, dtype=dtype)
        return st

    def _adamw_apply(self, entries: list[tuple], pg: dict, gscale) -> None:
        """``entries``: (param tensor, grad tensor, state dict, publish or None).
        Tensors with no gradient were filtered out by the caller, so every
        tensor keeps its own step count."""
        if not entries:
            return
        lr, (b1, b2), wd, eps = float(pg["lr"]), pg["betas"], float(pg["weight_decay"]), float(pg["eps"])
        for _, _, st, _ in entries:
            st["step"] += 1
        p0 = entries[0][0]
        if p0.is_cuda and _kernels_ok():
            from ..ops import multi_tensor as MT

            buckets: dict[tuple, list] = defaultdict(list)
            for e in entries:
                p, g, st, _ = e
                ok = p.is_contiguous() and g.is_contiguous() and p.dtype in MT._DT and g.dtype in MT._DT
                buckets[(p.dtype, g.dtype, st["exp_avg"].dtype) if ok else None].append(e)
            for key, items in buckets.items():
                if key is None:
                    self._adamw_torch(items, lr, b1, b2, wd, eps, gscale)
                    continue
                MT.adamw(
                    [p for p, _, _, _ in items], [g for _, g, _, _ in items],
                    [st["exp_avg"] for _, _, st, _ in items], [st["exp_avg_sq"] for _, _, st, _ in items],
                    [st["step"] for _, _, st, _ in items],
                    lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=wd,
                    publish=[pub for _, _, _, pub in items], gscale=gscale,
                )
        else:
            self._adamw_torch(entries, lr, b1, b2, wd, eps, gscale)

    @staticmethod
    def _adamw_torch(entries, lr, b1, b2, wd, eps, gscale) -> None:
        for p, g, st, pub in entries:
            m, v, t = st["exp_avg"], st["exp_avg_sq"], st["step"]
            gf = g.to(m.dtype)
            if gscale is not None:
                gf = gf * gscale.to(gf.dtype)
            p.mul_(1.0 - lr * wd)
            m.mul_(b1).add_(gf, alpha=1.0 - b1)
            v.mul_(b2).addcmul_(gf, gf, value=1.0 - b2)
            bc1, bc2 = 1.0 - b1**t, 1.0 - b2**t
            denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
            p.addcdiv_(m.to(p.dtype) if m.dtype != p.dtype else m, denom.to(p.dtype), value=-lr / bc1)
            if pub is not None:
                pub.copy_(p)

    def _step_dedicated_adamw(self, gi: int, pg: dict, gscale, only: Optional[set] = None) -> None:
        entries = []
        bucket = [dp for dp in self._bucket_dps.get(gi, ()) if only is None or id(dp) in only]
        rt = getattr(self.comm_ctx, "peer_runtime", None)
        if rt is not None:
            rt.materialize(bucket)
        for dp in bucket:
            if dp._dmuon_route == "sharded_adamw":
                g, p = dp._sharded_adamw_grad, dp._sharded_adamw_data
            else:
                # (tensor-parallel parameters too: AdamW is element-wise, every TP peer updates its own shard)
                g, p = dp._reduced_grad, dp._owned_data
            if g is None or p is None:
                continue
            st = self._adamw_state(id(dp), p, dp._optim_dtype)
            entries.append((p, g.reshape(p.shape), st, None))
        self._adamw_apply(entries, pg, gscale)
        if self.device.type == "cuda":
            # reduced gradients may have been allocated on the reduce lane; the AdamW kernels above read them on
            # this stream, so tell the allocator before the references are dropped (the lanes also wait for this
            # stream before they allocate again; this makes the lifetime independent of that)
            cur = torch.cuda.current_stream(self.device)
            for _, g, _, _ in entries:
                if g.is_cuda:
                    g.record_stream(cur)
        for dp in bucket:
            dp._reduced_grad = None
            dp._sharded_adamw_grad = None

    def _step_plain_adamw(self, gi: int, pg: dict, gscale) -> None:
        entries = []
        for p in self._bucket_plain.get(gi, ()):
            if p.grad is None:
                continue
            pl, gl = _local(p), _local(p.grad)
            if pl.numel() == 0:
                continue
            st = self._adamw_state(p, pl, torch.float32 if pl.dtype != torch.float64 else pl.dtype)
            entries.append((pl, gl, st, None))
        self._adamw_apply(entries, pg, gscale)

    # ------------------------------------------------------------------ misc API
    def zero_grad(self, set_to_none: bool = True) -> None:
        for dp in self._all_dedicated:
            dp._reduced_grad = None
            dp._sharded_adamw_grad = None
            dp._accumulated_grad = None
            dp._tp_full_grad = None
            dp._tp_gathered = False
            dp._peer_grad_pending = False
            if dp.mode == "ddp":
                dp.clear_local_grad()
        for p in self._plain_params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.detach_()
                    p.grad.zero_()

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0, **kwargs):
        """Clip the owned Muon gradients by their global norm (see
        :func:`dmuon_b200.grad_clip.clip_grad_norm_`)."""
        from ..grad_clip import clip_grad_norm_

        return clip_grad_norm_(self, max_norm, norm_type=norm_type, **kwargs)

    @property
    def last_muon_grad_clip_stats(self):
        return self._last_clip_stats

    def scale_grads_on_next_step(self, coef) -> None:
        """Multiply EVERY gradient of the next ``step()`` by ``coef`` (a float or a
        one-element tensor on the optimizer's device) inside the kernels that
        read the gradients anyway -- the Muon prologue and the AdamW passes --
        instead of in a separate pass over all gradients.  Meant for trainers
        that compute one global clip coefficient themselves (loss-scale
        unscaling, a norm over several models): ``opt.scale_grads_on_next_step
        (coef); opt.step()`` equals scaling all gradients by ``coef`` first.  The
        coefficient is used once; several calls before a step multiply."""
        t = coef if torch.is_tensor(coef) else torch.tensor(float(coef), dtype=torch.float32, device=self.device)
        t = t.detach().reshape(()).to(device=self.device, dtype=torch.float32)
        self._pending_gscale = t if self._pending_gscale is None else self._pending_gscale * t

    def consume_last_step_profile(self) -> Optional[dict]:
        prof, self._last_profile = self._last_profile, None
        return None if prof is None else prof.summary()

    def owned_muon_params(self) -> list:
        return [dp for i, pg in enumerate(self.param_groups) if pg["use_muon"] for dp in self._bucket_dps.get(i, ())]

    def owned_adamw_params(self) -> list:
        return [dp for i, pg in enumerate(self.param_groups) if not pg["use_muon"] for dp in self._bucket_dps.get(i, ())]


def _kernels_ok() -> bool:
    from ..ops import ns_sm100

    return ns_sm100.available()

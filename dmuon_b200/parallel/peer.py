"""Peer-memory data plane for 1-D dedicated ownership on one NVSwitch domain.

Instead of NCCL broadcasts and reduces, every rank holds two symmetric arenas
with the same layout on all ranks (one slot per dedicated parameter):

publish arena   bf16 weights.  The owner writes its slots (the last
                Newton-Schulz GEMM stores the bf16 copy there directly), every
                other rank PULLS the slots it needs with a copy kernel that
                reads the owner's arena through its peer mapping.
gradient arena  each rank's local gradients.  Nothing is sent after backward:
                the owner's Muon prologue kernel READS the N arenas through
                their peer mappings, sums them in rank order in fp32, scales by
                1/N and applies momentum / Nesterov / cast / Frobenius norm in
                the same pass.

Bulk data crosses NVLink in one of these ways (``DMUON_PEER_COPY``).  "nvls"
(needs an NVSwitch multicast mapping of the symmetric buffers): the owner's new
bf16 weights are stored with ``multimem.st`` -- by a copy kernel beside the next
Newton-Schulz batch, or by the last Newton-Schulz GEMM's own epilogue -- so they
land in every rank's arena and readers copy nothing; gradients are summed inside
the switch: per layer, during backward, a small kernel on the reduce lane reads
the owner's span through the multicast mapping with ``multimem.ld_reduce`` and
keeps ONE reduced copy, which the Muon prologue then reads locally.  "hybrid":
that in-switch reduce, with the publish left to the readers' copy engines (the
owner keeps one reduced copy instead of N - 1 staged slices: 6.7 GiB less at
four ranks of an 8B model).  "ce" (what "auto" picks: the fastest step measured
at two and at four ranks): copy-engine transfers.  Readers pull publish spans
with asynchronous copies, owners gather the peers' gradient slices of each layer
into local staging buffers while backward is still running, and the fixed-order
fp32 sum runs locally inside the Muon prologue; no SM is taken from the forward
and backward GEMMs.  "sm": the pull and reduce kernels load through the peer
mappings themselves (the form the fused forward GEMM builds on).

Ordering uses four monotonically increasing epoch words per rank in a
symmetric flag array (gradients ready / consumed, weights published /
consumed).  Waits are small kernels or kernel preambles with a cycle budget;
when a budget runs out the status word is set and ``check()`` raises.

This replaces the communication of the reference's FSDP2 backend
(dmuon/_backends/fsdp2/group.py:481-899 unshard, :998-1187 reduce) for the
common case (one data-parallel axis, no tensor parallelism); every other
placement keeps the collective implementation in ``dgroup.py``.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
from torch.profiler import record_function

from . import dgroup as _dgroup
from .dgroup import DedicatedParamGroup
from .dparam import DedicatedParam

KIND_GRAD_READY, KIND_GRAD_CONSUMED, KIND_PUB_READY, KIND_PUB_CONSUMED = 0, 1, 2, 3
MAX_PEERS = 8
ALIGN = 64          # elements; keeps every slot 128-byte aligned for bf16
#: CTAs per tensor of the in-backward reduce: enough loads in flight for NVLink
#: (about 28 KB per CTA) without taking many SMs from the backward GEMMs
REDUCE_BLOCKS_PER_TENSOR = 24
#: CTAs of the per-layer in-switch gradient reduce that runs beside the backward GEMMs: each 16-byte
#: reduce-load returns data already summed over all ranks, so a few CTAs keep up with a layer
#: (16 CTAs moved 105 GB/s on two B200s: 2 ms for a layer's 218 MB, against 8 ms of backward per layer)
NVLS_REDUCE_BLOCKS = 16
#: CTAs of the multicast publish that runs beside the Newton-Schulz products of the next shape batch
NVLS_PUBLISH_BLOCKS = 16


#: what ``DMUON_PEER_COPY=auto`` means.  Copy engines for both bulk transfers: on Llama-3-8B the step took
#: 487.6 ms at four ranks against 494.2 ms ("hybrid": in-switch reduce, copy-engine publish) and 496.2 ms
#: ("nvls"), because the in-switch reduce and the multicast stores take SMs from backward and from the
#: Newton-Schulz products while the copy engines take none.  "hybrid" holds 6.7 GiB less on the owner.
AUTO_COPY_MODE = "ce"


def nvls_publish_mode() -> str:
    """``DMUON_NVLS_PUBLISH``: how the owner's new bf16 weights reach the other
    ranks on the NVSwitch plane.  ``lane`` (default): the update kernel writes
    the local arena slot and a copy kernel on the publish lane stores the slot
    through the multicast mapping with fully coalesced 16-byte stores, while the
    next batch of Newton-Schulz products runs.  ``epilogue``: the last product's
    epilogue issues the ``multimem.st`` itself, tile by tile (one kernel does the
    GEMM and the broadcast); its stores are 16 bytes per row and lane, which the
    links carry at about a quarter of the coalesced rate (measured on two B200s:
    +58 ms per step for 7 GB), so it is the option, not the default."""
    mode = os.environ.get("DMUON_NVLS_PUBLISH", "lane").strip().lower()
    if mode not in ("lane", "epilogue"):
        raise ValueError("DMUON_NVLS_PUBLISH must be 'lane' or 'epilogue'")
    return mode
#: value of the guard words around the arenas in canary mode (exact in bf16, fp16 and fp32)
CANARY_VALUE = -1.5


def peer_backend_requested() -> str:
    return os.environ.get("DMUON_COMM_BACKEND", "auto").strip().lower()


def spans_hosts() -> bool:
    """True when the launcher says the job runs on more than one host
    (``LOCAL_WORLD_SIZE``, set by ``torchrun``, smaller than the world size).
    Peer memory needs every rank of a group on one NVLink domain; without the
    variable (single-host spawners) nothing is assumed."""
    local = os.environ.get("LOCAL_WORLD_SIZE")
    if not local or not (dist.is_available() and dist.is_initialized()):
        return False
    try:
        return dist.get_world_size() > int(local)
    except ValueError:
        return False


def peer_backend_possible(device: torch.device, dp_group, replicate_group, dparams) -> Optional[str]:
    """None when usable, else the reason it is not."""
    if device.type != "cuda":
        return "not a CUDA device"
    if dp_group is None or dp_group.size() < 2:
        return "single rank"
    if dp_group.size() > MAX_PEERS:
        return f"more than {MAX_PEERS} ranks on the shard axis"
    if spans_hosts():
        return "the job spans more than one host"
    if replicate_group is not None and replicate_group.size() > 1:
        return "replicate axis present"
    if any(p.tp_group is not None for p in dparams):
        return "tensor-parallel parameters"
    if any(p._dmuon_route == "sharded_adamw" for p in dparams):
        return "sharded_adamw route"
    if any(p._sharded_muon_data is not None for p in dparams):
        return "all_gather forward placement"
    if len({p._param_dtype for p in dparams}) != 1 or len({p._grad_dtype or p._param_dtype for p in dparams}) != 1:
        return "mixed publish or gradient dtypes"
    try:
        import torch.distributed._symmetric_memory as _symm  # noqa: F401
    except Exception as exc:  # pragma: no cover
        return f"symmetric memory unavailable: {exc}"
    return None


def peer_backend_possible_from_policies(device, dp_group, replicate_group, params, policies, is_tp) -> Optional[str]:
    """The same question as :func:`peer_backend_possible`, asked before the
    dedicated parameters are built (from the resolved per-parameter policies)."""
    if device.type != "cuda":
        return "not a CUDA device"
    if dp_group is None or dp_group.size() < 2:
        return "single rank"
    if dp_group.size() > MAX_PEERS:
        return f"more than {MAX_PEERS} ranks on the shard axis"
    if spans_hosts():
        return "the job spans more than one host"
    if replicate_group is not None and replicate_group.size() > 1:
        return "replicate axis present"
    if any(is_tp(p) for p in params):
        return "tensor-parallel parameters"
    pub, grad = set(), set()
    for p in params:
        pol = policies[p]
        if (pol.route or "") == "sharded_adamw":
            return "sharded_adamw route"
        if (pol.muon_forward_unshard or "broadcast") != "broadcast":
            return "all_gather forward placement"
        pd = pol.param_dtype or p.dtype
        pub.add(pd)
        grad.add(pol.grad_dtype or pd)
    if len(pub) != 1 or len(grad) != 1:
        return "mixed publish or gradient dtypes"
    try:
        import torch.distributed._symmetric_memory as _symm  # noqa: F401
    except Exception as exc:  # pragma: no cover
        return f"symmetric memory unavailable: {exc}"
    return None


class PeerSource:
    """What the fused prologue needs to read one batch of gradients."""

    def __init__(self, rt: "PeerRuntime", dparams: list[DedicatedParam]):
        if rt.reduce_via == "nvls":
            # the in-switch sum of all ranks' slices already sits in ONE local buffer
            self.peer_bases = [rt.reduced_base]
        elif rt.reduce_via == "ce":
            # the peers' slices were gathered into local staging buffers during backward
            self.peer_bases = rt.stage_bases
        else:
            self.peer_bases = rt.grad_ptrs
        self.offsets = [p._arena_offset for p in dparams]
        self.numels = [p.numel for p in dparams]
        self.grad_dtype = rt.grad_dtype
        self.scale = 1.0 / rt.world
        self.ready_flags = rt.flags[KIND_GRAD_READY * MAX_PEERS :]
        self.ready_want = rt.grad_epoch + 1
        self.status = rt.status


def fused_forward_requested() -> bool:
    return os.environ.get("DMUON_FUSED_PUBLISH", "0").strip().lower() in ("1", "true", "yes", "on")


def _fused_linear_forward(self, x):
    """``nn.Linear.forward`` replacement: the first use of the weight in a
    publish epoch runs the kernel that pulls it from its owner while
    multiplying; later uses (recompute, second micro-batch) read the local copy."""
    import torch.nn.functional as F

    rt, p = self._dmuon_fused
    w = self.weight
    if p._fused_epoch != rt.pub_epoch and w.numel() == p.numel:
        from ..ops import pull_linear as PL

        if PL.supported(x, w):
            p._fused_epoch = rt.pub_epoch
            remote, flag, want, budget = rt.fused_pull_args(p)
            return PL.PulledLinearFn.apply(x, w, self.bias, remote, flag, want, budget)
        # unsupported input this time: fetch the weight the ordinary way first
        rt.pull_params([p])
        p._fused_epoch = rt.pub_epoch
    return F.linear(x, w, self.bias)


def direct_wgrad_requested() -> bool:
    return os.environ.get("DMUON_DIRECT_WGRAD", "1").strip().lower() in ("1", "true", "yes", "on")


class _LinearGradToArena(torch.autograd.Function):
    """``F.linear`` whose weight gradient is written by the backward GEMM
    straight into this rank's slot of the gradient arena (the memory the owner
    reads through its peer mapping), instead of into a fresh tensor that is
    packed into the arena afterwards.  Later micro-batches accumulate in place."""

    @staticmethod
    def forward(ctx, x, w, b, rt, p):
        ctx.save_for_backward(x, w)
        ctx.rt, ctx.p, ctx.has_bias = rt, p, b is not None
        return torch.nn.functional.linear(x, w, b)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        rt, p = ctx.rt, ctx.p
        dx = dw = db = None
        dy2 = dy.reshape(-1, dy.shape[-1])
        if ctx.needs_input_grad[0]:
            dx = (dy2 @ w).view(x.shape)
        if ctx.needs_input_grad[1]:
            x2 = x.reshape(-1, x.shape[-1])
            slot = p._grad_view
            if slot.dtype == dy2.dtype == x2.dtype:
                rt.before_pack()                    # owners are done with last step's slots (once per step)
                if p._peer_grad_pending:
                    slot.addmm_(dy2.t(), x2)
                else:
                    torch.mm(dy2.t(), x2, out=slot)
                    p._peer_grad_pending = True
                p._grad_in_arena = True
            else:
                dw = dy2.t() @ x2
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(dim=0)
        return dx, dw, db, None, None


def _direct_wgrad_linear_forward(self, x):
    rt, p = self._dmuon_direct
    w = self.weight
    if torch.is_grad_enabled() and w.requires_grad and w.numel() == p.numel and x.dtype == w.dtype:
        return _LinearGradToArena.apply(x, w, self.bias, rt, p)
    return torch.nn.functional.linear(x, w, self.bias)


class PeerRuntime:
    def __init__(self, ctx, dp_group, groups: list["PeerParamGroup"], fused_forward: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import gemm as G

        self.ctx = ctx
        self.group = dp_group
        self.device = ctx.device
        self.rank = dp_group.rank()
        self.world = dp_group.size()
        self.groups = groups
        params = [p for g in groups for p in g.bcast_params]
        self.param_dtype = params[0]._param_dtype
        self.grad_dtype = params[0]._grad_dtype or params[0]._param_dtype
        # Debug aid (DMUON_DEBUG_CANARY=1): a guard band of known words before the first
        # and after the last slot of both arenas; ``check()`` verifies them, which catches
        # a kernel (local or a peer's) that writes outside the slots it was given.
        self.canary = os.environ.get("DMUON_DEBUG_CANARY", "0").strip().lower() in ("1", "true", "yes", "on")
        self.guard = 4 * ALIGN if self.canary else 0
        off = self.guard
        # owner-major layout: one contiguous span per owner, groups in forward order inside it
        for s in range(self.world):
            for g in groups:
                for p in g._pub_by_shard.get(s, ()):
                    p._arena_offset = off
                    off += (p.numel + ALIGN - 1) // ALIGN * ALIGN
        self.payload_end = off
        self.total = max(off, ALIGN) + self.guard
        self.pub = symm_mem.empty(self.total, dtype=self.param_dtype, device=self.device)
        self.grad = symm_mem.empty(self.total, dtype=self.grad_dtype, device=self.device)
        # four global epoch rows, then one "gradients packed" row per group
        self.flags = symm_mem.empty((4 + len(groups)) * MAX_PEERS, dtype=torch.int32, device=self.device)
        self.reduce_mode = os.environ.get("DMUON_PEER_REDUCE", "backward").strip().lower()
        if self.reduce_mode not in ("backward", "optimizer"):
            raise ValueError("DMUON_PEER_REDUCE must be 'backward' or 'optimizer'")
        for i, g in enumerate(groups):
            g._group_index = i
        # scratch of the in-kernel scalar all-reduce (clip norms): values and flags, two parities each
        self.sc_vals = symm_mem.empty(2 * 8, dtype=torch.float32, device=self.device)
        self.sc_flags = symm_mem.empty(2 * MAX_PEERS, dtype=torch.int32, device=self.device)
        self.sc_vals.zero_()
        self.sc_flags.zero_()
        self.sc_epoch = 0
        self.flags.zero_()
        self.grad.zero_()
        if self.canary:
            for arena in (self.pub, self.grad):
                arena[: self.guard].fill_(CANARY_VALUE)
                arena[self.payload_end :].fill_(CANARY_VALUE)
        torch.cuda.synchronize(self.device)
        name = dp_group.group_name
        self.pub_hdl = symm_mem.rendezvous(self.pub, name)
        self.grad_hdl = symm_mem.rendezvous(self.grad, name)
        self.flag_hdl = symm_mem.rendezvous(self.flags, name)
        self.pub_ptrs = [int(p) for p in self.pub_hdl.buffer_ptrs]
        self.grad_ptrs = [int(p) for p in self.grad_hdl.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self.flag_hdl.buffer_ptrs]
        self.sc_val_ptrs = [int(p) for p in symm_mem.rendezvous(self.sc_vals, name).buffer_ptrs]
        self.sc_flag_ptrs = [int(p) for p in symm_mem.rendezvous(self.sc_flags, name).buffer_ptrs]
        self.status = G.status_buffer(self.device)
        self.pub_epoch = 0
        self.grad_epoch = 0
        self._grads_signalled = False
        self._consumed_wait_queued = False
        self._pulled_groups = 0
        esz = self.pub.element_size()
        for g in groups:
            g.runtime = self
            for p in g.bcast_params:
                view = self.pub[p._arena_offset : p._arena_offset + p.numel].view(p._orig_size)
                p.make_unsharded_param(view)
                p._grad_view = self.grad[p._arena_offset : p._arena_offset + p.numel].view(p._orig_size)
                p._publish_view = view if p.is_owner else None
                p._peer_grad_pending = False
        self._remote_groups = sum(1 for g in groups if any(s != self.rank for s in g._pub_by_shard))
        self.fused_forward = fused_forward_requested() if fused_forward is None else bool(fused_forward)
        # How bulk data crosses NVLink: "ce" (default) uses copy-engine transfers -- publish pulls and a
        # gather of the peers' gradient slices into local staging buffers, the sum then happens locally
        # inside the Muon prologue -- so no SM is taken from the forward / backward GEMMs; "sm" uses the
        # pull / reduce kernels that load through the peer mappings themselves.
        self.pub_mc = int(getattr(self.pub_hdl, "multicast_ptr", 0) or 0)
        self.grad_mc = int(getattr(self.grad_hdl, "multicast_ptr", 0) or 0)
        self.copy_mode = os.environ.get("DMUON_PEER_COPY", "auto").strip().lower()
        if self.copy_mode not in ("auto", "nvls", "hybrid", "ce", "sm"):
            raise ValueError("DMUON_PEER_COPY must be 'auto', 'nvls', 'hybrid', 'ce' or 'sm'")
        if self.fused_forward:
            self.copy_mode = "sm"       # the fused forward kernels do their own fetching
        if self.copy_mode == "auto":
            self.copy_mode = AUTO_COPY_MODE
        if self.copy_mode in ("nvls", "hybrid"):
            # every rank must take the same decision: all need a multicast mapping of both arenas
            ok = torch.tensor(
                [int(self.pub_mc != 0 and self.grad_mc != 0 and self.pub.element_size() == 2)], device=self.device
            )
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=dp_group)
            if not bool(ok.item()):
                if os.environ.get("DMUON_PEER_COPY", "auto").strip().lower() in ("nvls", "hybrid"):
                    raise RuntimeError(
                        f"DMUON_PEER_COPY={self.copy_mode}: the symmetric arenas have no NVSwitch multicast mapping on "
                        "every rank (or the published dtype is not 16-bit)"
                    )
                self.copy_mode = "ce"
        # which mechanism carries each of the two bulk transfers
        self.reduce_via = {"nvls": "nvls", "hybrid": "nvls", "ce": "ce", "sm": "sm"}[self.copy_mode]
        self.publish_via = {"nvls": "nvls", "hybrid": "ce", "ce": "ce", "sm": "sm"}[self.copy_mode]
        for g in groups:
            g._span_by_owner = {}
            for s_, plist in g._pub_by_shard.items():
                lo = min(p._arena_offset for p in plist)
                hi = max(p._arena_offset + (p.numel + ALIGN - 1) // ALIGN * ALIGN for p in plist)
                g._span_by_owner[s_] = (lo, hi)
        mine = [sp[self.rank] for sp in (g._span_by_owner for g in groups) if self.rank in sp]
        self.own_lo = min((lo for lo, _ in mine), default=0)
        self.own_hi = max((hi for _, hi in mine), default=0)
        self.stage = None
        self.stage_bases = list(self.grad_ptrs)
        self.reduced = None
        self.reduced_base = 0
        self._consumed_signalled_epoch = 0
        self._ready_waited_epoch = 0
        self.nvls_publish = nvls_publish_mode()
        self._publish_ticket = None
        if self.reduce_via == "nvls":
            span = max(self.own_hi - self.own_lo, ALIGN)
            self.reduced = torch.zeros(span, dtype=self.grad_dtype, device=self.device)
            # address of arena offset 0 in the reduced copy (only [own_lo, own_hi) is backed)
            self.reduced_base = self.reduced.data_ptr() - self.own_lo * self.grad.element_size()
        if self.reduce_via == "ce" and self.own_hi > self.own_lo and self.world > 1:
            span = self.own_hi - self.own_lo
            self.stage = torch.empty((self.world - 1) * span, dtype=self.grad_dtype, device=self.device)
            gsz = self.grad.element_size()
            k = 0
            for r in range(self.world):
                if r == self.rank:
                    continue
                # address of arena offset 0 in rank r's staged copy (only [own_lo, own_hi) is backed)
                self.stage_bases[r] = self.stage.data_ptr() + (k * span - self.own_lo) * gsz
                k += 1
        if self.fused_forward:
            self._install_fused_linears()
        self.direct_wgrad = direct_wgrad_requested() and not self.fused_forward
        if self.direct_wgrad:
            self._install_direct_wgrad_linears()
        dist.barrier(group=dp_group)
        self.publish_owned()

    # ------------------------------------------------------------------ fused forward publish
    def _install_fused_linears(self) -> None:
        """Give every plain ``nn.Linear`` whose weight is a dedicated parameter
        owned by ANOTHER rank a forward that pulls the weight inside its GEMM.
        Anything else (shared weights, custom modules, direct ``.weight`` use)
        keeps the pull-then-compute path."""
        import types

        import torch.nn as nn

        for g in self.groups:
            for p in g.bcast_params:
                p._fused_linear = False
                if p.is_owner or len(p.alias_sites) != 1 or len(p._orig_size) != 2 or p._param_dtype != torch.bfloat16:
                    continue
                mod, attr = p.alias_sites[0]
                if type(mod) is not nn.Linear or attr != "weight" or p._orig_size[1] % 32 != 0:
                    continue
                p._fused_linear = True
                p._fused_epoch = -1
                mod._dmuon_fused = (self, p)
                mod.forward = types.MethodType(_fused_linear_forward, mod)

    def _install_direct_wgrad_linears(self) -> None:
        """Plain ``nn.Linear`` modules whose weight is a dedicated matrix get a
        forward whose backward writes the weight gradient into the arena slot.
        Shared weights, custom modules and direct ``.weight`` use keep the
        ordinary autograd path (their gradients are packed afterwards)."""
        import types

        import torch.nn as nn

        for g in self.groups:
            for p in g.bcast_params:
                p._grad_in_arena = False
                if len(p.alias_sites) != 1 or len(p._orig_size) != 2:
                    continue
                mod, attr = p.alias_sites[0]
                if type(mod) is not nn.Linear or attr != "weight":
                    continue
                mod._dmuon_direct = (self, p)
                mod.forward = types.MethodType(_direct_wgrad_linear_forward, mod)

    def fused_pull_args(self, p: DedicatedParam):
        esz = self.pub.element_size()
        remote = self.pub_ptrs[p.owner_shard] + p._arena_offset * esz
        flag = self.flags[KIND_PUB_READY * MAX_PEERS + p.owner_shard :]
        from ..ops import peer as P

        return remote, flag, self.pub_epoch, P.wait_budget_cycles()

    # ------------------------------------------------------------------ helpers
    def _signal(self, kind: int, value: int) -> None:
        from ..ops import peer as P

        P.signal_peers(self.flag_ptrs, kind * MAX_PEERS + self.rank, value, self.device)

    def _wait_all(self, kind: int, want: int) -> None:
        from ..ops import peer as P

        P.wait_flags(self.flags, kind * MAX_PEERS, self.world, want, self.status)

    def scalar_allreduce(self, local: torch.Tensor, max_norm: Optional[float] = None):
        """Sum up to 8 fp32 scalars over the ranks of this plane inside one
        kernel (symmetric scratch rows + flags, bounded wait); returns
        ``(sums, clip_coefficients or None)``.  Every rank must call it the
        same number of times."""
        from ..ops import peer as P

        local = local.reshape(-1).float().contiguous()
        out = torch.empty_like(local)
        coef = torch.empty_like(local) if max_norm is not None else None
        self.sc_epoch += 1
        P.scalar_allreduce(self.sc_val_ptrs, self.sc_flag_ptrs, self.rank, self.sc_epoch, local, out, self.status,
                           coef=coef, max_norm=float(max_norm or 0.0))
        return out, coef

    def check(self) -> None:
        """Synchronising status check (raises KernelTimeout when a wait gave up;
        with ``DMUON_DEBUG_CANARY=1`` also verifies the guard bands of the arenas)."""
        from ..ops import gemm as G

        G.check_status(self.device)
        if self.canary:
            for name, arena in (("publish", self.pub), ("gradient", self.grad)):
                lo, hi = arena[: self.guard], arena[self.payload_end :]
                if not (bool((lo == CANARY_VALUE).all()) and bool((hi == CANARY_VALUE).all())):
                    raise RuntimeError(f"rank {self.rank}: the guard band of the {name} arena was overwritten")

    # ------------------------------------------------------------------ publish side
    def before_owner_writes(self) -> None:
        """Queue the wait that protects readers still pulling the current epoch."""
        with record_function(f"dmuon.peer.before_owner_writes.epoch{self.pub_epoch}"):
            self._before_owner_writes()

    def _before_owner_writes(self) -> None:
        if self.publish_via == "nvls":
            # Owners store straight into every rank's arena, so "consumed" means: this rank has
            # finished every forward / backward that reads the current weights.  That is true at
            # this point of the current stream (the optimizer step or a checkpoint load follows).
            self._acknowledge_epoch()
            self._wait_all(KIND_PUB_CONSUMED, self.pub_epoch)
            return
        # a group whose forward did not run this epoch still has to acknowledge it
        lane = self.ctx.broadcast_lane
        pending = [g for g in self.groups if g._pulled_epoch != self.pub_epoch]
        if pending:
            lane.follow_current()
            with lane.use():
                for g in pending:
                    self.pull_group(g)
            lane.mark().wait_on_current()
        if self.fused_forward:
            # fused linears acknowledge from announce_grads(), which needs a backward; without one in
            # this epoch (checkpoint load right after construction, evaluation only) do it here, after
            # the pulls queued above
            self._acknowledge_epoch()
        if self.pub_epoch > 0:
            self._wait_all(KIND_PUB_CONSUMED, self.pub_epoch)

    def _acknowledge_epoch(self) -> None:
        """Tell every owner, once per publish epoch, that this rank no longer
        needs the epoch's weights to stay as they are (stream-ordered)."""
        if self._consumed_signalled_epoch != self.pub_epoch:
            self._signal(KIND_PUB_CONSUMED, self.pub_epoch)
            self._consumed_signalled_epoch = self.pub_epoch

    def publish_owned(self) -> None:
        """Bring the owner's publish slots up to date and announce the new epoch."""
        from ..ops import multi_tensor as MT

        stale = [p for g in self.groups for p in g.bcast_params if p.is_owner and not p._publish_fresh]
        with record_function(f"dmuon.peer.publish_owned.{self.copy_mode}.epoch{self.pub_epoch + 1}.stale{len(stale)}"):
            self._publish_owned(stale, MT)

    def _multicast_slots(self, plist: list[DedicatedParam], blocks: int = 0) -> None:
        """Store the local publish slots of ``plist`` to every rank's arena
        (current stream); adjacent slots travel as one span."""
        from ..ops import peer as P

        esz = self.pub.element_size()
        spans: list[list[int]] = []
        for p in sorted(plist, key=lambda q: q._arena_offset):
            lo = p._arena_offset * esz
            hi = lo + (p.numel + ALIGN - 1) // ALIGN * ALIGN * esz
            if spans and spans[-1][1] == lo:
                spans[-1][1] = hi
            else:
                spans.append([lo, hi])
        P.multicast_broadcast([self.pub.data_ptr() + lo for lo, _ in spans], [self.pub_mc + lo for lo, _ in spans],
                              [hi - lo for lo, hi in spans], self.device, blocks_per_tensor=blocks)

    def multicast_publish_async(self, plist: list[DedicatedParam]) -> None:
        """NVSwitch plane, ``lane`` mode: the update kernel has just written the
        local slots of ``plist``; replicate them to all ranks on the publish
        lane while the optimizer goes on with the next batch."""
        lane = self.ctx.broadcast_lane
        lane.follow_current()
        with lane.use(), record_function(f"dmuon.peer.multicast_publish.params{len(plist)}"):
            self._multicast_slots(plist, NVLS_PUBLISH_BLOCKS)
        self._publish_ticket = lane.mark()

    def _publish_owned(self, stale, MT) -> None:
        if stale:
            srcs = [p._owned_data.reshape(-1) for p in stale]
            dsts = [p._publish_view.reshape(-1) for p in stale]
            with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(tuple(p._unsharded_param for p in stale)):
                if srcs[0].dtype in MT._DT and dsts[0].dtype in MT._DT:
                    MT.cast(srcs, dsts)
                else:
                    torch._foreach_copy_(dsts, srcs)
                if self.publish_via == "nvls":
                    # slots that were not multicast during the step (AdamW-routed tensors, the first
                    # publish, a checkpoint load): replicate the local copy to every rank's arena
                    self._multicast_slots(stale)
        if self._publish_ticket is not None:
            # multicast stores queued on the publish lane during the step must be complete before
            # the new epoch is announced
            self._publish_ticket.wait_on_current()
            self._publish_ticket = None
        for g in self.groups:
            for p in g.bcast_params:
                p._publish_fresh = False
        self.pub_epoch += 1
        self._signal(KIND_PUB_READY, self.pub_epoch)
        self._pulled_groups = 0
        for g in self.groups:
            g._pulled_epoch = -1
        if self._remote_groups == 0 and self.publish_via != "nvls":
            # this rank reads nothing from anybody: acknowledge right away
            self._acknowledge_epoch()

    def pull_group(self, g: "PeerParamGroup") -> None:
        """Copy this group's slots from their owners into the local arena."""
        if g._pulled_epoch == self.pub_epoch:
            return
        with record_function(f"dmuon.peer.unshard.{self.copy_mode}.{g.name}"):
            self._pull_group(g)

    def _pull_group(self, g: "PeerParamGroup") -> None:
        from ..ops import peer as P

        if self.publish_via == "nvls":
            # the owners' stores already put the weights here: only wait (once per epoch and lane)
            # until every owner has announced the epoch
            if self._ready_waited_epoch != self.pub_epoch:
                P.wait_flags(self.flags, KIND_PUB_READY * MAX_PEERS, self.world, self.pub_epoch, self.status)
                self._ready_waited_epoch = self.pub_epoch
            g._pulled_epoch = self.pub_epoch
            return
        remote = [p for s, plist in g._pub_by_shard.items() if s != self.rank for p in plist]
        if remote:
            # weights consumed by a fused linear are fetched by that kernel instead
            self.pull_params([p for p in remote if not getattr(p, "_fused_linear", False)])
            self._pulled_groups += 1
            if self._pulled_groups == self._remote_groups and not self.fused_forward:
                self._acknowledge_epoch()
        g._pulled_epoch = self.pub_epoch

    def pull_params(self, plist: list[DedicatedParam]) -> None:
        """Copy the listed slots from their owners (current stream); adjacent
        slots of one owner travel as one span."""
        from ..ops import peer as P

        if not plist:
            return
        esz = self.pub.element_size()
        spans: list[list[int]] = []            # [owner, lo, hi] in elements
        for p in sorted(plist, key=lambda q: q._arena_offset):
            lo = p._arena_offset
            hi = lo + (p.numel + ALIGN - 1) // ALIGN * ALIGN
            if spans and spans[-1][0] == p.owner_shard and spans[-1][2] == lo:
                spans[-1][2] = hi
            else:
                spans.append([p.owner_shard, lo, hi])
        srcs = [self.pub_ptrs[s] + lo * esz for s, lo, _ in spans]
        dsts = [self.pub.data_ptr() + lo * esz for _, lo, _ in spans]
        nbytes = [(hi - lo) * esz for _, lo, hi in spans]
        slots = [KIND_PUB_READY * MAX_PEERS + s for s, _, _ in spans]
        live = tuple(p._unsharded_param for p in plist)
        with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(live):
            if self.publish_via == "ce":
                # one bounded wait for the owners' "published" flags, then copy-engine transfers
                P.wait_flags(self.flags, KIND_PUB_READY * MAX_PEERS, self.world, self.pub_epoch, self.status)
                for src, dst, nb in zip(srcs, dsts, nbytes):
                    P.copy_async(dst, src, nb, self.device)
            else:
                P.peer_pull(srcs, dsts, nbytes, slots, self.flags, self.pub_epoch, self.status, self.device,
                            blocks_per_tensor=max(4, 32 // len(srcs)))

    # ------------------------------------------------------------------ gradient side
    def before_pack(self) -> None:
        """First pack after an optimizer step: owners must be done reading."""
        if not self._consumed_wait_queued:
            if self.grad_epoch > 0:
                self._wait_all(KIND_GRAD_CONSUMED, self.grad_epoch)
            self._consumed_wait_queued = True

    def announce_grads(self) -> None:
        """All local gradients of this step are in the arena (stream-ordered)."""
        if not self._grads_signalled:
            self._signal(KIND_GRAD_READY, self.grad_epoch + 1)
            self._grads_signalled = True
            if self.fused_forward and self._remote_groups > 0:
                # fused linears pull on the compute stream during forward; this point
                # is stream-ordered after all of them
                self._acknowledge_epoch()

    # per-group reduce that overlaps with the rest of backward ("backward" mode)
    def signal_group_packed(self, g: "PeerParamGroup", count: int) -> None:
        from ..ops import peer as P

        P.signal_peers(self.flag_ptrs, (4 + g._group_index) * MAX_PEERS + self.rank, count, self.device)

    def launch_group_reduce(self, g: "PeerParamGroup", owned: list[DedicatedParam], count: int):
        """Queue, on the reduce lane, the kernel that sums this group's owned
        gradients over all ranks' arenas as soon as every rank has packed them."""
        with record_function(f"dmuon.peer.reduce.{self.copy_mode}.{g.name}.params{len(owned)}"):
            return self._launch_group_reduce(g, owned, count)

    def _launch_group_reduce(self, g: "PeerParamGroup", owned: list[DedicatedParam], count: int):
        from ..ops import peer as P

        lane = self.ctx.reduce_lane
        if self.reduce_via == "nvls":
            # one reduce-load per 16 bytes returns the sum over ALL ranks' arenas, formed in the switch:
            # the owner ingests its span once, not once per peer, and keeps a single reduced copy
            lo, hi = g._span_by_owner[self.rank]
            gsz = self.grad.element_size()
            lane.follow_current()
            with lane.use():
                P.wait_flags(self.flags, (4 + g._group_index) * MAX_PEERS, self.world, count, self.status)
                P.multicast_reduce([self.grad_mc + lo * gsz], [self.reduced_base + lo * gsz], [(hi - lo) * gsz],
                                   self.grad_dtype, self.device, blocks_per_tensor=NVLS_REDUCE_BLOCKS)
            return lane.mark()
        if self.reduce_via == "ce":
            # gather instead of reduce: bring every peer's slice of this group's owned span into the
            # local staging buffers with copy-engine transfers; the Muon prologue sums them later
            lo, hi = g._span_by_owner[self.rank]
            gsz = self.grad.element_size()
            lane.follow_current()
            with lane.use():
                P.wait_flags(self.flags, (4 + g._group_index) * MAX_PEERS, self.world, count, self.status)
                for r in range(self.world):
                    if r != self.rank:
                        P.copy_async(self.stage_bases[r] + lo * gsz, self.grad_ptrs[r] + lo * gsz, (hi - lo) * gsz, self.device)
            return lane.mark()
        for p in owned:
            if getattr(p, "_reduce_buf", None) is None:
                p._reduce_buf = torch.empty(p._orig_size, dtype=torch.float32, device=self.device)
        lane.follow_current()
        src = self.source_for(owned)
        base = (4 + g._group_index) * MAX_PEERS
        with lane.use():
            P.peer_prologue(src.peer_bases, src.offsets, src.numels, src.grad_dtype, [None] * len(owned),
                            [p._reduce_buf.reshape(-1) for p in owned], [0] * len(owned), None, scale=src.scale,
                            mu=0.0, nesterov=False, ready_flags=self.flags[base:], ready_want=count,
                            status=self.status, max_blocks_per_tensor=REDUCE_BLOCKS_PER_TENSOR)
        return lane.mark()

    def source_for(self, dparams: list[DedicatedParam]) -> PeerSource:
        return PeerSource(self, dparams)

    def materialize(self, dparams: list[DedicatedParam]) -> None:
        """Reduce the listed gradients into plain fp32 tensors on the owner
        (clip, AdamW-routed and PyTorch Newton-Schulz paths)."""
        from ..ops import peer as P

        todo = [p for p in dparams if p.is_owner and p._peer_grad_pending and p._reduced_grad is None]
        if not todo:
            return
        with record_function(f"dmuon.peer.materialize_reduced_grads.params{len(todo)}"):
            self._materialize(todo)

    def _materialize(self, todo: list[DedicatedParam]) -> None:
        from ..ops import peer as P

        outs = [torch.empty(p._orig_size, dtype=torch.float32, device=self.device) for p in todo]
        src = self.source_for(todo)
        P.peer_prologue(src.peer_bases, src.offsets, src.numels, src.grad_dtype, [None] * len(todo),
                        [o.reshape(-1) for o in outs], [0] * len(todo), None, scale=src.scale, mu=0.0,
                        nesterov=False, ready_flags=src.ready_flags, ready_want=src.ready_want, status=src.status)
        for p, o in zip(todo, outs):
            p._reduced_grad = o
            p._peer_grad_pending = False

    def after_optimizer_consumed(self) -> None:
        """Every owned gradient of this step has been read: let peers overwrite."""
        if self._grads_signalled:
            self.grad_epoch += 1
            self._signal(KIND_GRAD_CONSUMED, self.grad_epoch)
        self._grads_signalled = False
        self._consumed_wait_queued = False
        for g in self.groups:
            g._packed_this_step = False
            for p in g.bcast_params:
                p._peer_grad_pending = False


class PeerParamGroup(DedicatedParamGroup):
    """Same role as :class:`DedicatedParamGroup`, data moved by peer kernels."""

    mode = "fsdp"
    uses_peer_memory = True

    def __init__(self, *args, **kwargs):
        self.runtime: Optional[PeerRuntime] = None
        self._pulled_epoch = -1
        self._packed_this_step = False
        self._pack_count = 0
        self._reduce_ticket = None
        self._reduce_owned: list = []
        super().__init__(*args, **kwargs)

    def _build_packed_buffers(self) -> None:
        # slots live in the runtime's arenas; PeerRuntime wires them after all groups exist
        return

    def stage_publish_targets(self) -> None:
        # publish slots are fixed arena views, wired once by the runtime
        return

    def unshard(self, prefetch: bool = False) -> None:
        if self._is_unsharded or self._unshard_ticket is not None:
            return
        rt = self.runtime
        lane = self.comm_ctx.broadcast_lane
        lane.follow_current()
        with lane.use():
            rt.pull_group(self)
        self._unshard_ticket = lane.mark()
        self._prefetched = prefetch

    def wait_for_unshard(self) -> None:
        if self._unshard_ticket is not None:
            self._unshard_ticket.wait_on_current()
            self._unshard_ticket = None
        if not self._is_unsharded:
            for p in self.params:
                p.attach_to_modules()
                p._is_unsharded = True
            self._is_unsharded = True

    def reshard(self) -> None:
        # the arena is persistent: only the bookkeeping changes, so that the next
        # forward pulls the next published epoch
        if self._unshard_ticket is not None:
            self._unshard_ticket.wait_on_current()
            self._unshard_ticket = None
        self._is_unsharded = False

    def reduce_grads(self) -> None:
        with_grad = [(p, p.local_grad()) for p in self.bcast_params]
        # gradients the backward GEMMs already wrote into the arena
        direct = [p for p, g in with_grad if getattr(p, "_grad_in_arena", False)]
        if _dgroup.ZERO_FILL_MISSING_GRADS and not self._no_sync:
            # a slot nobody wrote would still hold last step's gradient when the owner sums the arenas
            with_grad = [(p, g) if (g is not None or getattr(p, "_grad_in_arena", False)) else
                         _dgroup.zero_fill_missing([(p, None)], self.device)[0] for p, g in with_grad]
        if _dgroup.CHECK_GRAD_PRESENCE and not self._no_sync and len(self.bcast_params) == len(self.params):
            # debugging aid: a rank that produced no gradient for a slot leaves LAST step's data there for the owner to sum
            self.check_grad_presence([g is not None or getattr(p, "_grad_in_arena", False) for p, g in with_grad])
        with_grad = [(p, g) for p, g in with_grad if g is not None]
        if not with_grad and not direct:
            return
        rt = self.runtime
        for p in direct:
            p._grad_in_arena = False
        with torch.no_grad(), record_function(f"dmuon.peer.pack_grads.{self.name}.copied{len(with_grad)}.direct{len(direct)}"):
            rt.before_pack()
            dsts = [p._grad_view for p, _ in with_grad]
            srcs = [g for _, g in with_grad]
            fresh = [i for i, (p, _) in enumerate(with_grad) if not p._peer_grad_pending]
            again = [i for i, (p, _) in enumerate(with_grad) if p._peer_grad_pending]
            if fresh:
                torch._foreach_copy_([dsts[i] for i in fresh], [srcs[i] for i in fresh])
            if again:      # gradient accumulation: later micro-batches add up locally
                torch._foreach_add_([dsts[i] for i in again], [srcs[i].to(dsts[i].dtype) for i in again])
            for p, _ in with_grad:
                p._peer_grad_pending = True
                p.clear_local_grad()
        self._packed_this_step = True
        if (rt.reduce_mode == "backward" or rt.reduce_via in ("ce", "nvls")) and not self._no_sync:
            # tell every rank this group's running sum is in the arena, then (as an
            # owner) reduce it on the side lane while backward continues.  A later
            # micro-batch repeats this and overwrites the result with the larger sum.
            self._pack_count += 1
            rt.signal_group_packed(self, self._pack_count)
            seen = {id(p) for p, _ in with_grad}
            owned = [p for p, _ in with_grad if p.is_owner] + [p for p in direct if p.is_owner and id(p) not in seen]
            if owned:
                self._reduce_ticket = rt.launch_group_reduce(self, owned, self._pack_count)
                # after a copy-engine gather the sum is still to be done (inside the Muon prologue); after
                # an in-switch reduce the scale, momentum and cast are
                self._reduce_owned = owned if rt.reduce_via == "sm" else []

    def has_pending_reduce(self) -> bool:
        if self._reduce_ticket is not None:
            return True
        return self._packed_this_step and not self.runtime._grads_signalled

    def wait_for_stage1_reduce(self) -> None:
        return      # reduce kernels only read; nothing to throttle

    def wait_for_reduce(self, lane=None) -> None:
        if self._reduce_ticket is not None:
            if lane is not None:
                self._reduce_ticket.wait_on(lane)
            else:
                self._reduce_ticket.wait_on_current()
            self._reduce_ticket = None
            for p in self._reduce_owned:
                p._reduced_grad = p._reduce_buf
            self._reduce_owned = []
        # "optimizer" mode: nothing travels until the owner's prologue reads the
        # arenas; the "gradients ready" epoch is announced after the last pack
        self.runtime.announce_grads()

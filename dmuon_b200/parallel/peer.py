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

from .dgroup import DedicatedParamGroup
from .dparam import DedicatedParam

KIND_GRAD_READY, KIND_GRAD_CONSUMED, KIND_PUB_READY, KIND_PUB_CONSUMED = 0, 1, 2, 3
MAX_PEERS = 8
ALIGN = 64          # elements; keeps every slot 128-byte aligned for bf16


def peer_backend_requested() -> str:
    return os.environ.get("DMUON_COMM_BACKEND", "auto").strip().lower()


def peer_backend_possible(device: torch.device, dp_group, replicate_group, dparams) -> Optional[str]:
    """None when usable, else the reason it is not."""
    if device.type != "cuda":
        return "not a CUDA device"
    if dp_group is None or dp_group.size() < 2:
        return "single rank"
    if dp_group.size() > MAX_PEERS:
        return f"more than {MAX_PEERS} ranks on the shard axis"
    if replicate_group is not None and replicate_group.size() > 1:
        return "replicate axis present"
    if any(p.tp_group is not None for p in dparams):
        return "tensor-parallel parameters"
    if any(p._dmuon_route == "sharded_adamw" for p in dparams):
        return "sharded_adamw route"
    if len({p._param_dtype for p in dparams}) != 1 or len({p._grad_dtype or p._param_dtype for p in dparams}) != 1:
        return "mixed publish or gradient dtypes"
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception as exc:  # pragma: no cover
        return f"symmetric memory unavailable: {exc}"
    return None


class PeerSource:
    """What the fused prologue needs to read one batch of gradients."""

    def __init__(self, rt: "PeerRuntime", dparams: list[DedicatedParam]):
        self.peer_bases = rt.grad_ptrs
        self.offsets = [p._arena_offset for p in dparams]
        self.numels = [p.numel for p in dparams]
        self.grad_dtype = rt.grad_dtype
        self.scale = 1.0 / rt.world
        self.ready_flags = rt.flags[KIND_GRAD_READY * MAX_PEERS :]
        self.ready_want = rt.grad_epoch + 1
        self.status = rt.status


class PeerRuntime:
    def __init__(self, ctx, dp_group, groups: list["PeerParamGroup"]):
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
        off = 0
        # owner-major layout: one contiguous span per owner, groups in forward order inside it
        for s in range(self.world):
            for g in groups:
                for p in g._pub_by_shard.get(s, ()):
                    p._arena_offset = off
                    off += (p.numel + ALIGN - 1) // ALIGN * ALIGN
        self.total = max(off, ALIGN)
        self.pub = symm_mem.empty(self.total, dtype=self.param_dtype, device=self.device)
        self.grad = symm_mem.empty(self.total, dtype=self.grad_dtype, device=self.device)
        self.flags = symm_mem.empty(4 * MAX_PEERS, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self.grad.zero_()
        torch.cuda.synchronize(self.device)
        name = dp_group.group_name
        self.pub_hdl = symm_mem.rendezvous(self.pub, name)
        self.grad_hdl = symm_mem.rendezvous(self.grad, name)
        self.flag_hdl = symm_mem.rendezvous(self.flags, name)
        self.pub_ptrs = [int(p) for p in self.pub_hdl.buffer_ptrs]
        self.grad_ptrs = [int(p) for p in self.grad_hdl.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self.flag_hdl.buffer_ptrs]
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
        dist.barrier(group=dp_group)
        self.publish_owned()

    # ------------------------------------------------------------------ helpers
    def _signal(self, kind: int, value: int) -> None:
        from ..ops import peer as P

        P.signal_peers(self.flag_ptrs, kind * MAX_PEERS + self.rank, value, self.device)

    def _wait_all(self, kind: int, want: int) -> None:
        from ..ops import peer as P

        P.wait_flags(self.flags, kind * MAX_PEERS, self.world, want, self.status)

    def check(self) -> None:
        """Synchronising status check (raises KernelTimeout when a wait gave up)."""
        from ..ops import gemm as G

        G.check_status(self.device)

    # ------------------------------------------------------------------ publish side
    def before_owner_writes(self) -> None:
        """Queue the wait that protects readers still pulling the current epoch."""
        # a group whose forward did not run this epoch still has to acknowledge it
        lane = self.ctx.broadcast_lane
        pending = [g for g in self.groups if g._pulled_epoch != self.pub_epoch]
        if pending:
            lane.follow_current()
            with lane.use():
                for g in pending:
                    self.pull_group(g)
            lane.mark().wait_on_current()
        if self.pub_epoch > 0:
            self._wait_all(KIND_PUB_CONSUMED, self.pub_epoch)

    def publish_owned(self) -> None:
        """Bring the owner's publish slots up to date and announce the new epoch."""
        from ..ops import multi_tensor as MT

        stale = [p for g in self.groups for p in g.bcast_params if p.is_owner and not p._publish_fresh]
        if stale:
            srcs = [p._owned_data.reshape(-1) for p in stale]
            dsts = [p._publish_view.reshape(-1) for p in stale]
            with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(tuple(p._unsharded_param for p in stale)):
                if srcs[0].dtype in MT._DT and dsts[0].dtype in MT._DT:
                    MT.cast(srcs, dsts)
                else:
                    torch._foreach_copy_(dsts, srcs)
        for g in self.groups:
            for p in g.bcast_params:
                p._publish_fresh = False
        self.pub_epoch += 1
        self._signal(KIND_PUB_READY, self.pub_epoch)
        self._pulled_groups = 0
        for g in self.groups:
            g._pulled_epoch = -1
        if self._remote_groups == 0:
            # this rank reads nothing from anybody: acknowledge right away
            self._signal(KIND_PUB_CONSUMED, self.pub_epoch)

    def pull_group(self, g: "PeerParamGroup") -> None:
        """Copy this group's slots from their owners into the local arena."""
        from ..ops import peer as P

        if g._pulled_epoch == self.pub_epoch:
            return
        srcs, dsts, nbytes, slots = [], [], [], []
        esz = self.pub.element_size()
        for s, plist in g._pub_by_shard.items():
            if s == self.rank:
                continue
            # the parameters of one owner inside one group are adjacent: one copy per owner
            lo = min(p._arena_offset for p in plist)
            hi = max(p._arena_offset + (p.numel + ALIGN - 1) // ALIGN * ALIGN for p in plist)
            srcs.append(self.pub_ptrs[s] + lo * esz)
            dsts.append(self.pub.data_ptr() + lo * esz)
            nbytes.append((hi - lo) * esz)
            slots.append(KIND_PUB_READY * MAX_PEERS + s)
        if srcs:
            live = tuple(p._unsharded_param for p in g.bcast_params)
            with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(live):
                P.peer_pull(srcs, dsts, nbytes, slots, self.flags, self.pub_epoch, self.status, self.device,
                            blocks_per_tensor=max(4, 32 // len(srcs)))
            self._pulled_groups += 1
            if self._pulled_groups == self._remote_groups:
                self._signal(KIND_PUB_CONSUMED, self.pub_epoch)
        g._pulled_epoch = self.pub_epoch

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

    def source_for(self, dparams: list[DedicatedParam]) -> PeerSource:
        return PeerSource(self, dparams)

    def materialize(self, dparams: list[DedicatedParam]) -> None:
        """Reduce the listed gradients into plain fp32 tensors on the owner
        (clip, AdamW-routed and PyTorch Newton-Schulz paths)."""
        from ..ops import peer as P

        todo = [p for p in dparams if p.is_owner and p._peer_grad_pending and p._reduced_grad is None]
        if not todo:
            return
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
        super().__init__(*args, **kwargs)

    def _build_packed_buffers(self) -> None:
        # slots live in the runtime's arenas; PeerRuntime wires them after all groups exist
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
        with_grad = [(p, g) for p, g in with_grad if g is not None]
        if not with_grad:
            return
        rt = self.runtime
        with torch.no_grad():
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

    def has_pending_reduce(self) -> bool:
        return self._packed_this_step and not self.runtime._grads_signalled

    def wait_for_reduce(self, lane=None) -> None:
        # nothing travels until the owner's prologue reads the arenas; make sure
        # the "gradients ready" epoch is announced after the last pack
        self.runtime.announce_grads()

"""Tensor-parallel gather and scatter of the Muon path over peer memory.

A matrix sharded over the ``T`` ranks of a tensor-parallel group is
orthogonalised as a whole by its TP owner.  The collective implementation
(``dgroup.tp_gather_grads`` / ``tp_scatter_delta``) moves the shards with NCCL
``gather`` / ``scatter`` and builds the full gradient with ``torch.cat``.  On
one NVSwitch domain this module replaces both moves:

gather   every rank of the data-parallel owner column copies its reduced shard
         into a symmetric buffer and raises a flag.  The TP owner's Muon
         prologue then reads each shard where it lies -- through the peer
         mapping -- and writes momentum, Nesterov mix, cast operand and sum of
         squares directly into the rows / columns the shard occupies in the
         full matrix.  No concatenated gradient exists at any time.
scatter  the owner's last Newton-Schulz product writes the pre-scaled update
         ``-lr * scale * NS(u)`` (fp32, full matrix) into a symmetric buffer;
         every rank pulls ITS slice through the peer mapping and applies
         ``w = w * (1 - lr*wd) + slice`` to its master shard in the same kernel.

Ordering: four monotonically increasing counters per rank in a symmetric flag
array (gradient shards ready / consumed, updates ready / consumed), written
with release and waited for with bounded acquire loops (status word on
time-out), exactly like the data-parallel peer plane.  Every rank of a TP
group runs the same sequence of gather and scatter calls, so "call number k"
is a consistent epoch on all of them.

Replaces dmuon/_backends/fsdp2/group.py:1376-1521 (gather, ``torch.cat``) and
:1536-1655 (scatter, fused ``mul_`` / ``add_``) of the reference.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
from torch.profiler import record_function

KIND_GRAD_READY, KIND_GRAD_CONSUMED, KIND_DELTA_READY, KIND_DELTA_CONSUMED = 0, 1, 2, 3
MAX_PEERS = 8
ALIGN = 64      # elements: keeps every slot 128-byte aligned for 16-bit types


def tp_peer_requested() -> bool:
    """``DMUON_TP_PEER`` (default on): use the peer-memory gather / scatter where
    the tensor-parallel group allows it."""
    return os.environ.get("DMUON_TP_PEER", "1").strip().lower() not in ("0", "false", "no", "off")


def tp_peer_possible(device: torch.device, tp_group) -> Optional[str]:
    """None when usable, else the reason it is not."""
    if device.type != "cuda":
        return "not a CUDA device"
    if tp_group is None or tp_group.size() < 2:
        return "single rank"
    if tp_group.size() > MAX_PEERS:
        return f"more than {MAX_PEERS} tensor-parallel ranks"
    from .peer import spans_hosts

    if dist.get_world_size() > torch.cuda.device_count() or spans_hosts():
        return "the job spans more than one host"
    try:
        import torch.distributed._symmetric_memory as _symm  # noqa: F401  (an alias: a plain "import torch.x" would
        # make "torch" a local name of this function and break the lines above)
    except Exception as exc:  # pragma: no cover
        return f"symmetric memory unavailable: {exc}"
    return None


class TPShardSource:
    """Stands where a gathered full gradient would stand (``dp._tp_full_grad``):
    the shards are still in the ranks' buffers and are read by the prologue."""

    dtype = "tp_peer"

    def __init__(self, exchange: "TPPeerExchange", dparam):
        self.exchange, self.dparam = exchange, dparam
        self.shape = torch.Size(dparam.full_shape)

    def numel(self) -> int:
        return int(self.shape.numel())

    def materialize(self) -> torch.Tensor:
        """The full gradient as an ordinary fp32 tensor (clipping, PyTorch paths)."""
        return self.exchange.materialize(self.dparam)


class TPGatherSource:
    """What the batched Muon update needs to read one batch of sharded gradients."""

    def __init__(self, sources: list[TPShardSource]):
        self.sources = sources
        self.exchange = sources[0].exchange

    def launch_prologue(self, moms, xs_out, slots, sumsq, *, mu, nesterov, gscale=None, xscale=None) -> None:
        self.exchange.gather_prologue([s.dparam for s in self.sources], moms, xs_out, slots, sumsq, mu=mu,
                                      nesterov=nesterov, gscale=gscale, xscale=xscale)


class TPPeerExchange:
    """Symmetric buffers and flags of ONE tensor-parallel group."""

    def __init__(self, ctx, tp_group, dparams: list):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import gemm as G

        self.ctx, self.group, self.device = ctx, tp_group, ctx.device
        self.rank, self.world = tp_group.rank(), tp_group.size()
        self.params = [p for p in dparams if p._dmuon_route == "muon"]
        # gradient slots: the reduced shards this rank holds as a member of the DP owner column.  Which
        # parameters those are, and how large each local shard is, is the same on all ranks of the group.
        off = 0
        self.grad_dtype = None
        for p in self.params:
            p._tp_grad_offset = None
            if p.is_owner:
                p._tp_grad_offset = off
                off += (p.numel + ALIGN - 1) // ALIGN * ALIGN
                gd = p._grad_dtype or p._param_dtype or p._orig_dtype
                if self.grad_dtype is None:
                    self.grad_dtype = gd
                elif gd != self.grad_dtype:
                    raise ValueError("tensor-parallel peer exchange needs one gradient dtype per TP group")
        self.grad_dtype = self.grad_dtype or torch.bfloat16
        self.grad_total = max(off, ALIGN)
        # update slots: full fp32 matrices of the parameters this rank is TP owner (and DP owner) of; the
        # layout differs per rank, readers compute the owner's offsets from the common parameter order
        self.delta_offsets: dict[int, int] = {}
        per_rank = [0] * self.world
        for p in self.params:
            if p.is_owner:
                r = p._tp_owner_local_rank
                self.delta_offsets[id(p)] = per_rank[r]
                per_rank[r] += (int(p.full_shape.numel()) + ALIGN - 1) // ALIGN * ALIGN
        need = torch.tensor([max(per_rank + [ALIGN])], dtype=torch.int64, device=self.device)
        dist.all_reduce(need, op=dist.ReduceOp.MAX, group=tp_group)       # symmetric: same size everywhere
        self.delta_total = int(need.item())
        self.grad = symm_mem.empty(self.grad_total, dtype=self.grad_dtype, device=self.device)
        self.delta = symm_mem.empty(self.delta_total, dtype=torch.float32, device=self.device)
        self.flags = symm_mem.empty(4 * MAX_PEERS, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        torch.cuda.synchronize(self.device)
        name = tp_group.group_name
        self.grad_ptrs = [int(x) for x in symm_mem.rendezvous(self.grad, name).buffer_ptrs]
        self.delta_ptrs = [int(x) for x in symm_mem.rendezvous(self.delta, name).buffer_ptrs]
        self.flag_ptrs = [int(x) for x in symm_mem.rendezvous(self.flags, name).buffer_ptrs]
        self.status = G.status_buffer(self.device)
        self.gather_epoch = 0         # gather calls issued so far (same number on every rank of the group)
        self.scatter_epoch = 0
        self._grad_waited_this_step = False
        self._gather_epoch_at_step_start = 0
        self._delta_waited_this_step = False
        self._gathered_since_step = False
        dist.barrier(group=tp_group)

    # ------------------------------------------------------------------ flags
    def _signal(self, kind: int, value: int) -> None:
        from ..ops import peer as P

        P.signal_peers(self.flag_ptrs, kind * MAX_PEERS + self.rank, value, self.device)

    def _wait_all(self, kind: int, want: int) -> None:
        from ..ops import peer as P

        if want > 0:
            P.wait_flags(self.flags, kind * MAX_PEERS, self.world, want, self.status)

    # ------------------------------------------------------------------ gather
    def publish_shards(self, dparams: list) -> None:
        """One gather call: copy the reduced shards of ``dparams`` (DP-owned
        here) into the symmetric buffer and announce them (current stream)."""
        from ..ops import multi_tensor as MT

        with record_function(f"dmuon.tp_peer.publish_shards.params{len(dparams)}"):
            if not self._grad_waited_this_step:
                # first gather after an optimizer step: the owners must be done reading the shards of the
                # step before (they announce that once, with the number of gathers that step had reached)
                self._wait_all(KIND_GRAD_CONSUMED, self._gather_epoch_at_step_start)
                self._grad_waited_this_step = True
            srcs, dsts = [], []
            for p in dparams:
                g = p._reduced_grad
                g = g if g.is_contiguous() else g.contiguous()
                srcs.append(g.reshape(-1))
                dsts.append(self.grad[p._tp_grad_offset : p._tp_grad_offset + p.numel])
            if srcs:
                if srcs[0].dtype in MT._DT and all(s.dtype == srcs[0].dtype for s in srcs):
                    MT.cast(srcs, dsts)
                else:
                    torch._foreach_copy_(dsts, srcs)
            self.gather_epoch += 1
            self._signal(KIND_GRAD_READY, self.gather_epoch)
            self._gathered_since_step = True
            for p in dparams:
                if p.is_tp_owner:
                    p._tp_full_grad = TPShardSource(self, p)

    def _jobs(self, dparams: list):
        from ..ops.tp_peer import ShardJob

        gsz = self.grad.element_size()
        jobs = []
        for i, p in enumerate(dparams):
            rows, cols = int(p.full_shape[0]), int(p.full_shape.numel() // p.full_shape[0])
            lrows = int(p._orig_size[0])
            lcols = p.numel // lrows
            for t in range(self.world):
                r_off = t * lrows if p.shard_dim == 0 else 0
                c_off = t * lcols if p.shard_dim != 0 else 0
                jobs.append(ShardJob(i, self.grad_ptrs[t] + p._tp_grad_offset * gsz, lrows, lcols,
                                     r_off * cols + c_off, cols))
        return jobs

    def gather_prologue(self, dparams, moms, xs_out, slots, sumsq, *, mu, nesterov, gscale=None, xscale=None) -> None:
        """Prologue of full matrices whose gradient shards are read from the
        ranks of the group (bounded wait for their "ready" flags first)."""
        from ..ops import tp_peer as K

        with record_function(f"dmuon.tp_peer.gather_prologue.params{len(dparams)}"):
            self._wait_all(KIND_GRAD_READY, self.gather_epoch)
            K.gather_prologue(self._jobs(dparams), self.grad_dtype, moms, xs_out, slots, sumsq, mu=mu,
                              nesterov=nesterov, gscale=gscale, xscale=xscale)

    def materialize(self, p) -> torch.Tensor:
        out = torch.empty(p.full_shape, dtype=torch.float32, device=self.device)
        self.gather_prologue([p], [None], [out.reshape(-1)], [0], None, mu=0.0, nesterov=False)
        p._tp_full_grad = out
        return out

    # ------------------------------------------------------------------ scatter
    def delta_view(self, p) -> torch.Tensor:
        """Where the TP owner's update of ``p`` goes (fp32, full shape)."""
        off = self.delta_offsets[id(p)]
        return self.delta[off : off + int(p.full_shape.numel())].view(p.full_shape)

    def before_delta_writes(self) -> None:
        """Once per step, before the first update is written: every rank must
        have applied the previous step's slices (within a step every parameter
        has its own slot, so nothing else needs protecting)."""
        if not self._delta_waited_this_step:
            self._wait_all(KIND_DELTA_CONSUMED, self.scatter_epoch)
            self._delta_waited_this_step = True

    def scatter_apply(self, dparams: list) -> None:
        """One scatter call (current stream): announce the updates this rank
        wrote as TP owner, then pull and apply this rank's slice of every
        parameter of ``dparams`` from its owner."""
        from ..ops import tp_peer as K

        with record_function(f"dmuon.tp_peer.scatter_apply.params{len(dparams)}"):
            for p in dparams:
                if p.is_tp_owner:
                    view = self.delta_view(p)
                    d = p._tp_full_delta
                    if d is None:
                        raise RuntimeError(f"{p.fqn}: the TP owner has no update to scatter")
                    if d.data_ptr() != view.data_ptr():
                        # produced outside the buffer (PyTorch Newton-Schulz path), on the compute stream;
                        # it is dropped below while this copy may still be queued on the scatter lane
                        self.before_delta_writes()
                        if d.is_cuda:
                            d.record_stream(torch.cuda.current_stream(d.device))
                        view.copy_(d.reshape(view.shape))
            self.scatter_epoch += 1
            self._signal(KIND_DELTA_READY, self.scatter_epoch)
            self._wait_all(KIND_DELTA_READY, self.scatter_epoch)
            srcs, pitches, dsts, decays = [], [], [], []
            for p in dparams:
                cols = int(p.full_shape.numel() // p.full_shape[0])
                lrows = int(p._orig_size[0])
                lcols = p.numel // lrows
                r_off = self.rank * lrows if p.shard_dim == 0 else 0
                c_off = self.rank * lcols if p.shard_dim != 0 else 0
                base = self.delta_ptrs[p._tp_owner_local_rank] + self.delta_offsets[id(p)] * 4
                srcs.append(base + (r_off * cols + c_off) * 4)
                pitches.append(cols)
                dsts.append(p._owned_data.view(lrows, lcols))
                decays.append(float(p._tp_wd_factor))
            K.apply_delta(srcs, pitches, dsts, decays)
            self._signal(KIND_DELTA_CONSUMED, self.scatter_epoch)
            for p in dparams:
                p._tp_full_delta = None
                p._tp_full_grad = None
                p._reduced_grad = None
                p._tp_gathered = False

    def after_step(self) -> None:
        """End of the optimizer step (current stream, after every prologue):
        peers may overwrite their gradient shards."""
        if self._gathered_since_step:
            self._signal(KIND_GRAD_CONSUMED, self.gather_epoch)
            self._gathered_since_step = False
        self._delta_waited_this_step = False
        self._grad_waited_this_step = False
        self._gather_epoch_at_step_start = self.gather_epoch

    def check(self) -> None:
        from ..ops import gemm as G

        G.check_status(self.device)

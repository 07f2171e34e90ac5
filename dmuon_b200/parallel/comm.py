"""Communication context shared by all dedicated-parameter groups of a model.

The context owns the side "lanes" communication runs on.  A lane is a CUDA
stream on a GPU and an inline no-op on CPU, so the same group code drives NCCL
on B200s and gloo in the CPU tests.  Ordering between lanes is expressed with
tickets (CUDA events on a GPU, nothing on CPU where every call completes
before it returns).

Lane roles and priorities follow the reference's five streams
(dmuon/_core/comm.py:98-110): publish and reduce lanes are high priority so
they are not starved by compute, the replicate-axis lanes run at default
priority.
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict
from typing import Optional

import torch


def _env_flag(name: str, default: bool = False) -> bool:
    raw = os.environ.get(name)
    if raw is None:
        return default
    return raw.strip().lower() not in ("", "0", "false", "no", "off")


class Ticket:
    """Completion marker of work queued on a lane."""

    __slots__ = ("event",)

    def __init__(self, event: Optional[torch.cuda.Event]):
        self.event = event

    def wait_on_current(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def wait_on(self, lane: "Lane") -> None:
        if self.event is not None and lane.stream is not None:
            lane.stream.wait_event(self.event)

    def done(self) -> bool:
        return True if self.event is None else self.event.query()

    def synchronize(self) -> None:
        if self.event is not None:
            self.event.synchronize()


class Lane:
    def __init__(self, device: torch.device, priority: int = 0):
        self.device = device
        self.stream = torch.cuda.Stream(device=device, priority=priority) if device.type == "cuda" else None

    def follow_current(self) -> None:
        """Work queued on this lane from now on runs after what the current
        stream has queued so far."""
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))

    def follow(self, other: "Lane") -> None:
        if self.stream is not None and other.stream is not None:
            self.stream.wait_stream(other.stream)

    def use(self):
        return torch.cuda.stream(self.stream) if self.stream is not None else contextlib.nullcontext()

    def mark(self) -> Ticket:
        if self.stream is None:
            return Ticket(None)
        ev = torch.cuda.Event()
        ev.record(self.stream)
        return Ticket(ev)

    def keep_alive(self, tensor: torch.Tensor) -> None:
        """Tell the caching allocator that ``tensor`` is in use on this lane."""
        if self.stream is not None and tensor.is_cuda:
            tensor.record_stream(self.stream)


def mark_current(device: torch.device) -> Ticket:
    if device.type != "cuda":
        return Ticket(None)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(device))
    return Ticket(ev)


class DedicatedCommContext:
    def __init__(
        self,
        device: torch.device,
        replicate_group=None,
        *,
        tp_buffer_reuse: bool | str = False,
        replicate_broadcast_bucket_mb: float = 0.0,
    ):
        self.device = torch.device(device)
        self.broadcast_lane = Lane(self.device, priority=-1)
        self.sharded_adamw_unshard_lane = Lane(self.device, priority=-1)
        self.reduce_lane = Lane(self.device, priority=-1)
        self.replicate_reduce_lane = Lane(self.device, priority=0)
        self.replicate_broadcast_lane = Lane(self.device, priority=0)
        self.sharded_adamw_unshard_separate_stream_enabled = False
        self.replicate_group = replicate_group
        self.tp_buffer_reuse = self._normalize_tp_buffer_reuse(tp_buffer_reuse)
        mb = float(replicate_broadcast_bucket_mb or 0.0)
        self.replicate_broadcast_bucket_bytes = int(mb * 1024 * 1024) if mb > 0 else 0

        self.post_forward_order: list = []
        self.all_states: list = []
        self.forward_prefetch_depth = 1
        self.post_backward_final_callback_queued = False
        self.last_reduced_group = None
        self.peer_backend = None          # set by the peer-memory runtime when enabled

        self.record_forward_profile = _env_flag("DMUON_RECORD_FORWARD_PROFILE")
        self.record_post_step_profile = self.record_forward_profile or _env_flag("DMUON_RECORD_POST_STEP_PROFILE")
        self._profile_events: dict[str, list] = {"forward": [], "post_step": []}
        self._profile_counts: dict[str, dict[str, int]] = defaultdict(lambda: defaultdict(int))

    # streams under the reference's attribute names (None on CPU)
    @property
    def broadcast_stream(self):
        return self.broadcast_lane.stream

    @property
    def reduce_stream(self):
        return self.reduce_lane.stream

    @property
    def replicate_reduce_stream(self):
        return self.replicate_reduce_lane.stream

    @property
    def replicate_broadcast_stream(self):
        return self.replicate_broadcast_lane.stream

    @property
    def sharded_adamw_unshard_stream(self):
        return self.sharded_adamw_unshard_lane.stream

    @staticmethod
    def _normalize_tp_buffer_reuse(value) -> str:
        if isinstance(value, bool):
            return "all" if value else "off"
        mode = str(value).strip().lower()
        mode = {"": "off", "0": "off", "false": "off", "no": "off", "1": "all", "true": "all", "yes": "all", "on": "all"}.get(
            mode, mode
        )
        if mode not in ("off", "all", "gather", "scatter"):
            raise ValueError("tp_buffer_reuse must be one of False, True, 'off', 'gather', 'scatter', or 'all'")
        return mode

    def tp_gather_buffer_reuse_enabled(self) -> bool:
        return self.tp_buffer_reuse in ("all", "gather")

    def tp_scatter_buffer_reuse_enabled(self) -> bool:
        return self.tp_buffer_reuse in ("all", "scatter")

    def reset_post_forward_order(self) -> None:
        self.post_forward_order.clear()
        for state in self.all_states:
            state.group._post_forward_index = None

    # the reference exposes its five side streams under these names (dmuon/_core/comm.py:98-110); here they are
    # the streams of the lanes (``None`` on CPU)
    @property
    def broadcast_stream(self):
        return self.broadcast_lane.stream

    @property
    def sharded_adamw_unshard_stream(self):
        return self.sharded_adamw_unshard_lane.stream

    @property
    def reduce_stream(self):
        return self.reduce_lane.stream

    @property
    def replicate_reduce_stream(self):
        return self.replicate_reduce_lane.stream

    @property
    def replicate_broadcast_stream(self):
        return self.replicate_broadcast_lane.stream

    # ------------------------------------------------------------------ profiling
    def count(self, group_name: str, key: str, inc: int = 1) -> None:
        if self.record_forward_profile or self.record_post_step_profile:
            self._profile_counts[group_name][key] += inc

    def time_region(self, kind: str, group_name: str, phase: str, lane: Optional[Lane] = None):
        """Context manager recording a CUDA-event pair around a region."""
        enabled = self.record_forward_profile if kind == "forward" else self.record_post_step_profile
        if not enabled or self.device.type != "cuda":
            return contextlib.nullcontext()
        return _TimedRegion(self, kind, group_name, phase, lane)

    # names of the reference's context (dmuon/_core/comm.py: record_* / consume_*), for code that feeds or reads
    # the profile directly
    def record_forward_unshard_counter(self, group_name: str, **values: int) -> None:
        for key, inc in values.items():
            self._profile_counts[group_name][key] += int(inc)

    def _record_event(self, kind: str, group_name: str, phase: str, start, end, nbytes: int, **flags) -> None:
        self._profile_events[kind].append({"group": group_name, "phase": phase, "start": start, "end": end})
        if nbytes:
            self._profile_counts[group_name][f"{phase}_bytes"] += int(nbytes)
        for key, on in flags.items():
            if on:
                self._profile_counts[group_name][f"{phase}_{key}_calls"] += 1

    def record_forward_unshard_event(self, *, group_name: str, phase: str, start, end, bytes: int = 0,
                                     prefetch: bool = False) -> None:
        """Queue a finished-or-pending CUDA-event pair of the forward publish."""
        self._record_event("forward", group_name, phase, start, end, bytes, prefetch=prefetch)

    def record_post_step_event(self, *, group_name: str, phase: str, start, end, bytes: int = 0) -> None:
        self._record_event("post_step", group_name, phase, start, end, bytes)

    def consume_forward_unshard_profile(self, *, clear: bool = True) -> dict:
        return self.drain_profile("forward", clear=clear)

    def consume_post_step_profile(self, *, clear: bool = True) -> dict:
        return self.drain_profile("post_step", clear=clear)

    def drain_profile(self, kind: str = "forward", clear: bool = True) -> dict:
        """Aggregate finished timers; unfinished ones stay queued.  With
        ``clear=False`` the finished ones and the counters are kept as well."""
        events = self._profile_events[kind]
        summary: dict[str, dict[str, float]] = defaultdict(lambda: defaultdict(float))
        pending = []
        for rec in events:
            if rec["end"].query():
                ms = rec["start"].elapsed_time(rec["end"])
                slot = summary[rec["group"]]
                slot[f"{rec['phase']}_ms"] += ms
                slot[f"{rec['phase']}_calls"] += 1
            else:
                pending.append(rec)
        if clear:
            self._profile_events[kind] = pending
        out = {g: dict(v) for g, v in summary.items()}
        for g, counts in self._profile_counts.items():
            out.setdefault(g, {}).update({k: int(v) for k, v in counts.items()})
        if clear:
            self._profile_counts.clear()
        return out


class _TimedRegion:
    def __init__(self, ctx: DedicatedCommContext, kind: str, group: str, phase: str, lane: Optional[Lane]):
        self.ctx, self.kind, self.group, self.phase, self.lane = ctx, kind, group, phase, lane

    def _stream(self):
        if self.lane is not None and self.lane.stream is not None:
            return self.lane.stream
        return torch.cuda.current_stream(self.ctx.device)

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record(self._stream())
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record(self._stream())
        self.ctx._profile_events[self.kind].append(
            {"group": self.group, "phase": self.phase, "start": self.start, "end": end}
        )
        return False

"""CUDA-graph replay for stand-alone Newton-Schulz calls.

``NewtonSchulz.local`` (one matrix at a time: ``newton_schulz(G)``, tensor-
parallel owners, user code) issues about twenty small launches per matrix; for
small matrices the host, not the GPU, sets the pace.  This cache captures the
launch sequence of one ``(shape, dtype, device, configuration)`` on its second
call and replays it afterwards, like the reference's ``dmuon/optim/ns_graph.py:
61-128`` (capture on the second call, one shared memory pool, permanent eager
fallback for a key whose capture failed).

The optimizer's own path does not come through here: it orthogonalises all
owned matrices of a shape in one batch (about twenty launches for the whole
batch), so there is nothing left to amortise.  That is why replay is opt-in
(``DMUON_NS_CUDA_GRAPH=1``) instead of the reference's default-on.

The tensor returned by a replay aliases the graph's output buffer: it is
overwritten by the next call with the same key.
"""
from __future__ import annotations

import logging
import os
from typing import Callable, Hashable

import torch

log = logging.getLogger(__name__)


def enabled() -> bool:
    return os.environ.get("DMUON_NS_CUDA_GRAPH", "0").strip().lower() in ("1", "true", "yes", "on")


class _Entry:
    __slots__ = ("calls", "graph", "static_in", "static_out", "failed")

    def __init__(self):
        self.calls = 0
        self.graph = None
        self.static_in = None
        self.static_out = None
        self.failed = False


class NSGraphCache:
    def __init__(self):
        self._entries: dict[Hashable, _Entry] = {}
        self._pool = None
        self.replays = 0
        self.captures = 0

    def stats(self) -> dict:
        return {
            "keys": len(self._entries),
            "captures": self.captures,
            "replays": self.replays,
            "failed": sum(1 for e in self._entries.values() if e.failed),
        }

    def clear(self) -> None:
        self._entries.clear()
        self._pool = None

    def run(self, key: Hashable, fn: Callable[[torch.Tensor], torch.Tensor], G: torch.Tensor) -> torch.Tensor:
        """``fn(G)``, replayed from a graph from the third call with ``key`` on.
        ``fn`` must be a pure function of its argument that launches only on
        the current stream and allocates only through PyTorch."""
        e = self._entries.get(key)
        if e is None:
            e = self._entries[key] = _Entry()
        e.calls += 1
        if e.failed or not G.is_cuda or e.calls == 1:
            # the first call also creates workspaces and tile tables (host-to-device
            # copies that a capture could not contain)
            return fn(G)
        if e.graph is None:
            try:
                self._capture(e, fn, G)
            except Exception as exc:  # capture is an optimisation, never a requirement
                e.failed = True
                e.graph = e.static_in = e.static_out = None
                log.warning("Newton-Schulz graph capture failed for %s (%s); staying eager for this key", key, exc)
                return fn(G)
        e.static_in.copy_(G)
        e.graph.replay()
        self.replays += 1
        return e.static_out

    def _capture(self, e: _Entry, fn, G: torch.Tensor) -> None:
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        static_in = torch.empty_like(G, memory_format=torch.contiguous_format)
        static_in.copy_(G)
        torch.cuda.current_stream(G.device).synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=self._pool):
            static_out = fn(static_in)
        e.graph, e.static_in, e.static_out = graph, static_in, static_out
        self.captures += 1


_CACHE = NSGraphCache()


def cache() -> NSGraphCache:
    return _CACHE

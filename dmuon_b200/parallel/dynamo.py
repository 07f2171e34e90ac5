"""Keeps the hook and scheduling code out of TorchDynamo traces.

The forward/backward hooks decide at run time which transfers to start, poke
CUDA streams and mutate module parameters -- none of which a tracing compiler
can capture.  A user who wraps a model (or a block) in ``torch.compile`` after
``dedicate_params`` must get graph breaks at these entry points instead of a
trace of one particular step.  Same purpose as the reference's
``dmuon/_core/dynamo.py:15``.
"""
from __future__ import annotations

from typing import Callable, TypeVar

F = TypeVar("F", bound=Callable)

try:
    from torch._dynamo import disable as _disable
except Exception:  # pragma: no cover - builds without torch._dynamo
    _disable = None


def dynamo_disable(fn: F) -> F:
    """Return ``fn`` marked eager-only (a graph break under ``torch.compile``);
    unchanged when this torch build has no Dynamo."""
    if _disable is None:
        return fn
    return _disable(fn)  # type: ignore[return-value]

"""Old import path of the owner-assignment code.

The balanced partition lives in :mod:`dmuon_b200.parallel.partition`; this
module keeps ``from dmuon_b200.partition import compute_balanced_assignment``
working, as the reference keeps ``dmuon/partition.py`` next to
``dmuon/_core/partition.py`` (dmuon/partition.py:1-26).
"""
from .parallel.partition import (  # noqa: F401
    SMALL_PARAM_THRESHOLD,
    AssignmentResult,
    OwnerCoord,
    OwnerValue,
    compute_balanced_assignment,
    layer_key,
)

__all__ = [
    "AssignmentResult",
    "OwnerCoord",
    "OwnerValue",
    "SMALL_PARAM_THRESHOLD",
    "compute_balanced_assignment",
    "layer_key",
]

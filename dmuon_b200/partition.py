"""Old import path of the owner-assignment code.

The balanced partition lives in :mod:`dmuon_b200.parallel.partition`.  This
module forwards every public name of it on first access, so that
``from dmuon_b200.partition import compute_balanced_assignment`` (the import
path the reference keeps alive with ``dmuon/partition.py``) works and can never
drift from the real module.
"""
from importlib import import_module

_TARGET = "dmuon_b200.parallel.partition"


def _public_names() -> list:
    mod = import_module(_TARGET)
    return sorted(n for n in vars(mod) if not n.startswith("_"))


def __getattr__(name: str):
    if name.startswith("__"):
        raise AttributeError(name)
    mod = import_module(_TARGET)
    try:
        value = getattr(mod, name)
    except AttributeError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    globals()[name] = value           # cache: later accesses do not come through here
    return value


def __dir__() -> list:
    return sorted(set(globals()) | set(_public_names()))

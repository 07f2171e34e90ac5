"""Make FSDP2's ``fully_shard`` skip dedicated parameters.

``fully_shard`` collects the parameters it manages through the private helper
``_get_managed_states``.  After ``dedicate_params`` a module holds zero-size
placeholders tagged ``_dedicated_owner_rank``; the wrapper installed here drops
every tagged parameter from what the helper returns, so the user can call
``fully_shard(layer)`` as usual and FSDP2 shards only what is left.

The helper is patched at its definition and at every module of the
``_fully_shard`` package that imported it by name; both the one- and the
two-argument signature of the helper are handled (reference:
dmuon/_backends/fsdp2/patch.py:9-88).
"""
from __future__ import annotations

import importlib
import pkgutil
import sys

_ORIG_ATTR = "_dmuon_b200_original"
_patched_sites: list[tuple[object, str]] = []


def _is_dedicated(param) -> bool:
    return hasattr(param, "_dedicated_owner_rank")


def _wrap(orig):
    def filtered(modules, *args, **kwargs):
        params, buffers = orig(modules, *args, **kwargs)
        return [p for p in params if not _is_dedicated(p)], buffers

    setattr(filtered, _ORIG_ATTR, orig)
    filtered.__name__ = getattr(orig, "__name__", "_get_managed_states")
    filtered.__doc__ = getattr(orig, "__doc__", None)
    return filtered


def install_patch() -> bool:
    """Idempotent.  Returns False when this torch has no FSDP2."""
    try:
        pkg = importlib.import_module("torch.distributed.fsdp._fully_shard")
        init = importlib.import_module("torch.distributed.fsdp._fully_shard._fsdp_init")
    except Exception:
        return False
    orig = getattr(init, "_get_managed_states", None)
    if orig is None:
        return False
    if hasattr(orig, _ORIG_ATTR):
        return True
    wrapped = _wrap(orig)
    init._get_managed_states = wrapped
    _patched_sites.append((init, "_get_managed_states"))
    # modules that did ``from ._fsdp_init import _get_managed_states``
    prefix = pkg.__name__ + "."
    names = [m.name for m in pkgutil.iter_modules(pkg.__path__, prefix)]
    for name in names + [n for n in list(sys.modules) if n.startswith("torch.distributed") and "replicate" in n]:
        mod = sys.modules.get(name)
        if mod is None or mod is init:
            continue
        if getattr(mod, "_get_managed_states", None) is orig:
            mod._get_managed_states = wrapped
            _patched_sites.append((mod, "_get_managed_states"))
    return True


def uninstall_patch() -> None:
    while _patched_sites:
        mod, attr = _patched_sites.pop()
        cur = getattr(mod, attr, None)
        orig = getattr(cur, _ORIG_ATTR, None)
        if orig is not None:
            setattr(mod, attr, orig)


def is_installed() -> bool:
    try:
        init = importlib.import_module("torch.distributed.fsdp._fully_shard._fsdp_init")
    except Exception:
        return False
    return hasattr(getattr(init, "_get_managed_states", None), _ORIG_ATTR)

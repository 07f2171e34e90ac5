"""Per-parameter routing and mixed-precision policy.

A policy says which optimizer a dedicated parameter gets (``route``), in which
dtype it is published for forward/backward (``param_dtype``), reduced
(``grad_dtype``), stored (``master_dtype``) and which dtype its optimizer
state uses (``optim_dtype``), and whether activations are cast at the hook
boundary.  Same fields, aliases and precedence as the reference
(dmuon/policy.py:63-82, :17-41, :176-276): defaults, then ordered overrides
whose ``name``/``contains`` tokens occur in the parameter name, then the
callable.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Any, Callable, Iterable, Mapping, Optional

import torch
import torch.nn as nn

ROUTES = ("muon", "adamw", "sharded_adamw")

_ROUTE_ALIASES = {
    "matrix": "muon",
    "matrix_optimizer": "muon",
    "base": "adamw",
    "base_adamw": "adamw",
    "dedicated_adamw": "adamw",
    "sharded": "sharded_adamw",
    "base_sharded": "sharded_adamw",
    "sharded_collective": "sharded_adamw",
    "base_sharded_adamw": "sharded_adamw",
}

_DTYPES = {
    torch.float32: ("fp32", "float32", "torch.float32", "f32"),
    torch.bfloat16: ("bf16", "bfloat16", "torch.bfloat16"),
    torch.float16: ("fp16", "float16", "torch.float16", "half"),
}
_DTYPE_BY_NAME = {alias: dt for dt, aliases in _DTYPES.items() for alias in aliases}

_DTYPE_FIELDS = ("param_dtype", "grad_dtype", "output_dtype", "master_dtype", "optim_dtype")


@dataclass(frozen=True)
class DMuonParamPolicy:
    route: Optional[str] = None
    param_dtype: Optional[torch.dtype] = None
    grad_dtype: Optional[torch.dtype] = None
    output_dtype: Optional[torch.dtype] = None
    cast_forward_inputs: bool = False
    master_dtype: Optional[torch.dtype] = torch.float32
    optim_dtype: Optional[torch.dtype] = torch.float32
    muon_forward_unshard: Optional[str] = None
    matched_overrides: tuple[int, ...] = ()

    def group_key(self) -> tuple:
        """Parameters with equal keys may share one communication group."""
        return (
            self.route,
            self.param_dtype,
            self.grad_dtype,
            self.output_dtype,
            self.cast_forward_inputs,
            self.master_dtype,
            self.optim_dtype,
            self.muon_forward_unshard,
        )


_SETTABLE = tuple(f.name for f in fields(DMuonParamPolicy) if f.name != "matched_overrides")


def normalize_route(route) -> Optional[str]:
    if route is None:
        return None
    key = str(route).strip().lower()
    key = _ROUTE_ALIASES.get(key, key)
    if key not in ROUTES:
        raise ValueError(f"DMuon route must be one of 'muon', 'adamw', or 'sharded_adamw', got {route!r}")
    return key


def normalize_dtype(value) -> Optional[torch.dtype]:
    if value is None or isinstance(value, torch.dtype):
        return value
    if isinstance(value, str):
        key = value.strip().lower()
        if key in ("", "none", "null"):
            return None
        if key in _DTYPE_BY_NAME:
            return _DTYPE_BY_NAME[key]
    raise ValueError(f"Unsupported dtype policy value: {value!r}")


def _clean(values: Mapping[str, Any], where: str) -> dict[str, Any]:
    extra = sorted(set(values) - set(_SETTABLE))
    if extra:
        raise ValueError(f"{where}: unknown DMuon param policy field(s): {extra}")
    out: dict[str, Any] = {}
    for k, v in values.items():
        if k == "route":
            out[k] = normalize_route(v)
        elif k in _DTYPE_FIELDS:
            out[k] = normalize_dtype(v)
        elif k == "cast_forward_inputs":
            out[k] = bool(v)
        elif k == "muon_forward_unshard":
            out[k] = None if v is None else str(v).strip().lower()
    return out


def coerce_policy(policy, where: str = "policy") -> DMuonParamPolicy:
    if policy is None:
        return DMuonParamPolicy()
    if isinstance(policy, DMuonParamPolicy):
        vals = _clean({k: getattr(policy, k) for k in _SETTABLE}, where)
        return replace(DMuonParamPolicy(), **vals, matched_overrides=policy.matched_overrides)
    if isinstance(policy, Mapping):
        return DMuonParamPolicy(**_clean(policy, where))
    raise TypeError(f"{where}: expected mapping or DMuonParamPolicy, got {type(policy)!r}")


def _selector_tokens(override: Mapping[str, Any]) -> tuple[str, ...]:
    if "name" in override and "contains" in override:
        raise ValueError("param_policy override accepts either 'name' or 'contains', not both")
    sel = override.get("name", override.get("contains"))
    if sel is None:
        return ()
    if isinstance(sel, str):
        return (sel,)
    if isinstance(sel, Iterable):
        return tuple(str(s) for s in sel)
    raise TypeError(f"name must be a string or iterable of strings, got {type(sel)!r}")


def _parse_overrides(param_policy: Mapping[str, Any]) -> list[Mapping[str, Any]]:
    raw = param_policy.get("overrides", ()) or ()
    if isinstance(raw, (str, bytes)) or not isinstance(raw, Iterable):
        raise TypeError("param_policy['overrides'] must be a sequence of mappings")
    out = []
    for i, ov in enumerate(raw):
        if not isinstance(ov, Mapping):
            raise TypeError(f"param_policy.overrides[{i}] must be a mapping")
        extra = sorted(set(ov) - {"name", "contains", "set"})
        if extra:
            raise ValueError(f"param_policy.overrides[{i}] has unknown selector field(s): {extra}")
        if "set" not in ov:
            raise ValueError(f"param_policy.overrides[{i}] is missing required 'set'")
        if not isinstance(ov["set"], Mapping):
            raise TypeError(f"param_policy.overrides[{i}]['set'] must be a mapping")
        out.append(ov)
    return out


def resolve_param_policies(
    *,
    params: Iterable[nn.Parameter],
    param_to_fqn: Mapping[nn.Parameter, str],
    compute_dtype: Optional[torch.dtype] = None,
    route_hint_fn: Optional[Callable[[str, nn.Parameter], Optional[str]]] = None,
    param_policy: Optional[Mapping[str, Any]] = None,
    param_policy_fn: Optional[Callable[[str, nn.Parameter], Any]] = None,
    default_muon_forward_unshard: Optional[str] = None,
) -> dict[nn.Parameter, DMuonParamPolicy]:
    if param_policy is not None and param_policy_fn is not None:
        raise ValueError("Pass at most one of param_policy and param_policy_fn")
    structured = param_policy is not None or param_policy_fn is not None
    if structured and route_hint_fn is not None:
        raise ValueError(
            "route_hint_fn is legacy route-only API and cannot be combined with param_policy or param_policy_fn"
        )
    base = DMuonParamPolicy(
        param_dtype=normalize_dtype(compute_dtype), muon_forward_unshard=default_muon_forward_unshard
    )
    overrides: list[Mapping[str, Any]] = []
    if param_policy is not None:
        defaults = param_policy.get("defaults", {})
        if not isinstance(defaults, Mapping):
            raise TypeError("param_policy['defaults'] must be a mapping")
        base = replace(base, **_clean(defaults, "param_policy.defaults"))
        overrides = _parse_overrides(param_policy)

    out: dict[nn.Parameter, DMuonParamPolicy] = {}
    for p in params:
        fqn = param_to_fqn[p]
        pol = base
        if route_hint_fn is not None:
            pol = replace(pol, route=normalize_route(route_hint_fn(fqn, p)))
        elif not structured:
            hint = getattr(p, "_dmuon_route_hint", None)
            if hint is not None:
                pol = replace(pol, route=normalize_route(hint))
        hit: list[int] = []
        for i, ov in enumerate(overrides):
            toks = _selector_tokens(ov)
            if toks and not any(t in fqn for t in toks):
                continue
            pol = replace(pol, **_clean(ov["set"], f"param_policy.overrides[{i}].set"))
            hit.append(i)
        if param_policy_fn is not None:
            res = param_policy_fn(fqn, p)
            if isinstance(res, DMuonParamPolicy):
                pol = coerce_policy(res, f"param_policy_fn({fqn!r})")
            elif res is not None:
                pol = replace(pol, **_clean(res, f"param_policy_fn({fqn!r})"))
        out[p] = replace(pol, matched_overrides=tuple(hit))
    return out

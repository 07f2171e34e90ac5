"""One dedicated parameter: who owns it, where its master copy lives, and how
the module attribute is swapped between a zero-size placeholder and the
full-size published view.

Two placements share this class:

* ``mode="fsdp"`` -- non-owners hold nothing between uses; the owner's shard
  column (every replicate row's rank with the owner's shard index) holds the
  master copy, everyone receives a published low-precision copy for forward
  and backward (reference: dmuon/_backends/fsdp2/param.py:116-628);
* ``mode="ddp"`` -- the live parameter stays resident on every rank, gradients
  are reduced to the owner and the owner's update is broadcast after the step
  (reference: dmuon/_backends/ddp/param.py:80-342).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..policy import DMuonParamPolicy, normalize_route
from .topology import normalize_owner_rank

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None


def alloc_storage(t: torch.Tensor) -> None:
    """Give ``t`` back the storage its size/stride metadata describes."""
    need = t.numel() * t.element_size()
    st = t.untyped_storage()
    if st.size() != need:
        st.resize_(need)


def free_storage(t: torch.Tensor) -> None:
    """Drop the storage of ``t`` but keep the tensor object and its views."""
    st = t.untyped_storage()
    if st.size() != 0:
        st.resize_(0)


def unsafe_setattr_param(module: nn.Module, name: str, param: nn.Parameter) -> None:
    """Swap ``module.<name>`` without nn.Module's registration checks."""
    if getattr(module.__setattr__, "__func__", None) is nn.Module.__setattr__:
        module._parameters[name] = param
    else:  # a subclass overrides __setattr__: go through it
        setattr(module, name, param)


def _group_rank(group) -> int:
    return group.rank() if group is not None else 0


def _group_size(group) -> int:
    return group.size() if group is not None else 1


class DedicatedParam:
    def __init__(
        self,
        param: nn.Parameter,
        module: nn.Module,
        param_name: str,
        owner_rank,
        dp_group,
        device: torch.device,
        *,
        policy: Optional[DMuonParamPolicy] = None,
        compute_dtype: Optional[torch.dtype] = None,
        replicate_group=None,
        tp_group=None,
        tp_owner_local_rank: int = 0,
        tp_shard_dim: Optional[int] = None,
        fqn: Optional[str] = None,
        mode: str = "fsdp",
        alias_sites: Optional[list[tuple[nn.Module, str]]] = None,
    ):
        policy = policy or DMuonParamPolicy(param_dtype=compute_dtype)
        self.param_name = param_name
        self.fqn = fqn or param_name
        self.module = module
        self.mode = mode
        self.device = torch.device(device)
        self.policy = policy
        self.alias_sites: list[tuple[nn.Module, str]] = list(alias_sites or [(module, param_name)])

        coord = normalize_owner_rank(owner_rank)
        self.owner_rank = coord
        self.owner_shard, self.owner_replicate = coord
        self.dp_group = dp_group
        self.replicate_group = replicate_group
        self.shard_rank = _group_rank(dp_group)
        self.shard_size = _group_size(dp_group)
        self.replicate_rank = _group_rank(replicate_group)
        self.replicate_size = _group_size(replicate_group)
        if self.owner_shard >= self.shard_size or self.owner_replicate >= self.replicate_size:
            raise ValueError(f"{self.fqn}: owner {coord} outside the {self.shard_size}x{self.replicate_size} grid")
        self.in_owner_column = self.shard_rank == self.owner_shard
        self.is_owner = self.in_owner_column and self.replicate_rank == self.owner_replicate

        # Tensor parallelism: the stored tensor is this rank's shard.
        self.is_dtensor = DTensor is not None and isinstance(param, DTensor)
        if self.is_dtensor:
            self._tp_spec = param._spec
            local = param._local_tensor
            self.full_shape = torch.Size(param.shape)
        else:
            self._tp_spec = None
            local = param.data
            self.full_shape = torch.Size(local.shape)
        self.tp_group = tp_group
        self.shard_dim = tp_shard_dim if tp_group is not None else None
        if tp_group is not None:
            if not 0 <= tp_owner_local_rank < tp_group.size():
                raise ValueError(f"{self.fqn}: tp owner {tp_owner_local_rank} outside TP group of {tp_group.size()}")
            self._tp_owner_local_rank = int(tp_owner_local_rank)
            self._tp_owner_global_rank = dist.get_global_rank(tp_group, self._tp_owner_local_rank)
            self.is_tp_owner = tp_group.rank() == self._tp_owner_local_rank
        else:
            self._tp_owner_local_rank = 0
            self._tp_owner_global_rank = None
            self.is_tp_owner = False

        self._orig_size = torch.Size(local.shape)
        self._orig_dtype = local.dtype
        self.numel = int(local.numel())
        self._requires_grad = bool(param.requires_grad)
        self._param_dtype = policy.param_dtype or self._orig_dtype
        self._grad_dtype = policy.grad_dtype
        self._output_dtype = policy.output_dtype
        self._cast_forward_inputs = bool(policy.cast_forward_inputs)
        self._master_dtype = policy.master_dtype or self._orig_dtype
        self._optim_dtype = policy.optim_dtype or torch.float32
        self._compute_dtype = self._param_dtype
        self._dmuon_route = normalize_route(policy.route) or self._default_route()
        self._muon_forward_unshard = (policy.muon_forward_unshard or "broadcast").lower()

        # Optimizer-facing state.
        self._reduced_grad: Optional[torch.Tensor] = None
        self._accumulated_grad: Optional[torch.Tensor] = None
        self._tp_full_grad: Optional[torch.Tensor] = None
        self._tp_full_delta: Optional[torch.Tensor] = None
        self._tp_wd_factor: float = 1.0
        self._sharded_adamw_grad: Optional[torch.Tensor] = None
        self._sharded_adamw_data: Optional[torch.Tensor] = None
        self._sharded_muon_data: Optional[torch.Tensor] = None   # forward shard of the "all_gather" Muon placement
        self._publish_fresh = False      # published copy already equals the master copy

        self._original_param = param
        self._unsharded_param: Optional[nn.Parameter] = None
        self._is_unsharded = False
        self._owned_data: Optional[torch.Tensor] = None

        if mode == "ddp":
            self._init_ddp(param, local)
        else:
            self._init_fsdp(param, local)

    # ---------------------------------------------------------------- construction
    def _default_route(self) -> str:
        return "muon" if len(self.full_shape) >= 2 else "adamw"

    def _init_fsdp(self, param: nn.Parameter, local: torch.Tensor) -> None:
        if self._dmuon_route == "sharded_adamw":
            self._init_flat_shard(local)
        elif self.in_owner_column:
            self._owned_data = local.detach().to(device=self.device, dtype=self._master_dtype).clone()
        if self.uses_sharded_muon_forward():
            self._sharded_muon_data = self._flat_shard_of(local, self._param_dtype)
        self._placeholder = nn.Parameter(
            torch.empty(0, dtype=self._orig_dtype, device=self.device), requires_grad=self._requires_grad
        )
        self._placeholder._dedicated_owner_rank = self.owner_rank
        self._placeholder._dedicated_mode = "fsdp"
        self.detach_from_modules()
        # The original full-size storage is no longer referenced by the module;
        # release it eagerly (the Parameter object may still be held by users).
        if not self.is_dtensor and local.device == self.device:
            free_storage(local)

    def uses_sharded_muon_forward(self) -> bool:
        """Muon route whose forward copy is rebuilt by all-gather from per-rank
        shards instead of a broadcast from the owner (the reference's
        experimental ``muon_forward_unshard="all_gather"``,
        dmuon/_backends/fsdp2/param.py:316-325)."""
        return (
            self.mode == "fsdp" and self._dmuon_route == "muon" and self._muon_forward_unshard == "all_gather"
            and self.tp_group is None and self.shard_size > 1
        )

    def _flat_shard_of(self, local: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """This rank's zero-padded slice of the flattened tensor."""
        n = self.shard_size
        per = (self.numel + n - 1) // n
        self._flat_shard_numel = per
        flat = local.detach().reshape(-1)
        lo = min(self.numel, self.shard_rank * per)
        hi = min(self.numel, lo + per)
        shard = torch.zeros(per, dtype=dtype, device=self.device)
        shard[: hi - lo].copy_(flat[lo:hi])
        return shard

    def _init_flat_shard(self, local: torch.Tensor) -> None:
        self._sharded_adamw_data = self._flat_shard_of(local, self._master_dtype)

    def forward_shard(self) -> torch.Tensor:
        """What this rank contributes to the forward all-gather."""
        return self._sharded_adamw_data if self._dmuon_route == "sharded_adamw" else self._sharded_muon_data

    def _init_ddp(self, param: nn.Parameter, local: torch.Tensor) -> None:
        self._owned_data = local.detach().to(device=self.device, dtype=self._master_dtype).clone()
        if local.dtype != self._param_dtype or local.device != self.device:
            param.data = local.to(device=self.device, dtype=self._param_dtype)
        self._unsharded_param = param
        self._placeholder = None
        self._is_unsharded = True
        param._dedicated_owner_rank = self.owner_rank
        param._dedicated_mode = "ddp"

    # ---------------------------------------------------------------- module attribute swap
    def make_unsharded_param(self, view: torch.Tensor) -> nn.Parameter:
        """Wrap a full-size view of the published buffer as the live Parameter."""
        if self.is_dtensor:
            data = DTensor.from_local(
                view, device_mesh=self._tp_spec.mesh, placements=self._tp_spec.placements, run_check=False,
                shape=self._tp_spec.shape, stride=self._tp_spec.stride,
            )
        else:
            data = view
        p = nn.Parameter(data, requires_grad=self._requires_grad)
        p._dedicated_owner_rank = self.owner_rank
        p._dedicated_mode = "fsdp"
        self._unsharded_param = p
        return p

    def attach_to_modules(self) -> None:
        for mod, name in self.alias_sites:
            unsafe_setattr_param(mod, name, self._unsharded_param)

    def detach_from_modules(self) -> None:
        for mod, name in self.alias_sites:
            unsafe_setattr_param(mod, name, self._placeholder)

    # ---------------------------------------------------------------- gradients
    def local_grad(self) -> Optional[torch.Tensor]:
        """The gradient autograd left on the live parameter, as a local tensor
        of this rank's stored shape."""
        p = self._unsharded_param
        if p is None or p.grad is None:
            return None
        g = p.grad
        if DTensor is not None and isinstance(g, DTensor):
            g = g._local_tensor
        if g.shape != self._orig_size:
            if self.tp_group is not None and self.shard_dim is not None and g.shape == self.full_shape:
                ext = self._orig_size[self.shard_dim]
                g = g.narrow(self.shard_dim, self.tp_group.rank() * ext, ext)
            elif g.numel() == self.numel:
                g = g.reshape(self._orig_size)
            else:
                raise RuntimeError(f"{self.fqn}: gradient shape {tuple(g.shape)} does not match {tuple(self._orig_size)}")
        return g

    def uses_sharded_adamw(self) -> bool:
        return self._dmuon_route == "sharded_adamw"

    def clear_reduced_grad(self) -> None:
        self._reduced_grad = None
        self._sharded_adamw_grad = None

    def clear_local_grad(self) -> None:
        if self._unsharded_param is not None:
            self._unsharded_param.grad = None

    def copy_owned_to_live(self) -> None:
        """DDP placement: refresh the resident live parameter from the master."""
        if self.mode == "ddp" and self._owned_data is not None:
            live = self._unsharded_param.data
            if DTensor is not None and isinstance(live, DTensor):
                live = live._local_tensor
            live.copy_(self._owned_data)

    # ---------------------------------------------------------------- misc
    @property
    def matrix_shape(self) -> tuple[int, int]:
        """``(rows, cols)`` the matrix optimizer sees: first dim x the rest."""
        shape = self.full_shape if self.tp_group is not None else self._orig_size
        rows = int(shape[0])
        return rows, int(self.full_shape.numel() // rows) if self.tp_group is not None else int(self.numel // rows)

    def __repr__(self) -> str:
        return (
            f"DedicatedParam({self.fqn}, shape={tuple(self._orig_size)}, owner={self.owner_rank}, "
            f"route={self._dmuon_route}, mode={self.mode})"
        )


class DedicatedParamDDP(DedicatedParam):
    """DDP placement under the reference's class name."""

    def __init__(self, *args, **kwargs):
        kwargs["mode"] = "ddp"
        super().__init__(*args, **kwargs)

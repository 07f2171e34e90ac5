"""Hook state machine of one (module, group) pair.

forward pre    consume last step's publish, publish this group's parameters,
               start the next groups' publish, tie a post-backward node to the
               module inputs
forward post   drop the published copy when it is not kept for backward,
               remember forward order, arm the pre-backward trigger on outputs
pre-backward   publish again if needed, prefetch the next group backward reaches
post-backward  pack and reduce gradients, drop the published copy
root callback  end of the backward pass: run post-backward for groups whose
               inputs carried no gradient, reset per-backward flags

The four phases and their order are the reference's
(dmuon/_core/state.py:158-280, :350-385).  The post-backward trigger is an
identity autograd node on the module inputs: it was created before every node
of the module, so the engine runs it after all of them, parameter gradient
accumulation included.
"""
from __future__ import annotations


import torch
import torch.nn as nn
from torch.autograd import Variable

from .comm import DedicatedCommContext
from .dynamo import dynamo_disable


def in_backward_pass() -> bool:
    return torch._C._current_graph_task_id() != -1


def defer_sharded_adamw_reduce_to_root() -> bool:
    """``DMUON_DEFER_SHARDED_ADAMW_REDUCE_TO_ROOT`` (default on): a group that
    holds ``sharded_adamw`` parameters reduces only from the end-of-backward
    callback.  Its reduce-scatter consumes and clears the full local gradient,
    so it must not start while another autograd edge (a second use of the
    module, a tied weight) can still add to it (reference
    ``dmuon/_core/state.py:45-47,245-252``)."""
    import os

    return os.environ.get("DMUON_DEFER_SHARDED_ADAMW_REDUCE_TO_ROOT", "1") not in ("", "0", "false", "False", "FALSE")


def _map_tensors(fn, obj):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, tuple):
        mapped = [_map_tensors(fn, o) for o in obj]
        return type(obj)(*mapped) if hasattr(obj, "_fields") else tuple(mapped)
    if isinstance(obj, list):
        return [_map_tensors(fn, o) for o in obj]
    if isinstance(obj, dict):
        return {k: _map_tensors(fn, v) for k, v in obj.items()}
    return obj


def _cast_floating(dtype: torch.dtype):
    def cast(t: torch.Tensor) -> torch.Tensor:
        return t.to(dtype) if torch.is_floating_point(t) and t.dtype != dtype else t

    return cast


class _PostBackwardNode(torch.autograd.Function):
    @staticmethod
    def forward(ctx, state, *tensors):
        ctx.state = state
        return tensors

    @staticmethod
    def backward(ctx, *grads):
        ctx.state._post_backward()
        return (None,) + grads


class _PreBackwardNode(torch.autograd.Function):
    @staticmethod
    def forward(ctx, state, *tensors):
        ctx.state = state
        return tensors

    @staticmethod
    def backward(ctx, *grads):
        ctx.state._pre_backward()
        return (None,) + grads


def _wrap_first_grad_tensor(node_cls, state, obj):
    """Route the first grad-requiring top-level tensor of ``obj`` through
    ``node_cls``.  Containers keep their type; dicts (incl. ModelOutput) are
    updated in place so attribute access on them keeps working."""
    if isinstance(obj, torch.Tensor):
        if obj.requires_grad:
            return node_cls.apply(state, obj)[0], True
        return obj, False
    if isinstance(obj, (tuple, list)):
        items = list(obj)
        for i, it in enumerate(items):
            if isinstance(it, torch.Tensor) and it.requires_grad:
                items[i] = node_cls.apply(state, it)[0]
                if isinstance(obj, list):
                    return items, True
                return (type(obj)(*items) if hasattr(obj, "_fields") else tuple(items)), True
        return obj, False
    if isinstance(obj, dict):
        for k, it in obj.items():
            if isinstance(it, torch.Tensor) and it.requires_grad:
                obj[k] = node_cls.apply(state, it)[0]
                return obj, True
        return obj, False
    return obj, False


def _wrap_every_grad_tensor(node_cls, state, obj):
    """Route every grad-requiring top-level tensor of a module output through
    its own ``node_cls`` node: whichever of them the loss is built from (the
    logits, or a loss the module computed itself), backward passes the node
    before it reaches the module's parameters."""
    def wrap(it):
        if isinstance(it, torch.Tensor) and it.requires_grad:
            return node_cls.apply(state, it)[0]
        return it

    if isinstance(obj, torch.Tensor):
        return wrap(obj)
    if isinstance(obj, list):
        return [wrap(it) for it in obj]
    if isinstance(obj, tuple):
        items = [wrap(it) for it in obj]
        return type(obj)(*items) if hasattr(obj, "_fields") else tuple(items)
    if isinstance(obj, dict):
        for k in list(obj.keys()):
            obj[k] = wrap(obj[k])           # in place: attribute access on ModelOutput-like dicts keeps working
        return obj
    return obj


class DedicatedState:
    def __init__(self, module: nn.Module, group, comm_ctx: DedicatedCommContext):
        self.module = module
        self.group = group
        self.comm_ctx = comm_ctx
        self._forward_ran = False
        self._post_backward_ran = False
        self.next_states: list["DedicatedState"] = []     # forward-order successors
        comm_ctx.all_states.append(self)
        states = getattr(module, "_dedicated_states", None)
        if states is None:
            states = []
            module._dedicated_states = states
        states.append(self)
        module._dedicated_state = states[0]
        self._pre_handle = module.register_forward_pre_hook(self._pre_forward, with_kwargs=True)
        self._post_handle = module.register_forward_hook(self._post_forward)

    # ------------------------------------------------------------------ forward
    def _is_first_state(self) -> bool:
        return bool(self.comm_ctx.all_states) and self.comm_ctx.all_states[0] is self

    @dynamo_disable
    def _pre_forward(self, module, args, kwargs):
        ctx, group = self.comm_ctx, self.group
        recompute = in_backward_pass()
        if not recompute and self._is_first_state():
            ctx.reset_post_forward_order()
        group._pre_forward_wait()
        group.unshard()
        group.wait_for_unshard()
        pol = group.params[0] if group.params else None
        if pol is not None and pol._cast_forward_inputs and pol._param_dtype is not None:
            cast = _cast_floating(pol._param_dtype)
            args = _map_tensors(cast, args)
            kwargs = _map_tensors(cast, kwargs)
        if not recompute:
            nxt = self.next_states[: max(0, int(ctx.forward_prefetch_depth))]
            for st in nxt:
                st.group._pre_forward_wait()
                st.group.unshard(prefetch=True)
        if torch.is_grad_enabled():
            args, hit = _wrap_first_grad_tensor(_PostBackwardNode, self, args)
            if not hit:
                kwargs, hit = _wrap_first_grad_tensor(_PostBackwardNode, self, kwargs)
        self._forward_ran = True
        self._post_backward_ran = False
        group._backward_done = False
        return args, kwargs

    @dynamo_disable
    def _post_forward(self, module, args, output):
        group = self.group
        recompute = in_backward_pass()
        if group.reshard_after_forward and not recompute:
            group.reshard()
        if not recompute:
            group._record_post_forward()
        if torch.is_grad_enabled() and not recompute:
            output = _wrap_every_grad_tensor(_PreBackwardNode, self, output)
        pol = group.params[0] if group.params else None
        if pol is not None and pol._output_dtype is not None:
            output = _map_tensors(_cast_floating(pol._output_dtype), output)
        return output

    # ------------------------------------------------------------------ backward
    @dynamo_disable
    def _pre_backward(self) -> None:
        self._queue_root_callback()
        group = self.group
        group.unshard()
        group.wait_for_unshard()
        group._backward_prefetch()

    @dynamo_disable
    def _post_backward(self) -> None:
        if self._post_backward_ran:
            return
        self._queue_root_callback()
        ctx, group = self.comm_ctx, self.group
        if (
            not getattr(ctx, "_in_root_post_backward", False)
            and any(p._dmuon_route == "sharded_adamw" for p in group.params)
            and defer_sharded_adamw_reduce_to_root()
        ):
            return      # the root callback runs this group once the whole graph has executed
        prev = ctx.last_reduced_group
        if prev is not None and prev is not group:
            # one reduce outstanding at a time: bounds the packed-gradient memory
            prev.wait_for_stage1_reduce()
        group.reduce_grads()
        group.reshard()
        group._backward_done = True
        self._post_backward_ran = True

    def _queue_root_callback(self) -> None:
        ctx = self.comm_ctx
        if ctx.post_backward_final_callback_queued:
            return
        ctx.post_backward_final_callback_queued = True
        Variable._execution_engine.queue_callback(lambda: _root_post_backward(ctx))

    def remove(self) -> None:
        self._pre_handle.remove()
        self._post_handle.remove()


@dynamo_disable
def _root_post_backward(ctx: DedicatedCommContext) -> None:
    """Runs once when the whole backward graph has been executed."""
    ctx._in_root_post_backward = True
    try:
        for st in ctx.all_states:
            if st._forward_ran and not st._post_backward_ran:
                has_grad = any(
                    p.local_grad() is not None or getattr(p, "_grad_in_arena", False) for p in st.group.params
                )
                if has_grad or st.group._is_unsharded:
                    st._post_backward_ran = False
                    st._post_backward()
            st._forward_ran = False
            st._post_backward_ran = False
    finally:
        ctx._in_root_post_backward = False
        ctx.post_backward_final_callback_queued = False
        ctx.last_reduced_group = None

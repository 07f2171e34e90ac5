"""Behavioural details a drop-in replacement has to keep (2 gloo ranks): tied
dedicated weights, dict-like model outputs, parameters that receive no
gradient, the constructor guard, ``zero_grad`` bookkeeping, activation casts."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from dist_utils import run_ranks


class Out(dict):
    """Minimal stand-in for a Hugging Face ``ModelOutput``: a dict with attribute access."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as exc:
            raise AttributeError(k) from exc


class Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.in_proj = nn.Linear(d, d, bias=False)
        self.out_proj = nn.Linear(d, d, bias=False)
        self.unused_proj = nn.Linear(d, d, bias=False)       # never called: no gradient, ever

    def forward(self, x):
        return x + self.out_proj(torch.tanh(self.in_proj(x)))


class TiedNet(nn.Module):
    def __init__(self, d=16, vocab=32):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList(Block(d) for _ in range(2))
        self.blocks[1].in_proj.weight = self.blocks[0].in_proj.weight      # one matrix, two call sites
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids, labels=None):
        x = self.embed(ids)
        for b in self.blocks:
            x = b(x)
        logits = self.head(self.norm(x))
        out = Out(logits=logits)
        if labels is not None:
            out["loss"] = F.cross_entropy(logits.flatten(0, 1), labels.flatten())
        return out


def _pred(n, p):
    return "proj" in n and p.ndim == 2


def _single_process_reference(steps, ids):
    import math

    from dmuon_b200.optim.newton_schulz import gram_newton_schulz

    torch.manual_seed(0)
    model = TiedNet()
    params = dict(model.named_parameters())             # tied weight appears once
    mom = {}
    losses = []
    for _ in range(steps):
        model.zero_grad()
        loss = model(ids, labels=ids).loss
        loss.backward()
        losses.append(loss.item())
        with torch.no_grad():
            for n, p in params.items():
                if not _pred(n, p) or p.grad is None:
                    continue
                buf = mom.setdefault(n, torch.zeros_like(p))
                buf.mul_(0.95).add_(p.grad)
                o = gram_newton_schulz(p.grad.add(buf, alpha=0.95))
                p.add_(o, alpha=-0.05 * 0.2 * math.sqrt(max(p.shape)))
    return losses, {n: p.detach().clone() for n, p in params.items() if _pred(n, p)}


def _body(rank, world, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = TiedNet()
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    # the guard: non-dedicated trainable parameters must be managed by FSDP2 or replicate
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=True)
    try:
        dmuon.Muon(model, first_step_progress_log=False)
        guard = False
    except RuntimeError:
        guard = True
    fully_shard(model, mesh=mesh)
    # adamw_lr 0: only the Muon matrices move, which is what the reference below reproduces
    opt = dmuon.Muon(model, lr=0.05, adamw_lr=0.0, adamw_weight_decay=0.0, first_step_progress_log=False)
    dps = {p.fqn: p for p in dmuon.get_dedicated_params(model)}
    tied = dps["blocks.0.in_proj.weight"]
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(7))
    losses, attr_ok = [], True
    for _ in range(steps):
        opt.zero_grad()
        out = model(ids, labels=ids)                       # same batch on both ranks: the mean equals one rank's gradient
        attr_ok = attr_ok and isinstance(out, Out) and out.loss is out["loss"]
        out.loss.backward()
        opt.step()
        losses.append(out.loss.item())
    # a parameter that never got a gradient: no momentum, untouched weights, no crash
    unused = dps["blocks.0.unused_proj.weight"]
    unused_state = "momentum_buffer" in opt.state.get(id(unused), {})
    opt.zero_grad()
    cleared = all(p._reduced_grad is None and p._accumulated_grad is None for p in dps.values())
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return (guard, sorted(tied.alias_fqns), losses, attr_ok, unused_state, cleared,
            {k: v for k, v in sd.items() if "proj" in k}, sorted(sd))


def test_tied_weights_dict_outputs_unused_parameters_and_guard():
    steps = 4
    ids = torch.randint(0, 32, (4, 8), generator=torch.Generator().manual_seed(7))
    ref_losses, ref_params = _single_process_reference(steps, ids)
    for guard, aliases, losses, attr_ok, unused_state, cleared, sd, names in run_ranks(_body, 2, args=(steps,)):
        assert guard and attr_ok and cleared and not unused_state
        assert aliases == ["blocks.0.in_proj.weight", "blocks.1.in_proj.weight"]
        assert "blocks.1.in_proj.weight" in names              # state dict lists every alias, like nn.Module.state_dict
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (losses, ref_losses)
        for n, p in ref_params.items():
            assert (sd[n] - p).abs().max().item() < 2e-4, n
        assert torch.equal(sd["blocks.0.in_proj.weight"], sd["blocks.1.in_proj.weight"])


def _cast_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8, bias=False), nn.Linear(8, 8, bias=False))
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(
        model, mesh, lambda n, p: p.ndim == 2, hook_boundary_predicate=lambda m: isinstance(m, nn.Linear),
        reshard_after_forward=False,
        param_policy={"defaults": {"param_dtype": "bf16", "output_dtype": "fp32", "cast_forward_inputs": True}},
    )
    fully_shard(model, mesh=mesh)
    seen = []
    model[1].register_forward_pre_hook(lambda m, a: seen.append(a[0].dtype))
    y = model(torch.randn(2, 8))
    live = model[0].weight.dtype
    masters = {p._owned_data.dtype for p in dmuon.get_owned_params(model)}
    return str(y.dtype), [str(d) for d in seen], str(live), sorted(str(m) for m in masters)


def test_activation_casts_at_the_hook_boundary():
    for y_dtype, seen, live, masters in run_ranks(_cast_body, 2):
        assert y_dtype == "torch.float32"                  # output_dtype
        assert live == "torch.bfloat16"                    # param_dtype of the live weights
        assert masters in (["torch.float32"], [])          # fp32 masters on the owner
        assert seen and seen[0] in ("torch.float32", "torch.bfloat16")


class ConvAsLinear(nn.Module):
    """A kernel-size-1 Conv1d whose weight the forward squeezes and uses as a matrix."""

    def __init__(self, d=16):
        super().__init__()
        self.mix_proj = nn.Conv1d(d, d, 1, bias=False)
        self.out_proj = nn.Linear(d, d, bias=False)

    def forward(self, x):
        w = self.mix_proj.weight.squeeze(-1)               # direct attribute access, then a view
        return self.out_proj(torch.tanh(F.linear(x, w)))


def _conv_body(rank, world, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = nn.Sequential(ConvAsLinear(), ConvAsLinear())
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n, reshard_after_forward=True,
                          hook_boundary_predicate=lambda m: isinstance(m, ConvAsLinear))
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.05, first_step_progress_log=False)
    x = torch.randn(4, 16, generator=torch.Generator().manual_seed(11))
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(x).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    shapes = {p.fqn: (tuple(p.full_shape), p._dmuon_route) for p in dmuon.get_dedicated_params(model)}
    mom = {p.fqn: tuple(opt.state[id(p)]["momentum_buffer"].shape) for p in dmuon.get_owned_params(model)}
    return losses, shapes, mom, dmuon.get_model_state_dict(model, rank0_only=False)


def test_three_dimensional_weights_are_orthogonalised_as_matrices():
    import math

    from dmuon_b200.optim.newton_schulz import gram_newton_schulz

    steps = 3
    torch.manual_seed(0)
    ref = nn.Sequential(ConvAsLinear(), ConvAsLinear())
    x = torch.randn(4, 16, generator=torch.Generator().manual_seed(11))
    moms = {n: torch.zeros_like(p) for n, p in ref.named_parameters()}
    ref_losses = []
    for _ in range(steps):
        ref.zero_grad()
        loss = ref(x).pow(2).mean()
        loss.backward()
        ref_losses.append(loss.item())
        with torch.no_grad():
            for n, p in ref.named_parameters():
                g2 = p.grad.reshape(p.shape[0], -1)
                buf = moms[n].view_as(g2)
                buf.mul_(0.95).add_(g2)
                o = gram_newton_schulz(g2.add(buf, alpha=0.95))
                p.add_(o.view_as(p), alpha=-0.05 * 0.2 * math.sqrt(max(g2.shape)))
    res = run_ranks(_conv_body, 2, args=(steps,))
    losses, shapes, _, sd = res[0]
    assert shapes["0.mix_proj.weight"] == ((16, 16, 1), "muon")          # a 3-D weight takes the Muon route
    owned = {}
    for r in res:
        owned.update(r[2])
    assert owned["0.mix_proj.weight"] == (16, 16) and len(owned) == 4      # momentum is kept as a (rows, rest) matrix
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (losses, ref_losses)
    for n, p in ref.named_parameters():
        assert sd[n].shape == p.shape and (sd[n] - p).abs().max().item() < 2e-4, n


class _WithBuffer(nn.Module):
    def __init__(self):
        super().__init__()
        self.a_proj = nn.Linear(16, 32, bias=False)
        self.b_proj = nn.Linear(32, 16, bias=False)
        self.norm = nn.LayerNorm(16)
        self.register_buffer("running", torch.zeros(16))

    def forward(self, x):
        return self.norm(self.b_proj(torch.relu(self.a_proj(x))) + self.running)


def _bcast_load_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    torch.manual_seed(0)
    model = _WithBuffer()
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2)
    fully_shard(model, mesh=mesh)
    # only rank 0 holds data; one parameter is absent from the file
    sd = {}
    if rank == 0:
        g = torch.Generator().manual_seed(9)
        sd = {"a_proj.weight": torch.randn(32, 16, generator=g), "norm.weight": torch.full((16,), 3.0),
              "norm.bias": torch.full((16,), -1.0), "running": torch.arange(16.0)}
    dmuon.set_model_state_dict(model, sd, strict=False, broadcast_from_rank0=True)
    out = dmuon.get_model_state_dict(model, rank0_only=False)
    return {k: v.clone() for k, v in out.items()}, model.running.clone()


def test_broadcast_load_carries_buffers_and_skips_missing_keys_on_every_rank():
    """``broadcast_from_rank0``: buffers travel like parameters, and a key that
    rank 0 does not have is skipped by ALL ranks (nobody waits in a broadcast
    that rank 0 never enters)."""
    res = run_ranks(_bcast_load_body, 2, timeout=120)
    g = torch.Generator().manual_seed(9)
    want_a = torch.randn(32, 16, generator=g)
    for sd, running in res:
        assert torch.equal(sd["a_proj.weight"], want_a)
        assert torch.equal(sd["norm.weight"], torch.full((16,), 3.0))
        assert torch.equal(running, torch.arange(16.0))
    # the absent matrix kept its initial value, identically on both ranks
    assert torch.equal(res[0][0]["b_proj.weight"], res[1][0]["b_proj.weight"])


def _scaled_step_body(rank, world, how):
    """One step with every gradient multiplied by 0.25: through the loss ("loss"),
    through ``scale_grads_on_next_step`` ("defer", twice 0.5), or not at all ("none")."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import HP, _build_model, _data, _pred

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=HP["lr"], adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"], adamw_eps=1e-3,
                     first_step_progress_log=False)
    x, y = _data(0)
    per = 4 // world
    x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
    loss = model(x, labels=y)
    (loss * 0.25 if how == "loss" else loss).backward()
    if how == "defer":
        opt.scale_grads_on_next_step(0.5)
        opt.scale_grads_on_next_step(torch.tensor(0.5))      # several calls multiply
    opt.step()
    assert opt._pending_gscale is None                       # used once
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    moms = {dp.fqn: opt.state[id(dp)]["momentum_buffer"].clone() for dp in opt.owned_muon_params()}
    return sd, moms


def test_deferred_gradient_scale_equals_scaling_the_loss():
    """``scale_grads_on_next_step(c)`` + ``step()`` gives what scaling every gradient
    by ``c`` gives: the Muon momentum buffers are ``c`` times the unscaled ones, and
    all weights (Muon and AdamW with a large eps, which makes AdamW scale-sensitive)
    equal those of a run whose loss was multiplied by ``c``."""
    a = run_ranks(_scaled_step_body, 2, args=("loss",))
    b = run_ranks(_scaled_step_body, 2, args=("defer",))
    c = run_ranks(_scaled_step_body, 2, args=("none",))
    for r in range(2):
        for k, v in a[r][0].items():
            assert (b[r][0][k].float() - v.float()).abs().max().item() < 1e-6, k
        for k, m in c[r][1].items():
            assert torch.allclose(b[r][1][k], 0.25 * m, atol=1e-7, rtol=1e-5), k
    # and it is not a no-op: AdamW-routed weights differ from the unscaled run
    diff = max((b[0][0][k].float() - c[0][0][k].float()).abs().max().item() for k in c[0][0] if "proj" not in k)
    assert diff > 1e-6


def _ctor_guard_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import _build_model, _pred

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    errors = []
    # (1) a model nobody prepared
    try:
        dmuon.Muon(_build_model())
    except RuntimeError as exc:
        errors.append(str(exc))
    # (2) dedicated matrices, but the remaining parameters neither sharded nor replicated: they would drift apart
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred)
    try:
        dmuon.Muon(model)
    except RuntimeError as exc:
        errors.append(str(exc))
    # (3) the same model once FSDP2 covers the rest
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    dmuon.Muon(model, first_step_progress_log=False)
    return errors


def test_optimizer_refuses_unprepared_models_and_unmanaged_parameters():
    for errors in run_ranks(_ctor_guard_body, 2):
        assert len(errors) == 2
        assert "dedicate_params" in errors[0]
        assert "neither dedicated nor covered" in errors[1] and "embed_tokens.weight" in errors[1]


class _SometimesBlock(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a_proj = nn.Linear(d, d, bias=False)
        self.b_proj = nn.Linear(d, d, bias=False)
        self.b_norm = nn.LayerNorm(d)

    def forward(self, x, use_b):
        x = x + torch.tanh(self.a_proj(x))
        if use_b:
            x = x + torch.tanh(self.b_proj(self.b_norm(x)))
        return x


class _SometimesNet(nn.Module):
    def __init__(self, vocab=64, d=32):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(_SometimesBlock(d) for _ in range(2))
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids, use_b):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x, use_b)
        return F.cross_entropy(self.head(x).flatten(0, 1), ids.flatten())


def _sometimes_data(step):
    return torch.randint(0, 64, (4, 16), generator=torch.Generator().manual_seed(500 + step))


def _sometimes_body(rank, world, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(3)
    model = _SometimesNet()
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2, adamw_weight_decay=0.01,
                     first_step_progress_log=False)
    per = 4 // world
    for s in range(steps):
        ids = _sometimes_data(s)[rank * per : (rank + 1) * per]
        opt.zero_grad()
        model(ids, use_b=(s % 2 == 1)).backward()
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


def test_parameters_without_a_gradient_are_skipped_and_keep_their_own_step_count():
    """A branch that only runs every other step: its Muon matrices and its AdamW
    tensors are skipped in the steps where they got no gradient (momentum and
    bias correction advance only when they are used), exactly like the
    single-process oracle does it."""
    from oracle import muon_adamw_run

    steps = 5
    torch.manual_seed(3)
    ref = _SometimesNet()
    muon_adamw_run(
        ref, lambda n, p: "proj" in n and p.ndim == 2, list(range(steps)),
        lambda m, s: m(_sometimes_data(s), use_b=(s % 2 == 1)),
        lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2, adamw_wd=0.01, betas=(0.9, 0.999), eps=1e-8,
    )
    sd = run_ranks(_sometimes_body, 2, args=(steps,))[0]
    for n, p in ref.named_parameters():
        assert (sd[n].float() - p.detach()).abs().max().item() < 5e-4, n


def _status_watch_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.ops import gemm as G
    from test_e2e_cpu import _build_model, _data, _pred

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, first_step_progress_log=False)
    x, y = _data(0)
    model(x, labels=y).backward()
    opt.step()                                      # on CPU nothing is polled
    polled_on_cpu = getattr(opt, "_status_polled", False)

    class _Landed:
        def query(self):
            return True

    class _InFlight:
        def query(self):
            return False

    # what a GPU step leaves behind: a host copy of the status word and the event that says it has landed
    fake_device_word = torch.tensor([4, 0, 0, 0], dtype=torch.int32)
    G_status = G.status_buffer
    G.status_buffer = lambda device: fake_device_word
    try:
        opt._status_host, opt._status_event, opt._status_polled = torch.tensor([4, 0, 0, 0], dtype=torch.int32), _InFlight(), True
        opt._raise_if_a_kernel_wait_ran_out()       # the copy has not landed: nothing is concluded, nothing waits
        still_pending = opt._status_polled
        opt._status_event = _Landed()
        msg = None
        try:
            opt._raise_if_a_kernel_wait_ran_out()
        except G.KernelTimeout as exc:
            msg = str(exc)
        cleared = int(fake_device_word[0]) == 0 and not opt._status_polled
        opt._status_host, opt._status_polled = torch.zeros(4, dtype=torch.int32), True
        opt._raise_if_a_kernel_wait_ran_out()       # a clean word raises nothing
    finally:
        G.status_buffer = G_status
    return polled_on_cpu, still_pending, msg, cleared


def test_a_wait_that_ran_out_is_reported_on_the_next_step_without_synchronising():
    (polled_on_cpu, still_pending, msg, cleared), = run_ranks(_status_watch_body, 1)
    assert polled_on_cpu is False and still_pending is True
    assert msg is not None and "code 4" in msg and "previous step" in msg
    assert cleared


def _presence_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.parallel import dgroup

    dgroup.CHECK_GRAD_PRESENCE = True          # what DMUON_CHECK_GRAD_PRESENCE=1 sets at import
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(3)
    model = _SometimesNet()
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, first_step_progress_log=False)
    ids = _sometimes_data(0)[rank * 2 : rank * 2 + 2]
    # same branch on every rank: fine
    model(ids, use_b=True).backward()
    opt.step()
    opt.zero_grad()
    # rank 0 takes the optional branch, rank 1 does not: b_proj has a gradient on rank 0 only
    err = None
    try:
        model(ids, use_b=(rank == 0)).backward()
    except RuntimeError as exc:
        err = str(exc)
    return err


def test_debug_check_names_parameters_whose_gradient_exists_on_some_ranks_only():
    """The packed reduce needs the same parameters to have gradients on every
    rank; with ``DMUON_CHECK_GRAD_PRESENCE=1`` a disagreement is reported (instead
    of a hang) with the parameter and the ranks."""
    for err in run_ranks(_presence_body, 2):
        assert err is not None and "ranks disagree" in err
        assert "b_proj.weight: gradient on data-parallel ranks [0] only" in err


class _ExpertBlock(nn.Module):
    """The optional branch holds dedicated matrices only (like the experts of an
    MoE layer): nothing of it is left to FSDP2, whose own reduce-scatter needs
    the same parameters to have gradients on every rank."""

    def __init__(self, d):
        super().__init__()
        self.a_proj = nn.Linear(d, d, bias=False)
        self.b_proj = nn.Linear(d, d, bias=False)

    def forward(self, x, use_b):
        x = x + torch.tanh(self.a_proj(x))
        if use_b:
            x = x + torch.tanh(self.b_proj(x))
        return x


class _ExpertNet(nn.Module):
    def __init__(self, vocab=64, d=32):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList(_ExpertBlock(d) for _ in range(2))
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids, use_b):
        x = self.embed(ids)
        for layer in self.layers:
            x = layer(x, use_b)
        return F.cross_entropy(self.head(x).flatten(0, 1), ids.flatten())


def _zero_fill_body(rank, world, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.parallel import dgroup

    dgroup.ZERO_FILL_MISSING_GRADS = True      # what DMUON_ZERO_FILL_MISSING_GRADS=1 sets at import
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(3)
    model = _ExpertNet()
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    fully_shard(model, mesh=mesh)              # embedding and head: used on every rank
    opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2, adamw_weight_decay=0.01,
                     first_step_progress_log=False)
    for s in range(steps):
        ids = _sometimes_data(s)[rank * 2 : rank * 2 + 2]
        opt.zero_grad()
        model(ids, use_b=(rank == 0)).backward()          # only rank 0 ever runs the optional branch
        opt.step()
    return dmuon.get_model_state_dict(model, rank0_only=False)


def test_zero_fill_lets_ranks_disagree_about_which_branch_ran():
    """With ``DMUON_ZERO_FILL_MISSING_GRADS=1`` a dedicated matrix without a
    gradient on a rank contributes zeros: rank 0 runs the optional branch, rank 1
    never does, nothing hangs, and all weights follow the single-process run whose
    loss is the mean of both ranks' losses (the branch's gradient is then half of
    rank 0's)."""
    from oracle import muon_adamw_run

    steps = 3
    torch.manual_seed(3)
    ref = _ExpertNet()

    def loss_fn(m, s):
        ids = _sometimes_data(s)
        return 0.5 * (m(ids[0:2], use_b=True) + m(ids[2:4], use_b=False))

    muon_adamw_run(
        ref, lambda n, p: "proj" in n and p.ndim == 2, list(range(steps)), loss_fn,
        lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2, adamw_wd=0.01, betas=(0.9, 0.999), eps=1e-8,
    )
    sd = run_ranks(_zero_fill_body, 2, args=(steps,), timeout=120)[0]
    for n, p in ref.named_parameters():
        assert (sd[n].float() - p.detach()).abs().max().item() < 5e-4, n


def _eval_between_body(rank, world, reshard):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from test_e2e_cpu import HP, _build_model, _data, _pred

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build_model()
    dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=reshard)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, reshard_after_forward=reshard)
    fully_shard(model, mesh=mesh, reshard_after_forward=reshard)
    opt = dmuon.Muon(model, lr=HP["lr"], ns_steps=5, adamw_lr=HP["adamw_lr"], weight_decay=HP["weight_decay"],
                     momentum=HP["momentum"], adamw_weight_decay=HP["adamw_wd"], first_step_progress_log=False)
    per = 4 // world
    evals = []
    for s in range(3):
        x, y = _data(s)
        x, y = x[rank * per : (rank + 1) * per], y[rank * per : (rank + 1) * per]
        opt.zero_grad()
        model(x, labels=y).backward()
        opt.step()
        # evaluation between steps: forwards without a backward, in eval mode and under no_grad, twice
        model.eval()
        with torch.no_grad():
            evals.append([float(model(x, labels=y)) for _ in range(2)])
        model.train()
    return dmuon.get_model_state_dict(model, rank0_only=False), evals


@pytest.mark.parametrize("reshard", [False, True])
def test_evaluation_forwards_between_steps_do_not_disturb_training(reshard):
    """Forward-only passes (``eval()`` + ``no_grad``) between optimizer steps see
    the freshly updated weights (both passes give the same loss) and leave the
    trajectory on the single-process one, with the published copies kept (Z2) or
    dropped (Z3) after forward."""
    from test_e2e_cpu import oracle_run

    _, ref_params = oracle_run(3)
    for sd, evals in run_ranks(_eval_between_body, 2, args=(reshard,)):
        assert all(abs(a - b) < 1e-6 for a, b in evals), evals
        for n, p in ref_params.items():
            assert (sd[n].float() - p).abs().max().item() < 5e-4, (reshard, n)

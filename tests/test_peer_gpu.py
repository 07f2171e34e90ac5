"""Peer-memory kernels.  On one GPU the "ranks" are emulated as one kernel
reading several local arenas; with two or more GPUs the whole data plane is
compared against the NCCL implementation."""
import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def test_peer_prologue_reduces_in_rank_order_and_applies_momentum():
    from dmuon_b200.ops import peer as P

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    W = 4
    sizes = [1024 * 3 + 8, 4096, 40]
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + 63) // 64 * 64
    arenas = [torch.randn(total, device=dev).bfloat16() for _ in range(W)]
    moms = [torch.randn(n, device=dev) for n in sizes]
    m0 = [m.clone() for m in moms]
    xs = [torch.empty(n, device=dev, dtype=torch.bfloat16) for n in sizes]
    sumsq = torch.zeros(3, device=dev)
    flags = torch.full((8,), 5, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    P.peer_prologue([a.data_ptr() for a in arenas], offs, sizes, torch.bfloat16, moms, xs, [0, 1, 2], sumsq,
                    scale=1.0 / W, mu=0.95, nesterov=True, ready_flags=flags, ready_want=5, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    for i, n in enumerate(sizes):
        g = torch.zeros(n, device=dev)
        for a in arenas:                       # same order as the kernel
            g = g + a[offs[i] : offs[i] + n].float()
        g = g / W
        m = 0.95 * m0[i] + g
        u = g + 0.95 * m
        assert torch.allclose(moms[i], m, atol=1e-5)
        assert (xs[i].float() - u).abs().max().item() < 0.02 * u.abs().max().item()
        assert abs(sumsq[i].item() - float((u * u).sum())) < 1e-3 * float((u * u).sum())
    # reduce only (no momentum): fp32 result
    outs = [torch.empty(n, device=dev) for n in sizes]
    P.peer_prologue([a.data_ptr() for a in arenas], offs, sizes, torch.bfloat16, [None] * 3, outs, [0, 0, 0], None,
                    scale=1.0 / W, mu=0.0, nesterov=False)
    torch.cuda.synchronize()
    for i, n in enumerate(sizes):
        g = sum(a[offs[i] : offs[i] + n].float() for a in arenas) / W
        assert torch.allclose(outs[i], g, atol=1e-5)


def test_pull_and_signal_on_one_device():
    from dmuon_b200.ops import peer as P

    dev = torch.device("cuda", 0)
    src = torch.randn(1 << 20, device=dev).bfloat16()
    dst = torch.zeros_like(src)
    flags = torch.zeros(32, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    P.signal_peers([flags.data_ptr()], 3, 7, dev)            # "owner" announces epoch 7 in slot 3
    P.peer_pull([src.data_ptr()], [dst.data_ptr()], [src.numel() * 2], [3], flags, 7, status, dev)
    torch.cuda.synchronize()
    assert int(flags[3]) == 7 and int(status[0]) == 0
    assert torch.equal(src, dst)


@pytest.mark.parametrize("M,N,K", [(1000, 600, 512), (4096, 1024, 2048), (300, 256, 96), (128, 2304, 1152)])
def test_pull_linear_fetches_and_multiplies(M, N, K):
    """The "owner" is a second buffer on the same GPU: the kernel must leave an
    exact copy in the local slot and multiply with it."""
    import torch.nn.functional as F

    from dmuon_b200.ops import gemm as G
    from dmuon_b200.ops import pull_linear as PL

    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    x = (torch.randn(M, K, device=dev) * 0.1).bfloat16()
    w_owner = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
    w_local = torch.zeros_like(w_owner)
    flag = torch.full((4,), 3, dtype=torch.int32, device=dev)
    y = PL.pull_linear(x, w_local, w_owner.data_ptr(), pub_flag=flag[1:], pub_want=3)
    torch.cuda.synchronize()
    G.check_status(dev)
    assert torch.equal(w_local, w_owner)
    ref = F.linear(x.float(), w_owner.float())
    assert (y.float() - ref).abs().max().item() < 2e-2 * (ref.abs().max().item() + 1e-6)
    # second use in the same epoch: plain multiplication with the local copy
    y2 = PL.pull_linear(x, w_local)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    # autograd wrapper
    xg = x.clone().requires_grad_(True)
    wp = torch.nn.Parameter(torch.zeros_like(w_owner))
    out = PL.PulledLinearFn.apply(xg, wp, None, w_owner.data_ptr(), flag[1:], 3, 0)
    out.float().square().sum().backward()
    xr = x.float().clone().requires_grad_(True)
    wr = w_owner.float().clone().requires_grad_(True)
    F.linear(xr, wr).bfloat16().float().square().sum().backward()
    assert (xg.grad.float() - xr.grad).abs().max().item() < 3e-2 * (xr.grad.abs().max().item() + 1e-6)
    assert (wp.grad.float() - wr.grad).abs().max().item() < 3e-2 * (wr.grad.abs().max().item() + 1e-6)


def test_flag_wait_times_out_cleanly():
    """A flag nobody sets: the wait gives up after its budget, reports status 4
    and the context stays usable."""
    from dmuon_b200.ops import peer as P

    dev = torch.device("cuda", 0)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    P.wait_flags(flags, 0, 2, 1, status, budget_cycles=20_000_000)      # ~10 ms
    torch.cuda.synchronize()
    assert int(status[0]) == 4
    status.zero_()
    out = torch.empty(64, device=dev)
    P.peer_prologue([flags.data_ptr()], [0], [8], torch.float32, [None], [out[:8]], [0], None, scale=1.0, mu=0.0,
                    nesterov=False, ready_flags=flags, ready_want=9, status=status, budget_cycles=20_000_000)
    torch.cuda.synchronize()
    assert int(status[0]) == 4
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0


def _train_body(rank, world, backend, steps):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    import os

    if backend == "peer-fused":
        os.environ["DMUON_FUSED_PUBLISH"] = "1"
        backend = "peer"
    if backend == "peer-optimizer-reduce":
        os.environ["DMUON_PEER_REDUCE"] = "optimizer"
        os.environ["DMUON_PEER_COPY"] = "ce"
        backend = "peer"
    if backend in ("peer-ce", "peer-nvls", "peer-hybrid"):
        os.environ["DMUON_PEER_COPY"] = backend[5:]
        backend = "peer"
    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=2048, d_model=512, n_layers=3, n_heads=8, n_kv_heads=4, head_dim=64,
                      ffn_hidden=1536, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg)
    hsdp = backend == "hsdp-flat"
    if hsdp:
        # a replicate x shard grid on one host: ownership is flattened onto the peer plane
        mesh = init_device_mesh("cuda", (world, 1), mesh_dim_names=("replicate", "shard"))
        owners = dmuon.dedicate_params(model, mesh["shard"], lambda n, p: "proj" in n and p.ndim == 2,
                                       param_policy={"defaults": {"param_dtype": "bf16", "grad_dtype": "fp32"}},
                                       reshard_after_forward=False, replicate_mesh=mesh["replicate"])
        assert model._dedicated_comm_ctx.hsdp_flattened
        assert all(isinstance(o, tuple) and o[0] == 0 and o[1] in range(world) for o in owners.values())
        assert len({o for o in owners.values()}) == world
    else:
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
        # fp32 gradient buffers on both data planes: with two ranks the sum is then the
        # same number whoever computes it, so the trajectories can be compared tightly
        dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2,
                              param_policy={"defaults": {"param_dtype": "bf16", "grad_dtype": "fp32"}},
                              reshard_after_forward=False, comm_backend=backend)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3, weight_decay=0.1)
    used_peer = model._dedicated_comm_ctx.peer_runtime is not None
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for s in range(steps):
        ids = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)
        opt.zero_grad()
        if s == 1:                      # one accumulation step with two micro-batches
            (model(ids[:1, :-1], labels=ids[:1, 1:]) / 2).backward()
            loss = model(ids[1:, :-1], labels=ids[1:, 1:]) / 2
        else:
            loss = model(ids[:, :-1], labels=ids[:, 1:])
        loss.backward()
        if s == 2:
            dmuon.clip_grad_norm_(opt, 0.5)
        opt.step()
        lt = loss.detach().float().clone()
        dist.all_reduce(lt)
        losses.append(float(lt) / world)
    if used_peer:
        model._dedicated_comm_ctx.peer_runtime.check()
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    # weight gradients of plain Linear layers go straight into the arena unless the fused publish owns the forward
    direct = sum(1 for m in model.modules() if hasattr(m, "_dmuon_direct"))
    return losses, {k: v for k, v in sd.items() if "proj" in k}, used_peer, direct


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_data_plane_matches_nccl():
    world = 2
    steps = 4
    ref = run_ranks(_train_body, world, args=("nccl", steps), backend="nccl", timeout=600)
    got = run_ranks(_train_body, world, args=("peer-ce", steps), backend="nccl", timeout=600)
    alt = run_ranks(_train_body, world, args=("peer-optimizer-reduce", steps), backend="nccl", timeout=600)
    nvls = run_ranks(_train_body, world, args=("peer-nvls", steps), backend="nccl", timeout=600)
    assert nvls[0][2] and nvls[0][3] == 21
    for a, b in zip(nvls[0][0], ref[0][0]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (nvls[0][0], ref[0][0])
    for k, v in ref[0][1].items():
        rel = (nvls[0][1][k].float() - v.float()).norm().item() / (v.float().norm().item() + 1e-12)
        assert rel < 0.15, (k, rel)
    flat = run_ranks(_train_body, world, args=("hsdp-flat", steps), backend="nccl", timeout=600)
    assert flat[0][2] and flat[0][3] == 21
    for a, b in zip(flat[0][0], ref[0][0]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (flat[0][0], ref[0][0])
    assert not ref[0][2] and got[0][2] and alt[0][2]
    assert ref[0][3] == 0 and got[0][3] == 21 and alt[0][3] == 21      # 3 layers x 7 projections
    for a, b, c in zip(got[0][0], ref[0][0], alt[0][0]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (got[0][0], ref[0][0])
        assert abs(c - b) < 2e-2 * max(1.0, abs(b)), (alt[0][0], ref[0][0])
    # Two separate runs never see bit-identical gradients (the attention backward
    # and the sharded reductions are not deterministic) and the fp16 Gram iteration
    # amplifies last-bit differences along singular directions below fp16's
    # resolution of the Gram matrix: two runs of ONE implementation already differ
    # by 1-4 % in square matrices after three steps (measured in
    # tests/test_tp_peer_gpu.py).  So this end-to-end check is a sanity bound;
    # exactness of reduce and publish is asserted by the test below.
    for k, v in ref[0][1].items():
        rel = (got[0][1][k].float() - v.float()).norm().item() / (v.float().norm().item() + 1e-12)
        assert rel < 0.15, (k, rel)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_forward_publish_matches_nccl():
    """Weights pulled inside the first forward GEMM instead of by a copy kernel."""
    steps = 4
    ref = run_ranks(_train_body, 2, args=("nccl", steps), backend="nccl", timeout=600)
    got = run_ranks(_train_body, 2, args=("peer-fused", steps), backend="nccl", timeout=600)
    assert got[0][2]
    for a, b in zip(got[0][0], ref[0][0]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (got[0][0], ref[0][0])
    for k, v in ref[0][1].items():
        rel = (got[0][1][k].float() - v.float()).norm().item() / (v.float().norm().item() + 1e-12)
        assert rel < 0.15, (k, rel)


def _reduce_check_body(rank, world, fused=False, reduce_mode="backward", copy_mode="ce"):
    import os

    import torch.distributed as dist

    if reduce_mode == "epilogue":
        # NVSwitch plane with the multicast store issued by the update GEMM's epilogue
        os.environ["DMUON_NVLS_PUBLISH"] = "epilogue"
        reduce_mode = "backward"
    os.environ["DMUON_PEER_REDUCE"] = reduce_mode
    os.environ["DMUON_PEER_COPY"] = copy_mode
    os.environ["DMUON_DEBUG_CANARY"] = "1"          # guard bands around both arenas, verified by rt.check()
    if fused:
        os.environ["DMUON_FUSED_PUBLISH"] = "1"
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=4, head_dim=64,
                      ffn_hidden=512, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg).bfloat16()
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, comm_backend="peer")
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02)
    rt = model._dedicated_comm_ctx.peer_runtime
    worst = 0.0
    for step in range(2):
        g = torch.Generator().manual_seed(7 + rank + 10 * step)
        ids = torch.randint(0, cfg.vocab_size, (2, 65), generator=g).to(dev)
        opt.zero_grad()
        model(ids[:, :-1], labels=ids[:, 1:]).backward()
        # what an all-reduce of the local arenas would give
        want = {}
        for dp in dmuon.get_dedicated_params(model):
            t = dp._grad_view.float().clone()
            dist.all_reduce(t)
            want[dp.fqn] = t / world
        opt._ensure_grads_ready(materialize=True)
        for dp in dmuon.get_owned_params(model):
            got = dp._reduced_grad
            worst = max(worst, (got - want[dp.fqn]).abs().max().item() / (want[dp.fqn].abs().max().item() + 1e-12))
        # published weights: every rank's copy equals the owner's master weights in bf16
        opt.step()
        model(ids[:, :-1])                       # forward pulls the new epoch
        torch.cuda.synchronize()
        for dp in dmuon.get_dedicated_params(model):
            ref = dp._owned_data.to(torch.bfloat16) if dp.is_owner else torch.empty(dp._orig_size, dtype=torch.bfloat16, device=dev)
            dist.broadcast(ref, src=dp.owner_shard)
            assert torch.equal(dp._unsharded_param.data, ref), dp.fqn
    assert rt.canary and rt.guard > 0 and rt.copy_mode == ("sm" if fused else copy_mode)
    rt.check()
    return worst


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize(
    "fused,reduce_mode,copy_mode",
    [(False, "backward", "nvls"), (False, "epilogue", "nvls"), (False, "backward", "hybrid"), (False, "backward", "ce"), (False, "optimizer", "ce"), (False, "backward", "sm"),
     (False, "optimizer", "sm"), (True, "backward", "sm")],
)
def test_peer_reduce_and_publish_are_exact(fused, reduce_mode, copy_mode):
    """Copy-engine transfers + local sum ("ce") and the kernels that load through the
    peer mappings ("sm") must both deliver exactly the mean gradient and the owner's weights.
    The NVSwitch form ("nvls") publishes exactly as well (the update kernel's multicast
    store carries the same bf16 values); its gradient sum is formed in the switch with fp32
    accumulation and rounded once to the bf16 gradient type, so it is within one bf16
    rounding of the exact mean, in the switch's order rather than rank order."""
    world = min(8, torch.cuda.device_count())
    worst = run_ranks(_reduce_check_body, world, args=(fused, reduce_mode, copy_mode), backend="nccl", timeout=600)
    assert max(worst) < (1e-5 if copy_mode not in ("nvls", "hybrid") else 1.2e-2), worst


def _scalar_body(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=256, d_model=128, n_layers=1, n_heads=2, n_kv_heads=2, head_dim=64,
                      ffn_hidden=256, rope_theta=10000.0)
    with torch.device(dev):
        model = LlamaModel(cfg).bfloat16()
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, comm_backend="peer")
    fully_shard(model, mesh=mesh)
    rt = model._dedicated_comm_ctx.peer_runtime
    worst = 0.0
    for it in range(5):                                    # odd count: both slot parities get reused
        local = torch.tensor([rank + 1.0 + it, 10.0 * (rank + 1), 0.5 * it], device=dev)
        sums, coef = rt.scalar_allreduce(local, max_norm=2.0)
        want = local.clone()
        dist.all_reduce(want)
        worst = max(worst, (sums - want).abs().max().item())
        want_coef = torch.clamp(2.0 / (want.sqrt() + 1e-6), max=1.0)
        worst = max(worst, (coef - want_coef).abs().max().item())
    rt.check()
    return worst


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_in_kernel_scalar_allreduce_matches_nccl():
    world = min(8, torch.cuda.device_count())
    worst = run_ranks(_scalar_body, world, backend="nccl", timeout=300)
    assert max(worst) < 1e-5, worst


def _ckpt_body(rank, world, plane="auto"):
    import os

    if plane == "fused":
        os.environ["DMUON_FUSED_PUBLISH"] = "1"
    else:
        os.environ["DMUON_PEER_COPY"] = plane
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=256, d_model=128, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=64,
                      ffn_hidden=256, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg).bfloat16()
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, comm_backend="peer")
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, 65), generator=torch.Generator().manual_seed(3)).to(dev)

    def step():
        opt.zero_grad()
        model(ids[:, :-1], labels=ids[:, 1:]).backward()
        opt.step()

    def evaluate():
        with torch.no_grad():
            return float(model(ids[:, :-1], labels=ids[:, 1:]))

    # a load before any step (the usual resume) and one after an evaluation-only forward: neither epoch
    # saw a backward, so the owners' "everybody is done with the old weights" wait must not depend on one
    initial = dmuon.get_model_state_dict(model, rank0_only=False)
    dmuon.set_model_state_dict(model, initial)
    first = evaluate()
    dmuon.set_model_state_dict(model, initial)
    assert evaluate() == first
    step()
    saved = dmuon.get_model_state_dict(model, rank0_only=False)
    at_save = evaluate()
    step()
    step()
    moved = evaluate()
    dmuon.set_model_state_dict(model, saved)
    restored = evaluate()
    model._dedicated_comm_ctx.peer_runtime.check()
    return at_save, moved, restored


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("plane", ["auto", "nvls", "ce", "fused"])
def test_loading_a_state_dict_republishes_on_the_peer_plane(plane):
    for at_save, moved, restored in run_ranks(_ckpt_body, 2, args=(plane,), backend="nccl", timeout=300):
        assert abs(moved - at_save) > 1e-3          # training did change the weights
        assert restored == at_save                  # and every rank reads the restored ones again


def _accum_body(rank, world, use_no_sync, plane):
    import contextlib
    import os

    os.environ["DMUON_PEER_COPY"] = plane
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=256, d_model=128, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=64,
                      ffn_hidden=256, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg)
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, comm_backend="peer",
                          param_policy={"defaults": {"param_dtype": "bf16", "grad_dtype": "fp32"}})
    from torch.distributed.fsdp import MixedPrecisionPolicy

    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    opt = dmuon.Muon(model, lr=0.02)
    g = torch.Generator().manual_seed(50 + rank)
    for _ in range(2):
        ids = torch.randint(0, cfg.vocab_size, (4, 65), generator=g).to(dev)
        opt.zero_grad()
        hold = dmuon.no_sync(model) if use_no_sync else contextlib.nullcontext()
        with hold:      # first micro-batch: with no_sync nothing is announced to the owners yet
            (model(ids[:2, :-1], labels=ids[:2, 1:]) / 2).backward()
        (model(ids[2:, :-1], labels=ids[2:, 1:]) / 2).backward()
        opt.step()
    model._dedicated_comm_ctx.peer_runtime.check()
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return {k: v for k, v in sd.items() if "proj" in k}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("plane", ["auto", "nvls", "ce"])
def test_no_sync_accumulation_on_the_peer_plane(plane):
    """Two micro-batches per step: accumulating the first one locally under
    ``no_sync`` gives the weights that two synchronised backward passes give
    (the reference's criterion is 1e-2 max abs, tests/distributed/test_grad_accum.py:226-229)."""
    a = run_ranks(_accum_body, 2, args=(False, plane), backend="nccl", timeout=300)
    b = run_ranks(_accum_body, 2, args=(True, plane), backend="nccl", timeout=300)
    for k, v in a[0].items():
        assert (b[0][k].float() - v.float()).abs().max().item() < 1e-2, k
        assert torch.equal(b[0][k], b[1][k])


def _ddp_peer_body(rank, world, plane):
    import os

    import torch.distributed as dist

    os.environ["DMUON_PEER_COPY"] = plane
    from torch.distributed.device_mesh import init_device_mesh

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=4, head_dim=64,
                      ffn_hidden=512, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg).bfloat16()
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params_ddp(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, comm_backend="peer")
    dmuon.replicate(model, mesh)
    ctx = model._dedicated_comm_ctx
    assert ctx.ddp_on_peer_plane and ctx.peer_runtime is not None and ctx.mode == "ddp"
    assert ctx.peer_runtime.copy_mode == plane
    opt = dmuon.Muon(model, lr=0.02)
    worst, losses = 0.0, []
    g = torch.Generator().manual_seed(7 + rank)
    ids = torch.randint(0, cfg.vocab_size, (2, 65), generator=g).to(dev)      # one batch, so the loss must fall
    for step in range(3):
        opt.zero_grad()
        loss = model(ids[:, :-1], labels=ids[:, 1:])
        loss.backward()
        want = {}
        for dp in dmuon.get_dedicated_params(model):
            t = dp._grad_view.float().clone()
            dist.all_reduce(t)
            want[dp.fqn] = t / world
        opt._ensure_grads_ready(materialize=True)
        for dp in dmuon.get_owned_params(model):
            worst = max(worst, (dp._reduced_grad - want[dp.fqn]).abs().max().item() / (want[dp.fqn].abs().max().item() + 1e-12))
        opt.step()
        lt = loss.detach().float().clone()
        dist.all_reduce(lt)
        losses.append(float(lt) / world)
        model(ids[:, :-1])
        torch.cuda.synchronize()
        for dp in dmuon.get_dedicated_params(model):
            ref = dp._owned_data.to(torch.bfloat16) if dp.is_owner else torch.empty(dp._orig_size, dtype=torch.bfloat16, device=dev)
            dist.broadcast(ref, src=dp.owner_shard)
            assert torch.equal(dp._unsharded_param.data, ref), dp.fqn
    # the replicated (non-dedicated) parameters stay identical across ranks
    for n, p in model.named_parameters():
        if "proj" not in n:
            q = p.detach().float().clone()
            dist.broadcast(q, src=0)
            assert torch.equal(q, p.detach().float()), n
    ctx.peer_runtime.check()
    return worst, losses


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("plane", ["nvls", "ce"])
def test_replicated_placement_runs_on_the_peer_plane(plane):
    """``dedicate_params_ddp`` + ``replicate`` on one NVSwitch domain: the
    dedicated matrices are reduced out of the ranks' gradient arenas and the
    owner's update reaches every rank's copy (no NCCL reduce / fp32 broadcast);
    the mean gradient and the published weights are checked against collectives."""
    world = min(4, torch.cuda.device_count())
    res = run_ranks(_ddp_peer_body, world, args=(plane,), backend="nccl", timeout=600)
    assert max(r[0] for r in res) < (1e-5 if plane == "ce" else 1.2e-2)
    losses = res[0][1]
    assert losses[-1] < losses[0]

"""Tensor-parallel gather -> Newton-Schulz -> scatter with the shards moved over
peer memory (``parallel/tp_peer.py``) against the collective implementation
(NCCL gather / ``torch.cat`` / scatter) on the same ranks."""
import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _body(rank, world, use_peer, clip, steps, single_pass=True, torch_ns=False):
    import os

    os.environ["DMUON_TP_PEER"] = "1" if use_peer else "0"
    os.environ["DMUON_NS_SINGLE_PASS"] = "1" if single_pass else "0"      # read when the kernels' module is imported
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    dev = torch.device("cuda", rank)
    tp = 2
    mesh = init_device_mesh("cuda", (world // tp, tp), mesh_dim_names=("dp", "tp"))
    cfg = LlamaConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64,
                      ffn_hidden=768, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg)
    plan = {
        "self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(),
        "self_attn.v_proj": ColwiseParallel(), "self_attn.o_proj": RowwiseParallel(),
        "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel(),
    }
    for layer in model.layers:
        parallelize_module(layer, mesh["tp"], plan)
    dmuon.dedicate_params(model, mesh["dp"], lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh["dp"])
    fully_shard(model, mesh=mesh["dp"])
    extra = {}
    if torch_ns:
        # fp32 PyTorch Newton-Schulz: no fp16 rounding to amplify, so the two transports must agree tightly
        extra["ns_backend"] = dmuon.NewtonSchulz(kernel="torch", compute_dtype=torch.float32)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3, weight_decay=0.1, first_step_progress_log=False, **extra)
    ctx = model._dedicated_comm_ctx
    assert bool(ctx.tp_exchanges) == use_peer
    g = torch.Generator().manual_seed(31 + mesh["dp"].get_local_rank())      # TP peers see the same batch
    losses, first = [], None
    from torch.nn.attention import SDPBackend, sdpa_kernel

    for _ in range(steps):
        # 512 tokens: the 256-wide matrices get full-rank gradients (Newton-Schulz amplifies rounding noise
        # along the null directions of a rank-deficient one); matmul attention: its backward has no atomics,
        # so the two runs that are compared see the same gradients
        ids = torch.randint(0, cfg.vocab_size, (4, 129), generator=g).to(dev)
        opt.zero_grad()
        with sdpa_kernel(SDPBackend.MATH):
            loss = model(ids[:, :-1], labels=ids[:, 1:])
            loss.backward()
        if clip:
            dmuon.clip_grad_norm_(opt, 0.5)
        opt.step()
        if first is None:
            first = {k: v for k, v in dmuon.get_model_state_dict(model, rank0_only=False).items() if "proj" in k}
        lt = loss.detach().float().clone()
        dist.all_reduce(lt)
        losses.append(float(lt) / world)
    for ex in ctx.tp_exchanges.values():
        ex.check()
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return losses, {k: v for k, v in sd.items() if "proj" in k}, first


def _rel(a: dict, b: dict) -> dict:
    return {k: (a[k].float() - v.float()).norm().item() / (v.float().norm().item() + 1e-12) for k, v in b.items()}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("clip", [False, True])
def test_tp_gather_scatter_over_peer_memory_matches_collectives(clip):
    """Row- and column-sharded matrices, DP x TP = (1 or 2) x 2, peer-memory
    path against the collective path.

    The two paths differ only in the order in which the shards' sums of squares
    are added (atomics: the order is not even fixed within one path).  Where
    the sum comes out the same, the weights after one step agree to the last
    bit or two; where it differs in the last bit, another fp16 rounding of the
    Newton-Schulz operand follows, and the fp16 Gram iteration turns that into
    a visible difference along the gradient's weak singular directions (they
    sit below fp16's resolution of the Gram matrix; on this model up to 4 % of
    a square matrix after three steps).  How large "visible" is gets measured,
    not assumed: the collective path is run once more with the other, equally
    valid operand rounding (two-pass instead of single-pass cast), and the peer
    path has to stay within a small multiple of that distance -- and, without
    clipping (a clip coefficient reaches every matrix), at least half of the
    matrices must agree to 1e-6 after the first step, which only holds if every
    shard lands where it belongs on the way in and on the way out."""
    world = 4 if torch.cuda.device_count() >= 4 else 2
    ref = run_ranks(_body, world, args=(False, clip, 3), backend="nccl", timeout=600)
    alt = run_ranks(_body, world, args=(False, clip, 3, False), backend="nccl", timeout=600)
    got = run_ranks(_body, world, args=(True, clip, 3), backend="nccl", timeout=600)
    for a, b in zip(got[0][0], ref[0][0]):
        assert abs(a - b) < 1e-2 * max(1.0, abs(b)), (got[0][0], ref[0][0])
    one = _rel(got[0][2], ref[0][2])
    noise = _rel(alt[0][1], ref[0][1])
    three = _rel(got[0][1], ref[0][1])
    fmt = lambda d: {k.replace("layers.", "").replace(".weight", ""): f"{r:.1e}" for k, r in d.items()}  # noqa: E731
    print("after one step, peer vs collective:", fmt(one))
    print("after three steps, collective vs collective with the other operand rounding:", fmt(noise))
    print("after three steps, peer vs collective:", fmt(three))
    if not clip:
        exact = sum(1 for r in one.values() if r < 1e-6)
        assert 2 * exact >= len(one), one
    for k in three:
        assert one[k] < 3.0 * noise[k] + 5e-3, (k, one[k], noise[k])
        assert three[k] < 3.0 * noise[k] + 5e-3, (k, three[k], noise[k])
    # every rank reports the same full tensors
    for k, v in got[0][1].items():
        assert torch.equal(v, got[-1][1][k]), k


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_peer_exchange_is_exact_when_newton_schulz_runs_in_fp32():
    """With the fp32 PyTorch iteration nothing amplifies last-bit differences, and
    the peer path then only moves bytes (shards copied into the symmetric buffer,
    assembled by the gather kernel, the update copied into the owner's slot, slices
    pulled and applied): weights must match the collective path to rounding, with
    clipping in the loop (its norm is summed in another order)."""
    world = 4 if torch.cuda.device_count() >= 4 else 2
    ref = run_ranks(_body, world, args=(False, True, 3, True, True), backend="nccl", timeout=600)
    got = run_ranks(_body, world, args=(True, True, 3, True, True), backend="nccl", timeout=600)
    worst = _rel(got[0][1], ref[0][1])
    print("fp32 Newton-Schulz, peer vs collective after three steps:", {k: f"{r:.1e}" for k, r in worst.items()})
    assert max(worst.values()) < 3e-4, worst

"""Whole training steps on one GPU through the public API (collective data
plane with a world of one): the update kernels leave the bf16 publish copy in
the packed forward buffer, so the next forward reads exactly ``bf16(master)``
without a copy-in, and the loss goes down on a fixed batch."""
import pytest
import torch

from dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _body(rank, world, reshard_after_forward, steps):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel
    from dmuon_b200.ops.multi_tensor import launch_count

    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(vocab_size=2048, d_model=512, n_layers=3, n_heads=8, n_kv_heads=4, head_dim=64,
                      ffn_hidden=1536, rope_theta=10000.0, loss_chunk=128)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaModel(cfg)
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, compute_dtype=torch.bfloat16,
                          reshard_after_forward=reshard_after_forward)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3, weight_decay=0.1)
    ids = torch.randint(0, cfg.vocab_size, (2, 257), generator=torch.Generator().manual_seed(5)).to(dev)
    losses, fresh_hits, mismatches = [], 0, 0
    before = launch_count()
    for s in range(steps):
        opt.zero_grad()
        loss = model(ids[:, :-1], labels=ids[:, 1:])
        if s > 0:
            # the forward that just ran consumed the copies the update kernels wrote
            for p in dmuon.get_dedicated_params(model):
                live = p._unsharded_param.data
                if live.untyped_storage().size() and not torch.equal(live, p._owned_data.to(torch.bfloat16)):
                    mismatches += 1
        loss.backward()
        opt.step()
        fresh_hits += sum(1 for p in dmuon.get_dedicated_params(model) if p._publish_fresh)
        losses.append(float(loss))
    n_ded = len(dmuon.get_dedicated_params(model))
    return losses, fresh_hits, mismatches, n_ded, launch_count() - before


@pytest.mark.parametrize("reshard_after_forward", [False, True])
def test_single_gpu_training_step(reshard_after_forward):
    steps = 4
    losses, fresh_hits, mismatches, n_ded, launches = run_ranks(
        _body, 1, args=(reshard_after_forward, steps), backend="nccl", timeout=600
    )[0]
    assert n_ded == 21
    assert fresh_hits == steps * n_ded        # every owned matrix was published by the update kernel
    assert mismatches == 0
    assert launches > 0
    assert losses[-1] < losses[0] - 0.5, losses

"""Pi0-style VLA model: shapes, flow-matching loss, and a 2-rank FSDP2 +
dedicated Muon run with per-block hook boundaries on CPU."""
import torch

from dist_utils import run_ranks


def test_pi0_tiny_forward_backward_single_process():
    from dmuon_b200.models.pi0 import Pi0Config, Pi0Model, sample_flow_time, synthetic_batch

    torch.manual_seed(0)
    cfg = Pi0Config.tiny()
    model = Pi0Model(cfg)
    batch = synthetic_batch(cfg, 3, "cpu")
    v = model.velocity(*batch[:3], batch[3], torch.full((3,), 0.5))
    assert v.shape == (3, cfg.action_horizon, cfg.action_dim)
    loss = model(*batch)
    loss.backward()
    assert torch.isfinite(loss)
    # the prefix stream of the last layer is unused (only its keys/values matter)
    no_grad = [n for n, p in model.named_parameters() if p.grad is None]
    assert all(n.startswith("layers.1.backbone.") and ("k_proj" not in n and "v_proj" not in n) for n in no_grad), no_grad
    t = sample_flow_time(1000, "cpu")
    assert 0.001 <= float(t.min()) and float(t.max()) <= 1.0 and 0.55 < float(t.mean()) < 0.65   # Beta(1.5, 1) mean 0.6
    full = Pi0Config()
    assert full.tokens_per_image == 256 and full.vit_mlp == 4304 and full.head_dim == 256


def _body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.pi0 import Pi0Config, Pi0Model, synthetic_batch

    torch.manual_seed(0)
    cfg = Pi0Config.tiny()
    model = Pi0Model(cfg)
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    owners = dmuon.dedicate_params(model, mesh, lambda n, p: "proj" in n and p.ndim == 2, reshard_after_forward=False)
    for blk in list(model.vision.blocks) + list(model.layers):
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, adamw_lr=1e-3)
    g = torch.Generator().manual_seed(5 + rank)
    batch = synthetic_batch(cfg, 2, "cpu", g)
    noise = torch.randn(batch[3].shape, generator=g)
    t = torch.full((2,), 0.4)
    losses = []
    for _ in range(6):
        opt.zero_grad()
        loss = model(*batch, noise=noise, t=t)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    plan = dmuon.summarize_comm_plan(model)
    names = sorted(g["name"] for g in plan["groups"])
    return losses, names, len(owners), sorted(set(owners.values()))


def test_pi0_two_rank_training_uses_block_boundaries():
    res = run_ranks(_body, 2)
    losses, names, n_owned, owner_set = res[0]
    assert losses[-1] < losses[0] and all(l == l for l in losses)
    assert owner_set == [0, 1]
    # one hook boundary per ViT block and per joint layer, plus the projection outside any block
    assert "vision.blocks.0" in names and "vision.blocks.1" in names
    assert "layers.0" in names and "layers.1" in names and "vision.out_proj" in names
    # 2 ViT blocks x 6 + out_proj + 2 joint layers x 14 matrices
    assert n_owned == 2 * 6 + 1 + 2 * 14

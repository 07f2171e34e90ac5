"""Mixture-of-experts decoder under dedicated ownership (2 gloo ranks): with so
few tokens per rank that most experts are idle on a rank, training follows the
single-process run on the union of the ranks' data."""
import torch

from dist_utils import run_ranks

STEPS = 3


def _cfg():
    from dmuon_b200.models.moe import MoEConfig

    # 8 experts, top-1, 4 tokens per rank: at least four experts per layer get no token on a rank
    return MoEConfig.tiny(n_experts=8, top_k=1, expert_hidden=64, d_model=64, n_heads=2, n_kv_heads=2, head_dim=32, vocab_size=128)


def _ids(step):
    return torch.randint(0, 128, (2, 5), generator=torch.Generator().manual_seed(900 + step))


def _pred(name, p):
    return "proj" in name and p.ndim == 2


def _body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.moe import MoEModel
    from dmuon_b200.parallel import dgroup

    dgroup.ZERO_FILL_MISSING_GRADS = True      # what DMUON_ZERO_FILL_MISSING_GRADS=1 sets at import
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    torch.manual_seed(5)
    model = MoEModel(_cfg())
    owners = dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2, adamw_weight_decay=0.01,
                     first_step_progress_log=False)
    idle = 0
    for s in range(STEPS):
        ids = _ids(s)[rank : rank + 1]
        opt.zero_grad()
        model(ids[:, :-1], labels=ids[:, 1:]).backward()
        opt.step()
    # how many expert matrices were idle on this rank in a fresh forward/backward (sanity of the premise)
    ids = _ids(0)[rank : rank + 1]
    probe = MoEModel(_cfg())
    probe(ids[:, :-1], labels=ids[:, 1:]).backward()
    idle = sum(1 for n, p in probe.named_parameters() if "experts" in n and p.grad is None)
    plan = dmuon.summarize_comm_plan(model)
    return dmuon.get_model_state_dict(model, rank0_only=False), idle, len(owners), plan["groups"][0]["param_count"]


def test_moe_decoder_with_idle_experts_follows_the_single_process_run():
    from dmuon_b200.models.moe import MoEModel
    from oracle import muon_adamw_run

    torch.manual_seed(5)
    ref = MoEModel(_cfg())

    def loss_fn(m, s):
        ids = _ids(s)
        # with zero-fill an expert that no rank used still gets a (zero) gradient, so its momentum and weight
        # decay keep acting; the single-process run gets the same by touching every expert weight with a zero
        touch = sum(p.sum() for n, p in m.named_parameters() if "experts" in n)
        return 0.5 * (m(ids[0:1, :-1], labels=ids[0:1, 1:]) + m(ids[1:2, :-1], labels=ids[1:2, 1:])) + 0.0 * touch

    muon_adamw_run(ref, _pred, list(range(STEPS)), loss_fn, lr=0.02, momentum=0.95, weight_decay=0.1, adamw_lr=1e-2,
                   adamw_wd=0.01, betas=(0.9, 0.999), eps=1e-8)
    res = run_ranks(_body, 2, timeout=180)
    sd, idle, n_dedicated, per_group = res[0]
    assert idle >= 12 and res[1][1] >= 12              # 2 layers x at least 4 idle experts x 3 matrices, on each rank
    assert n_dedicated == 2 * (4 + 3 * 8) and per_group == 4 + 3 * 8      # one group per decoder layer: attention + experts
    for n, p in ref.named_parameters():
        assert (sd[n].float() - p.detach()).abs().max().item() < 1e-3, n

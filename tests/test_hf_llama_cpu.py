"""A Hugging Face ``LlamaForCausalLM`` (not this package's model) through the
public path ``dedicate_params -> fully_shard -> Muon`` on 2 gloo ranks, against
the single-process oracle.  Covers what a user's own ``nn.Module`` brings that
the package's model does not: HF module names (``model.layers.N.self_attn.q_proj``),
keyword-only forward arguments, and a dict-like ``ModelOutput`` whose ``.loss``
attribute must survive the output hook."""
import pytest
import torch

from dist_utils import run_ranks

transformers = pytest.importorskip("transformers")

STEPS = 4


def _pred(name, p):
    return "proj" in name and p.ndim == 2


def _build():
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(
        hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        head_dim=16, vocab_size=256, max_position_embeddings=64, rope_theta=10000.0, use_cache=False,
        tie_word_embeddings=False, attn_implementation="sdpa",
    )
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg)


def _data(step):
    g = torch.Generator().manual_seed(500 + step)
    return torch.randint(0, 256, (4, 33), generator=g)


def _loss(model, ids):
    out = model(input_ids=ids[:, :-1], labels=ids[:, 1:])
    assert hasattr(out, "loss") and out["loss"] is out.loss      # still a ModelOutput after the hooks
    return out.loss


def _oracle():
    from oracle import muon_adamw_run

    model = _build()
    losses = muon_adamw_run(model, _pred, [_data(s) for s in range(STEPS)], _loss)
    return losses, {n: p.detach().clone() for n, p in model.named_parameters()}


def _body(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import dmuon_b200 as dmuon

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
    model = _build()
    owners = dmuon.dedicate_params(model, mesh, _pred, reshard_after_forward=False)
    for layer in model.model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1)
    per = 4 // world
    losses = []
    for s in range(STEPS):
        ids = _data(s)[rank * per : (rank + 1) * per]
        loss = _loss(model, ids)
        opt.zero_grad()
        loss.backward()
        opt.step()
        lt = loss.detach().clone()
        dist.all_reduce(lt)
        losses.append((lt / world).item())
    sd = dmuon.get_model_state_dict(model, rank0_only=False)
    return losses, sd, len(owners), sorted({int(v) for v in owners.values()})


def test_hf_llama_two_ranks_match_single_process_oracle():
    ref_losses, ref_params = _oracle()
    (losses, sd, n_dedicated, owners), other = run_ranks(_body, 2)
    assert n_dedicated == 2 * 7 and owners == [0, 1]
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (losses, ref_losses)
    assert set(sd) == set(ref_params)
    for n, p in ref_params.items():
        assert (sd[n].float() - p).abs().max().item() < 5e-4, n
    assert losses[-1] < losses[0]
    for n in sd:
        assert torch.equal(sd[n], other[1][n])

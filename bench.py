#!/usr/bin/env python
"""Headline benchmark: full training step (forward + backward + optimizer) of a
Llama-3-8B-shaped decoder under FSDP2 + dedicated Muon, bf16 compute with fp32
master weights and optimizer state, synthetic tokens, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference from baseline/_ref

Rank 0 prints one JSON line.  ``value`` is the device-timed step time in ms
(max over ranks); ``e2e`` is the same step driven through the public API with
the token batch copied from pinned host memory and the loss read back every
step.  Per-GPU work is fixed (weak scaling): micro-batch x seq tokens per GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.abspath(__file__))

MODELS = {
    # name: (d_model, layers, heads, kv_heads, head_dim, ffn, vocab, default seq, default micro-batch)
    "llama3-8b": (4096, 32, 32, 8, 128, 14336, 128256, 8192, 1),
    "llama3.2-3b": (3072, 28, 24, 8, 128, 8192, 128256, 4096, 2),
    "llama-1b": (2048, 16, 32, 8, 64, 8192, 128256, 4096, 2),
    "tiny": (256, 4, 4, 4, 64, 1024, 1024, 128, 4),
    # Pi0-style VLA (vision tower + Gemma-2B-shaped backbone + action expert); "seq" is the
    # token count per sample (3 x 256 image tokens + 48 prompt + 51 action tokens), batch 32 per GPU
    "pi0": (2048, 18, 8, 1, 256, 16384, 257152, 867, 32),
}


def pi0_host_batch(dims, mb, gen):
    import torch

    images = torch.rand(mb, 3, 3, 224, 224, generator=gen) * 2 - 1
    prompt = torch.randint(0, dims["vocab_size"], (mb, 48), generator=gen)
    state = torch.randn(mb, 32, generator=gen)
    actions = torch.randn(mb, 50, 32, generator=gen)
    return images.to(torch.bfloat16), prompt, state, actions


#: published by the reference for this model class: DMuon's full-step time over FSDP2 + AdamW's.  Llama-3.1-8B,
#: FSDP-Z2, 128 x A800, best configuration of each: MFU 49.9 % (AdamW) vs 46.2 % (DMuon) = 1.08
#: (reference docs/index.md:135; its 8 x A800 figure for the 1.5-8 B range is "4-13 % overhead", docs/index.md:26-27)
PUBLISHED_OVERHEAD_VS_ADAMW = 1.08


def mfu(args, dims, tokens_per_step, step_ms, world):
    if args.model == "pi0":
        return None
    d, L, ffn, v = dims["d_model"], dims["n_layers"], dims["ffn_hidden"], dims["vocab_size"]
    kv = dims["n_kv_heads"] * dims["head_dim"]
    q = dims["n_heads"] * dims["head_dim"]
    per_layer = d * q + 2 * d * kv + q * d + 3 * d * ffn
    params = L * per_layer + v * d                      # lm_head; the embedding lookup costs no FLOPs
    attn = 6 * L * q * dims["seq"]                      # causal: half of 12 * L * d_attn * seq per token
    flops = tokens_per_step * (6 * params + attn)
    return round(flops / (step_ms / 1e3) / (world * 2250e12), 4)


def adamw_step_ms(args, world):
    """FSDP2 + fused AdamW step time of the same model, placement and GPU count,
    measured on this pool with ``--optimizer adamw`` and recorded in
    ``baseline/adamw_step_ms.json`` (None when that cell was not measured)."""
    path = os.path.join(ROOT, "baseline", "adamw_step_ms.json")
    try:
        table = json.load(open(path))
    except (OSError, ValueError):
        return None
    impl = "hf" if (args.impl == "reference" or args.model_impl == "hf") else "own"
    key = f"{args.model}|{impl}|{args.parallelism}|{world}"
    val = table.get(key)
    return float(val["ms"]) if isinstance(val, dict) and "ms" in val else None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--model", choices=tuple(MODELS), default="llama3-8b")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--optimizer", choices=("muon", "adamw"), default="muon")
    ap.add_argument("--parallelism", default="fsdp", help="fsdp | hsdpRxS (e.g. hsdp2x4) | ddp | tpTxdpD (e.g. tp2xdp4)")
    ap.add_argument("--reshard-after-forward", action="store_true", help="drop published weights after forward")
    ap.add_argument("--ns", choices=("gram", "direct"), default="gram")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--act-ckpt", action="store_true", help="checkpoint every decoder layer")
    ap.add_argument("--momentum-dtype", choices=("fp32", "bf16"), default="fp32")
    ap.add_argument("--comm", choices=("auto", "peer", "nccl"), default="auto",
                    help="data plane for dedicated parameters (this package only)")
    ap.add_argument("--fused-publish", action="store_true",
                    help="pull each dedicated Linear weight inside its first forward GEMM (peer data plane only)")
    ap.add_argument("--attention", choices=("cudnn", "flash"), default="cudnn",
                    help="SDPA backend preference of this package's model (the reference arm uses Hugging Face's default)")
    ap.add_argument("--clip-norm", type=float, default=0.0,
                    help="global gradient-norm clip applied after backward (this package's arm, Muon only; 0 = off)")
    ap.add_argument("--plain-model-ops", action="store_true",
                    help="plain PyTorch SwiGLU / rotary embedding / cross-entropy instead of this package's fused kernels")
    ap.add_argument("--model-impl", choices=("own", "hf"), default="own",
                    help="this package's arm only: 'own' = dmuon_b200.models (fused model kernels), 'hf' = the same "
                         "Hugging Face LlamaForCausalLM the reference arm builds, so that both arms run one model "
                         "and the difference is the framework alone")
    return ap.parse_args()


def init_dist():
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs (rank 0 only)."""

    FIELDS = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, enabled: bool):
        self.enabled = enabled
        self.proc = None
        self.path = None

    def start(self):
        if not self.enabled:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if not self.enabled or self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    clk, cmax, pw = float(f[1]), float(f[2]), float(f[3])
                except ValueError:
                    continue
                if pw > 250:                      # under load
                    sm.append(clk)
                mx.append(cmax)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples_under_load": len(sm),
        }


def model_dims(args):
    d, L, h, kv, hd, ffn, vocab, seq, mb = MODELS[args.model]
    return dict(d_model=d, n_layers=L, n_heads=h, n_kv_heads=kv, head_dim=hd, ffn_hidden=ffn, vocab_size=vocab,
                seq=args.seq or seq, mb=args.micro_batch or mb)


def make_mesh(args, world):
    from torch.distributed.device_mesh import init_device_mesh

    par = args.parallelism
    args.data_ranks, args.data_rank = world, None
    if par.startswith("tp"):
        # "tp2xdp4": tensor parallel inside groups of 2 neighbouring ranks, dedicated ownership + FSDP2 over 4
        t, d = (int(x) for x in par[2:].split("xdp"))
        assert t * d == world, f"{par} needs {t * d} ranks, got {world}"
        mesh2 = init_device_mesh("cuda", (d, t), mesh_dim_names=("dp", "tp"))
        args.tp_mesh = mesh2["tp"]
        args.data_ranks, args.data_rank = d, mesh2["dp"].get_local_rank()
        return mesh2["dp"], mesh2["dp"], None
    if par.startswith("hsdp"):
        r, s = (int(x) for x in par[4:].split("x"))
        assert r * s == world, f"{par} needs {r * s} ranks, got {world}"
        mesh2 = init_device_mesh("cuda", (r, s), mesh_dim_names=("replicate", "shard"))
        return mesh2, mesh2["shard"], mesh2["replicate"]
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    return mesh, mesh, None


def _plane_name(ctx) -> str:
    rt = getattr(ctx, "peer_runtime", None)
    if rt is None:
        if getattr(ctx, "tp_exchanges", None):
            return ("nccl on the data-parallel axis; tensor-parallel shards read in place over peer memory by the "
                    "Muon prologue, update slices pulled and applied by one kernel")
        return "nccl"
    reduce = {
        "nvls": "gradients summed in the switch per layer during backward (multimem.ld_reduce), one reduced copy read by the Muon prologue kernel",
        "ce": "copy-engine gradient gather, sum fused into the Muon prologue kernel",
        "sm": "gradients read through peer mappings by the Muon prologue kernel",
    }[rt.reduce_via]
    if rt.publish_via == "nvls":
        how = ("by the update GEMM's epilogue" if rt.nvls_publish == "epilogue"
               else "by a copy kernel on the publish lane while the next Newton-Schulz batch runs")
        publish = f"weights stored to all ranks {how} (multimem.st)"
    elif rt.publish_via == "ce":
        publish = "weights pulled by the readers' copy engines"
    else:
        publish = "weights pulled by a kernel through peer mappings"
    return f"peer memory [{rt.copy_mode}]: {publish}; {reduce}"


def _pred(name, p):
    return "proj" in name and p.ndim == 2


def build_ours(args, dims, rank, world, device):
    import torch
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    sys.path.insert(0, ROOT)
    import dmuon_b200 as dmuon
    from dmuon_b200.models import llama as llama_mod
    from dmuon_b200.models.llama import LlamaConfig, LlamaModel

    llama_mod.ATTENTION_BACKEND = args.attention
    llama_mod.FUSED_OPS = not args.plain_model_ops
    if args.fused_publish:
        os.environ["DMUON_FUSED_PUBLISH"] = "1"
    if args.model == "pi0":
        return build_ours_pi0(args, dims, rank, world, device)
    if args.model_impl == "hf":
        return build_ours_hf(args, dims, rank, world, device)
    cfg = LlamaConfig(
        vocab_size=dims["vocab_size"], d_model=dims["d_model"], n_layers=dims["n_layers"], n_heads=dims["n_heads"],
        n_kv_heads=dims["n_kv_heads"], head_dim=dims["head_dim"], ffn_hidden=dims["ffn_hidden"], rope_theta=500000.0,
    )
    torch.manual_seed(42)
    with torch.device(device):
        model = LlamaModel(cfg)
    mesh_all, shard_mesh, rep_mesh = make_mesh(args, world)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    fsdp_mesh = mesh_all
    if getattr(args, "tp_mesh", None) is not None:
        apply_tp(model.layers, args.tp_mesh)
    if args.act_ckpt:
        from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper

        for i, layer in enumerate(model.layers):
            model.layers[i] = checkpoint_wrapper(layer)
    if args.optimizer == "muon":
        policy = None
        if args.momentum_dtype == "bf16":
            policy = {"defaults": {"param_dtype": "bf16", "optim_dtype": "bf16"}}
        if args.parallelism == "ddp":
            model.to(torch.bfloat16)
            dmuon.dedicate_params_ddp(model, shard_mesh, _pred, compute_dtype=torch.bfloat16, param_policy=policy)
            dmuon.replicate(model, shard_mesh)
        else:
            dmuon.dedicate_params(
                model, shard_mesh, _pred, compute_dtype=None if policy else torch.bfloat16,
                reshard_after_forward=args.reshard_after_forward, replicate_mesh=rep_mesh, param_policy=policy,
                comm_backend=args.comm,
            )
            for layer in model.layers:
                fully_shard(layer, mesh=fsdp_mesh, mp_policy=mp)
            fully_shard(model, mesh=fsdp_mesh, mp_policy=mp)
        opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1,
                         ns_backend=dmuon.NewtonSchulz(backend=args.ns))
    else:
        for layer in model.layers:
            fully_shard(layer, mesh=fsdp_mesh, mp_policy=mp)
        fully_shard(model, mesh=fsdp_mesh, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=True)

    clip = float(args.clip_norm)

    def fwd_bwd(b):
        loss = model(b[:, :-1], labels=b[:, 1:])
        loss.backward()
        if clip > 0 and args.optimizer == "muon":
            dmuon.clip_grad_norm_(opt, clip)
        return loss

    def launches():
        from dmuon_b200.ops import multi_tensor as MT

        return MT.launch_count()

    ctx = getattr(model, "_dedicated_comm_ctx", None)
    args.comm_used = _plane_name(ctx)
    return fwd_bwd, opt, launches


def hf_llama(dims, device, act_ckpt):
    """The Hugging Face model both arms can run: built exactly like the
    reference's own LLM benchmark builds it (benchmarks/bench_llm.py:38-83)."""
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    config = LlamaConfig(
        hidden_size=dims["d_model"], intermediate_size=dims["ffn_hidden"], num_hidden_layers=dims["n_layers"],
        num_attention_heads=dims["n_heads"], num_key_value_heads=dims["n_kv_heads"], head_dim=dims["head_dim"],
        vocab_size=dims["vocab_size"], max_position_embeddings=dims["seq"], rope_theta=500000.0, use_cache=False,
        tie_word_embeddings=False, attn_implementation="sdpa",
    )
    torch.manual_seed(42)
    with torch.device(device):
        model = LlamaForCausalLM(config)
    if act_ckpt:
        model.gradient_checkpointing_enable()
    return model


TP_PLAN_NAMES = {
    "self_attn.q_proj": "col", "self_attn.k_proj": "col", "self_attn.v_proj": "col", "self_attn.o_proj": "row",
    "mlp.gate_proj": "col", "mlp.up_proj": "col", "mlp.down_proj": "row",
}


def apply_tp(layers, tp_mesh):
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    plan = {k: (ColwiseParallel() if v == "col" else RowwiseParallel()) for k, v in TP_PLAN_NAMES.items()}
    for layer in layers:
        parallelize_module(layer, tp_mesh, plan)


def build_ours_hf(args, dims, rank, world, device):
    """This package's framework around the Hugging Face model of the reference
    arm (same module code, same SDPA default): the framework-only comparison."""
    import torch
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon

    model = hf_llama(dims, device, args.act_ckpt)
    mesh_all, shard_mesh, rep_mesh = make_mesh(args, world)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    if getattr(args, "tp_mesh", None) is not None:
        apply_tp(model.model.layers, args.tp_mesh)
    if args.optimizer == "muon":
        if args.parallelism == "ddp":
            model.to(torch.bfloat16)
            dmuon.dedicate_params_ddp(model, shard_mesh, _pred, compute_dtype=torch.bfloat16)
            dmuon.replicate(model, shard_mesh)
        else:
            dmuon.dedicate_params(model, shard_mesh, _pred, compute_dtype=torch.bfloat16,
                                  reshard_after_forward=args.reshard_after_forward, replicate_mesh=rep_mesh,
                                  comm_backend=args.comm)
            for layer in model.model.layers:
                fully_shard(layer, mesh=mesh_all, mp_policy=mp)
            fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1,
                         ns_backend=dmuon.NewtonSchulz(backend=args.ns))
    else:
        for layer in model.model.layers:
            fully_shard(layer, mesh=mesh_all, mp_policy=mp)
        fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=True)
    clip = float(args.clip_norm)

    def fwd_bwd(b):
        out = model(input_ids=b[:, :-1], labels=b[:, 1:])
        out.loss.backward()
        if clip > 0 and args.optimizer == "muon":
            dmuon.clip_grad_norm_(opt, clip)
        return out.loss

    def launches():
        from dmuon_b200.ops import multi_tensor as MT

        return MT.launch_count()

    args.comm_used = _plane_name(getattr(model, "_dedicated_comm_ctx", None))
    return fwd_bwd, opt, launches


def build_ours_pi0(args, dims, rank, world, device):
    import torch
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon_b200 as dmuon
    from dmuon_b200.models.pi0 import Pi0Config, Pi0Model

    cfg = Pi0Config()
    torch.manual_seed(42)
    with torch.device(device):
        model = Pi0Model(cfg)
    mesh_all, shard_mesh, rep_mesh = make_mesh(args, world)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    blocks = list(model.vision.blocks) + list(model.layers)
    if args.optimizer == "muon":
        dmuon.dedicate_params(model, shard_mesh, _pred, compute_dtype=torch.bfloat16,
                              reshard_after_forward=args.reshard_after_forward, replicate_mesh=rep_mesh,
                              comm_backend=args.comm)
        for blk in blocks:
            fully_shard(blk, mesh=mesh_all, mp_policy=mp)
        fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1,
                         ns_backend=dmuon.NewtonSchulz(backend=args.ns))
    else:
        for blk in blocks:
            fully_shard(blk, mesh=mesh_all, mp_policy=mp)
        fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=True)

    def fwd_bwd(images, prompt, state, actions):
        loss = model(images, prompt, state, actions)
        loss.backward()
        return loss

    def launches():
        from dmuon_b200.ops import multi_tensor as MT

        return MT.launch_count()

    ctx = getattr(model, "_dedicated_comm_ctx", None)
    args.comm_used = _plane_name(ctx)
    return fwd_bwd, opt, launches


def build_reference(args, dims, rank, world, device):
    if args.model == "pi0":
        raise RuntimeError("the reference ships no vision-language-action model to run this configuration with")
    """The unmodified reference installed under baseline/_ref, driven through
    its public API the way its own LLM benchmark does (Hugging Face Llama,
    dedicate_params -> fully_shard -> Muon)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dmuon")):
        raise RuntimeError("baseline/_ref/dmuon is missing (reference not installed)")
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, ref_dir)
    import torch
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import dmuon  # the reference package

    assert os.path.abspath(dmuon.__file__).startswith(ref_dir), dmuon.__file__
    model = hf_llama(dims, device, args.act_ckpt)
    mesh_all, shard_mesh, rep_mesh = make_mesh(args, world)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    if getattr(args, "tp_mesh", None) is not None:
        # stock DTensor tensor parallelism on the stock model; the reference detects the sharded
        # matrices itself (dmuon/_core/tp.py:41-77) and takes its gather -> NS -> scatter route
        apply_tp(model.model.layers, args.tp_mesh)
    clip = float(args.clip_norm)
    if args.optimizer == "muon":
        dmuon.dedicate_params(model, shard_mesh, _pred, compute_dtype=torch.bfloat16,
                              reshard_after_forward=args.reshard_after_forward, replicate_mesh=rep_mesh)
        for layer in model.model.layers:
            fully_shard(layer, mesh=mesh_all, mp_policy=mp)
        fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = dmuon.Muon(model, lr=0.02, ns_steps=5, adamw_lr=1e-3, weight_decay=0.1)
    else:
        for layer in model.model.layers:
            fully_shard(layer, mesh=mesh_all, mp_policy=mp)
        fully_shard(model, mesh=mesh_all, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01, fused=True)

    def fwd_bwd(b):
        out = model(input_ids=b[:, :-1], labels=b[:, 1:])
        out.loss.backward()
        if clip > 0 and args.optimizer == "muon":
            dmuon.clip_grad_norm_(opt, clip)
        return out.loss

    return fwd_bwd, opt, (lambda: 0)


def run(args):
    import torch
    import torch.distributed as dist

    rank, world, local = init_dist()
    device = torch.device("cuda", local)
    dims = model_dims(args)
    build = build_ours if args.impl == "ours" else build_reference
    fwd_bwd, opt, launches = build(args, dims, rank, world, device)
    mb, seq, vocab = dims["mb"], dims["seq"], dims["vocab_size"]

    # ranks of one tensor-parallel group see the same batch
    data_rank = rank if getattr(args, "data_rank", None) is None else args.data_rank
    data_ranks = getattr(args, "data_ranks", world)
    gen = torch.Generator().manual_seed(1234 + data_rank)
    n_batches = 4
    if args.model == "pi0":
        host = [tuple(t.pin_memory() for t in pi0_host_batch(dims, mb, gen)) for _ in range(n_batches)]
    else:
        host = [(torch.randint(0, vocab, (mb, seq + 1), generator=gen).pin_memory(),) for _ in range(n_batches)]
    dev_batches = [tuple(t.to(device) for t in h) for h in host]
    h2d_bytes = sum(t.numel() * t.element_size() for t in host[0])

    def step_device(i):
        opt.zero_grad()
        return fwd_bwd(*dev_batches[i % n_batches])

    def step_e2e(i):
        b = tuple(t.to(device, non_blocking=True) for t in host[i % n_batches])
        opt.zero_grad()
        loss = fwd_bwd(*b)
        opt.step()
        return float(loss.item())          # device -> host read of the step's result

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step_device(i)
        opt.step()
    sync()

    sampler = ClockSampler(rank == 0)
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    l0 = launches()
    sync()
    ev[0].record()
    for i in range(args.steps):
        loss = step_device(i)
        ev[2 * i + 1].record()
        opt.step()
        ev[2 * i + 2].record()
    sync()
    total_ms = ev[0].elapsed_time(ev[2 * args.steps])
    opt_ms = sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)) / args.steps
    l1 = launches()
    last_loss = float(loss.item())

    e2e_ms = None
    if not args.no_e2e:
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            last_loss = step_e2e(i)
        b.record()
        sync()
        e2e_ms = a.elapsed_time(b) / args.steps
    clocks = sampler.stop()

    t = torch.tensor([total_ms / args.steps, opt_ms, e2e_ms or 0.0], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, opt_ms, e2e_max = (float(x) for x in t.tolist())
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=device)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    # every device-side wait of this package is bounded and records in a status word when it ran out; a run in which
    # that happened on any rank did not do the work it claims to have timed
    status_code = 0
    try:
        status = torch.zeros(1, dtype=torch.int32, device=device)
        if args.impl == "ours":
            from dmuon_b200.ops import gemm as _gemm

            status.copy_(_gemm.status_buffer(device)[:1])
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
        status_code = int(status.item())
    except Exception as exc:          # the check itself must not cost a measurement
        print(f"bench.py: could not read the kernel status word ({exc})", file=sys.stderr)
        status_code = -1
    if status_code > 0:
        raise RuntimeError(f"a kernel wait ran out during the benchmark (status code {status_code}): no valid timing")
    tokens = mb * seq * data_ranks
    if rank == 0:
        adamw_ms = adamw_step_ms(args, world) if args.optimizer == "muon" else None
        vs_adamw = round(step_ms / adamw_ms, 4) if adamw_ms else None
        out = {
            "metric": "train_step_ms",
            "value": round(step_ms, 3),
            "unit": "ms/step",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(step_ms, 3),
            "higher_is_better": False,
            "scaling": "weak",
            # overhead over FSDP2 + AdamW divided by the overhead the reference publishes (1.08): below 1 means
            # Muon costs less on top of AdamW here than the reference reports for itself; null when the AdamW
            # step of this configuration has not been measured on this pool
            "vs_baseline": round(vs_adamw / PUBLISHED_OVERHEAD_VS_ADAMW, 4) if vs_adamw else None,
            "vs_adamw": {"ratio": vs_adamw, "adamw_ms": adamw_ms, "published_reference_ratio": PUBLISHED_OVERHEAD_VS_ADAMW}
            if vs_adamw else None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights N(0, 0.02)",
            "impl": args.impl,
            "tokens_per_s": round(tokens / (step_ms / 1e3), 1),
            # model FLOP utilisation: 6 FLOPs per parameter and token plus causal attention, against the
            # nominal dense bf16 peak of a B200 (2250 TFLOP/s per GPU); null for the vision-language model
            "mfu": mfu(args, dims, tokens, step_ms, world),
            "optimizer_step_ms": round(opt_ms, 3),
            "fwd_bwd_ms": round(step_ms - opt_ms, 3),
            "loss": last_loss,
            "peak_mem_gib": round(float(peak.item()), 2),
            "gpu_launches": int(l1 - l0),
            "kernel_status": status_code,
            "clocks": clocks,
            "config": {
                "model": args.model,
                "model_impl": ("Hugging Face LlamaForCausalLM" if (args.impl == "reference" or args.model_impl == "hf")
                               else "dmuon_b200.models"),
                "optimizer": args.optimizer,
                "global_batch": mb * data_ranks,
                "micro_batch_per_gpu": mb,
                "seq_len": seq,
                "parallelism": (args.parallelism if args.parallelism != "fsdp" else f"fsdp{world}")
                + ("-z3" if args.reshard_after_forward else "-z2"),
                "newton_schulz": args.ns,
                "dedicated_data_plane": getattr(args, "comm_used", "nccl")
                + (" + publish fused into forward GEMMs" if args.fused_publish else ""),
                "attention": (args.attention + " SDPA backend" if (args.impl == "ours" and args.model_impl == "own")
                              else "Hugging Face sdpa default"),
                "model_ops": ("n/a" if (args.impl != "ours" or args.model_impl == "hf") else
                              "plain PyTorch" if args.plain_model_ops else "fused SwiGLU / RoPE / linear-cross-entropy kernels"),
                "activation_checkpointing": bool(args.act_ckpt),
                "clip_norm": (float(args.clip_norm) if float(args.clip_norm) > 0 else None),
                "l2": "per-step working set (weights + activations, tens of GB) is far larger than the 126 MB L2",
            },
        }
        if e2e_ms is not None:
            out["e2e"] = {
                "value": round(e2e_max, 3),
                "unit": "ms/step",
                "tokens_per_s": round(tokens / (e2e_max / 1e3), 1),
                "h2d_bytes_per_step": int(h2d_bytes),
                "d2h_bytes_per_step": 4,
            }
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        try:
            run(args)
        except Exception as exc:  # the reference could not run here: say why, exit 0
            import traceback

            traceback.print_exc(file=sys.stderr)
            if int(os.environ.get("RANK", "0")) == 0:
                why = f"{type(exc).__name__}: {str(exc).splitlines()[0] if str(exc) else ''}"[:300]
                print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
            sys.exit(0)
    else:
        run(args)


if __name__ == "__main__":
    main()

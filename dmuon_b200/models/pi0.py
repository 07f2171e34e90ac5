"""Pi0-style vision-language-action model for flow-matching training.

Three towers, shaped like the published Pi0 recipe:

vision   SigLIP-So400m-shaped ViT: patch 14 on 224x224 RGB (256 tokens per
         image), 27 blocks of width 1152, 16 heads, MLP 4304
backbone Gemma-2B-shaped decoder: 18 layers, width 2048, 8 query heads / 1 KV
         head of dimension 256, GeGLU FFN 16384, vocabulary 257152; reads the
         projected image tokens followed by the prompt tokens (bidirectional
         prefix attention)
expert   action expert: 18 layers of width 1024 with the backbone's head layout
         and FFN 4096; its tokens (robot state + a 50 x 32 noisy action chunk
         with the flow time embedded) attend to the backbone's keys/values of
         the same layer and to themselves

Loss: flow matching.  With ``t ~ Beta(1.5, 1)`` scaled to [0.001, 1],
``x_t = t * noise + (1 - t) * actions`` and the target velocity
``noise - actions``, the model regresses the velocity with an MSE.

Every 2-D matrix inside a block is called ``*_proj`` so the predicate
``"proj" in name and p.ndim == 2`` selects them; blocks are ``blocks.N`` /
``layers.N`` so the default hook boundary and owner packing apply.  The
reference has no model code (its VLA numbers come from external trainers,
README.md:102-108).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import model_ops
from . import llama as _llama
from .llama import RMSNorm, RopeTables, apply_rope, rope_tables


@dataclass
class Pi0Config:
    image_size: int = 224
    patch: int = 14
    images_per_sample: int = 3
    vit_width: int = 1152
    vit_layers: int = 27
    vit_heads: int = 16
    vit_mlp: int = 4304
    width: int = 2048
    layers: int = 18
    heads: int = 8
    kv_heads: int = 1
    head_dim: int = 256
    ffn: int = 16384
    vocab_size: int = 257152
    prompt_len: int = 48
    expert_width: int = 1024
    expert_ffn: int = 4096
    state_dim: int = 32
    action_dim: int = 32
    action_horizon: int = 50
    rope_theta: float = 10000.0
    init_std: float = 0.02

    @staticmethod
    def tiny(**kw) -> "Pi0Config":
        base = dict(image_size=28, patch=14, images_per_sample=2, vit_width=64, vit_layers=2, vit_heads=4, vit_mlp=144,
                    width=128, layers=2, heads=4, kv_heads=1, head_dim=32, ffn=256, vocab_size=512, prompt_len=6,
                    expert_width=64, expert_ffn=128, state_dim=8, action_dim=8, action_horizon=5)
        base.update(kw)
        return Pi0Config(**base)

    @property
    def tokens_per_image(self) -> int:
        return (self.image_size // self.patch) ** 2


def _sdpa(q, k, v, mask=None, gqa=False):
    if q.is_cuda and mask is None and q.dtype in (torch.bfloat16, torch.float16):
        from torch.nn.attention import SDPBackend, sdpa_kernel

        order = [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]
        with sdpa_kernel(order, set_priority=True):
            return F.scaled_dot_product_attention(q, k, v, enable_gqa=gqa)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=gqa)


class ViTBlock(nn.Module):
    def __init__(self, c: Pi0Config):
        super().__init__()
        w = c.vit_width
        self.heads = c.vit_heads
        self.norm1 = nn.LayerNorm(w)
        self.q_proj = nn.Linear(w, w)
        self.k_proj = nn.Linear(w, w)
        self.v_proj = nn.Linear(w, w)
        self.o_proj = nn.Linear(w, w)
        self.norm2 = nn.LayerNorm(w)
        self.up_proj = nn.Linear(w, c.vit_mlp)
        self.down_proj = nn.Linear(c.vit_mlp, w)

    def forward(self, x):
        b, s, w = x.shape
        h = self.norm1(x)
        shp = (b, s, self.heads, w // self.heads)
        q, k, v = (f(h).view(shp).transpose(1, 2) for f in (self.q_proj, self.k_proj, self.v_proj))
        x = x + self.o_proj(_sdpa(q, k, v).transpose(1, 2).reshape(b, s, w))
        return x + self.down_proj(F.gelu(self.up_proj(self.norm2(x)), approximate="tanh"))


class VisionTower(nn.Module):
    def __init__(self, c: Pi0Config):
        super().__init__()
        self.patch_embed = nn.Conv2d(3, c.vit_width, c.patch, stride=c.patch)
        self.pos_embed = nn.Parameter(torch.zeros(1, c.tokens_per_image, c.vit_width))
        self.blocks = nn.ModuleList(ViTBlock(c) for _ in range(c.vit_layers))
        self.norm = nn.LayerNorm(c.vit_width)
        self.out_proj = nn.Linear(c.vit_width, c.width)

    def forward(self, pixels):           # [N, 3, H, W] -> [N, tokens, width]
        x = self.patch_embed(pixels).flatten(2).transpose(1, 2) + self.pos_embed.to(pixels.dtype)
        for blk in self.blocks:
            x = blk(x)
        return self.out_proj(self.norm(x))


class GemmaAttnMLP(nn.Module):
    """One decoder layer body with the backbone's head layout; used by both the
    backbone (width 2048) and the expert (width 1024)."""

    def __init__(self, width: int, ffn: int, c: Pi0Config):
        super().__init__()
        self.h, self.kv, self.hd = c.heads, c.kv_heads, c.head_dim
        self.input_layernorm = RMSNorm(width, 1e-6)
        self.q_proj = nn.Linear(width, c.heads * c.head_dim, bias=False)
        self.k_proj = nn.Linear(width, c.kv_heads * c.head_dim, bias=False)
        self.v_proj = nn.Linear(width, c.kv_heads * c.head_dim, bias=False)
        self.o_proj = nn.Linear(c.heads * c.head_dim, width, bias=False)
        self.post_attention_layernorm = RMSNorm(width, 1e-6)
        self.gate_proj = nn.Linear(width, ffn, bias=False)
        self.up_proj = nn.Linear(width, ffn, bias=False)
        self.down_proj = nn.Linear(ffn, width, bias=False)

    def qkv(self, x, rope: RopeTables):
        b, s, _ = x.shape
        h = self.input_layernorm(x)
        q, k = self.q_proj(h), self.k_proj(h)
        v = self.v_proj(h).view(b, s, self.kv, self.hd).transpose(1, 2)
        if _llama.FUSED_OPS and q.is_cuda:
            q, k = model_ops.rope_qk_(q, k, rope.cos, rope.sin, self.hd)
            q = q.view(b, s, self.h, self.hd).transpose(1, 2)
            k = k.view(b, s, self.kv, self.hd).transpose(1, 2)
        else:
            cos, sin = rope.as_dtype(q.dtype)
            q = apply_rope(q.view(b, s, self.h, self.hd).transpose(1, 2), cos, sin)
            k = apply_rope(k.view(b, s, self.kv, self.hd).transpose(1, 2), cos, sin)
        return q, k, v

    def finish(self, x, attn):
        b, s, _ = x.shape
        x = x + self.o_proj(attn.transpose(1, 2).reshape(b, s, self.h * self.hd))
        h = self.post_attention_layernorm(x)
        g, u = self.gate_proj(h), self.up_proj(h)
        return x + self.down_proj(model_ops.geglu(g, u) if _llama.FUSED_OPS else F.gelu(g, approximate="tanh") * u)


class JointLayer(nn.Module):
    """Backbone layer + expert layer that share one attention: prefix tokens
    attend to the prefix, action tokens attend to prefix and action tokens."""

    def __init__(self, c: Pi0Config, last: bool = False):
        super().__init__()
        self.last = last
        self.backbone = GemmaAttnMLP(c.width, c.ffn, c)
        self.expert = GemmaAttnMLP(c.expert_width, c.expert_ffn, c)

    def forward(self, xp, xa, rope_p, rope_a):
        qp, kp, vp = self.backbone.qkv(xp, rope_p)
        qa, ka, va = self.expert.qkv(xa, rope_a)
        gqa = self.backbone.kv != self.backbone.h
        if not self.last:
            # the prefix stream of the last layer feeds nothing: only its keys and values are used
            xp = self.backbone.finish(xp, _sdpa(qp, kp, vp, gqa=gqa))
        k_all, v_all = torch.cat((kp, ka), dim=2), torch.cat((vp, va), dim=2)
        xa = self.expert.finish(xa, _sdpa(qa, k_all, v_all, gqa=gqa))
        return xp, xa


def _time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freq = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    ang = t.float()[:, None] * freq[None] * 1000.0
    return torch.cat((ang.sin(), ang.cos()), dim=-1)


class Pi0Model(nn.Module):
    def __init__(self, c: Pi0Config):
        super().__init__()
        self.cfg = c
        self.vision = VisionTower(c)
        self.embed_tokens = nn.Embedding(c.vocab_size, c.width)
        self.layers = nn.ModuleList(JointLayer(c, last=(i == c.layers - 1)) for i in range(c.layers))
        self.state_in = nn.Linear(c.state_dim, c.expert_width)
        self.action_in = nn.Linear(c.action_dim, c.expert_width)
        self.time_mlp_in = nn.Linear(2 * c.expert_width, c.expert_width)
        self.time_mlp_out = nn.Linear(c.expert_width, c.expert_width)
        self.expert_norm = RMSNorm(c.expert_width, 1e-6)
        self.action_out = nn.Linear(c.expert_width, c.action_dim)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding, nn.Conv2d)):
                m.weight.normal_(0.0, self.cfg.init_std)
                if getattr(m, "bias", None) is not None:
                    m.bias.zero_()
        self.vision.pos_embed.normal_(0.0, self.cfg.init_std)

    def velocity(self, images, prompt, state, noisy_actions, t):
        """images [B, I, 3, H, W], prompt [B, P] ids, state [B, state_dim],
        noisy_actions [B, horizon, action_dim], t [B] -> velocity [B, horizon, action_dim]."""
        c = self.cfg
        b = images.shape[0]
        dtype = self.embed_tokens.weight.dtype if self.embed_tokens.weight.numel() else images.dtype
        img_tok = self.vision(images.flatten(0, 1).to(dtype)).view(b, -1, c.width)
        xp = torch.cat((img_tok, self.embed_tokens(prompt).to(img_tok.dtype) * math.sqrt(c.width)), dim=1)
        a_tok = self.action_in(noisy_actions.to(xp.dtype))
        temb = _time_embedding(t, c.expert_width).to(xp.dtype)[:, None].expand(-1, a_tok.shape[1], -1)
        a_tok = self.time_mlp_out(F.silu(self.time_mlp_in(torch.cat((a_tok, temb), dim=-1))))
        xa = torch.cat((self.state_in(state.to(xp.dtype))[:, None], a_tok), dim=1)
        sp, sa = xp.shape[1], xa.shape[1]
        cos, sin = rope_tables(sp + sa, c.head_dim, c.rope_theta, xp.device)
        rope_p, rope_a = RopeTables(cos[:sp], sin[:sp]), RopeTables(cos[sp:], sin[sp:])
        for layer in self.layers:
            xp, xa = layer(xp, xa, rope_p, rope_a)
        return self.action_out(self.expert_norm(xa[:, 1:]))

    def forward(self, images, prompt, state, actions, noise=None, t=None):
        """Flow-matching loss of one batch."""
        b = actions.shape[0]
        if noise is None:
            noise = torch.randn_like(actions)
        if t is None:
            t = sample_flow_time(b, actions.device)
        tt = t.to(actions.dtype)[:, None, None]
        x_t = tt * noise + (1 - tt) * actions
        v = self.velocity(images, prompt, state, x_t, t)
        return F.mse_loss(v.float(), (noise - actions).float())


def sample_flow_time(batch: int, device) -> torch.Tensor:
    """t ~ Beta(1.5, 1), scaled into [0.001, 1]."""
    beta = torch.distributions.Beta(torch.tensor(1.5), torch.tensor(1.0))
    return (beta.sample((batch,)) * 0.999 + 0.001).to(device)


def synthetic_batch(c: Pi0Config, batch: int, device, generator=None):
    """Random inputs of the training shapes: pixels uniform in [-1, 1], prompt
    ids uniform over the vocabulary, state and actions N(0, 1)."""
    g = generator
    images = torch.rand(batch, c.images_per_sample, 3, c.image_size, c.image_size, generator=g) * 2 - 1
    prompt = torch.randint(0, c.vocab_size, (batch, c.prompt_len), generator=g)
    state = torch.randn(batch, c.state_dim, generator=g)
    actions = torch.randn(batch, c.action_horizon, c.action_dim, generator=g)
    return tuple(x.to(device) for x in (images, prompt, state, actions))

"""Llama-style decoder (pre-RMSNorm, RoPE, grouped-query attention, SwiGLU).

The reference ships no models (its benchmarks build Hugging Face Llama/Qwen
from configs, benchmarks/bench_llm.py:38-83); this one exists so the framework
can be trained, tested and benchmarked without external packages.  Parameter
names follow the Hugging Face layout (``layers.N.self_attn.q_proj.weight``,
``layers.N.mlp.down_proj.weight``, ...) so the usual predicate
``"proj" in name and p.ndim == 2`` selects exactly the seven matrices of every
layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import model_ops

#: Use the fused kernels (rotary embedding in place on the projection outputs,
#: one-pass SwiGLU, linear + cross-entropy with in-chunk gradients) for CUDA
#: tensors.  False keeps the plain PyTorch formulation everywhere.
FUSED_OPS = True


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: Optional[int] = None
    ffn_hidden: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = False
    init_std: float = 0.02
    loss_chunk: int = 4096          # tokens per cross-entropy chunk (0 = one shot)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.d_model // self.n_heads

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(128256, 4096, 32, 32, 8, 128, 14336, 500000.0, **kw)

    @staticmethod
    def llama32_3b(**kw) -> "LlamaConfig":
        return LlamaConfig(128256, 3072, 28, 24, 8, 128, 8192, 500000.0, **kw)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        """4 layers, width 256, 4 heads of 64, FFN 1024, vocab 1024, tied embeddings."""
        base = dict(vocab_size=1024, d_model=256, n_layers=4, n_heads=4, n_kv_heads=4, head_dim=64,
                    ffn_hidden=1024, rope_theta=10000.0, tie_embeddings=True)
        base.update(kw)
        return LlamaConfig(**base)

    def param_count(self) -> int:
        per_layer = (
            self.d_model * self.head_dim * (self.n_heads * 2 + self.n_kv_heads * 2)
            + 3 * self.d_model * self.ffn_hidden
            + 2 * self.d_model
        )
        emb = self.vocab_size * self.d_model * (1 if self.tie_embeddings else 2)
        return self.n_layers * per_layer + emb + self.d_model

    def flops_per_token(self, seq_len: int) -> float:
        """Training flops per token (forward + backward), attention included."""
        matmul = 6 * (self.param_count() - self.vocab_size * self.d_model * (0 if self.tie_embeddings else 1))
        attn = 12 * self.n_layers * self.n_heads * self.head_dim * seq_len / 2
        return float(matmul + attn)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.eps)


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


class RopeTables:
    """fp32 position tables handed from the model to its layers.  A plain
    object rather than tensors in the argument list: wrappers that cast
    floating-point forward inputs to the compute dtype (FSDP2 mixed precision)
    leave it alone, so the rotation keeps fp32 angles."""

    def __init__(self, cos: torch.Tensor, sin: torch.Tensor):
        self.cos, self.sin = cos, sin
        self._cast: dict = {}

    def as_dtype(self, dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
        if dtype == self.cos.dtype:
            return self.cos, self.sin
        if dtype not in self._cast:
            self._cast[dtype] = (self.cos.to(dtype), self.sin.to(dtype))
        return self._cast[dtype]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [B, H, S, D]; rotate-half convention
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, None], sin[None, None]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


#: "cudnn" prefers the cuDNN fused attention (the Blackwell-native library
#: kernel, about 4x faster than the flash-attention-2 path on a B200 at
#: sequence length 8192), "flash" keeps PyTorch's default order.
ATTENTION_BACKEND = "cudnn"


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gqa: bool) -> torch.Tensor:
    if q.is_cuda and ATTENTION_BACKEND == "cudnn" and q.dtype in (torch.bfloat16, torch.float16):
        from torch.nn.attention import SDPBackend, sdpa_kernel

        order = [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]
        with sdpa_kernel(order, set_priority=True):
            return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gqa)
    return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gqa)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_heads, self.n_kv, self.hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        self.q_proj = nn.Linear(cfg.d_model, cfg.n_heads * cfg.head_dim, bias=False)
        self.k_proj = nn.Linear(cfg.d_model, cfg.n_kv_heads * cfg.head_dim, bias=False)
        self.v_proj = nn.Linear(cfg.d_model, cfg.n_kv_heads * cfg.head_dim, bias=False)
        self.o_proj = nn.Linear(cfg.n_heads * cfg.head_dim, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor, rope: RopeTables) -> torch.Tensor:
        b, s, _ = x.shape
        q, k = self.q_proj(x), self.k_proj(x)
        v = self.v_proj(x).view(b, s, -1, self.hd).transpose(1, 2)   # -1: local heads under tensor parallelism
        if FUSED_OPS and q.is_cuda:
            # rotated in place, in the [b, s, h, d] layout the projections wrote
            q, k = model_ops.rope_qk_(q, k, rope.cos, rope.sin, self.hd)
            q = q.view(b, s, -1, self.hd).transpose(1, 2)
            k = k.view(b, s, -1, self.hd).transpose(1, 2)
        else:
            cos, sin = rope.as_dtype(q.dtype)
            q = apply_rope(q.view(b, s, -1, self.hd).transpose(1, 2), cos, sin)
            k = apply_rope(k.view(b, s, -1, self.hd).transpose(1, 2), cos, sin)
        o = causal_attention(q, k, v, self.n_kv != self.n_heads)
        return self.o_proj(o.transpose(1, 2).reshape(b, s, -1))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.d_model, cfg.ffn_hidden, bias=False)
        self.up_proj = nn.Linear(cfg.d_model, cfg.ffn_hidden, bias=False)
        self.down_proj = nn.Linear(cfg.ffn_hidden, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g, u = self.gate_proj(x), self.up_proj(x)
        return self.down_proj(model_ops.swiglu(g, u) if FUSED_OPS else F.silu(g) * u)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.mlp = MLP(cfg)

    def forward(self, x: torch.Tensor, rope: RopeTables) -> torch.Tensor:
        x = x + self.self_attn(self.input_layernorm(x), rope)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaModel(nn.Module):
    """``forward(input_ids, labels=None)`` returns logits, or the mean
    next-token cross-entropy when ``labels`` is given (``labels[t]`` is the
    target for position ``t``; the caller shifts)."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(DecoderLayer(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        std = self.cfg.init_std
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                m.weight.normal_(0.0, std)
            elif isinstance(m, RMSNorm):
                m.weight.fill_(1.0)

    def hidden(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = self.embed_tokens(input_ids)
        rope = RopeTables(*rope_tables(input_ids.shape[1], self.cfg.head_dim, self.cfg.rope_theta, x.device))
        for layer in self.layers:
            x = layer(x, rope)
        return self.norm(x)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = self.hidden(input_ids)
        if labels is None:
            return self.lm_head(h)
        return self.loss_from_hidden(h, labels)

    def loss_from_hidden(self, h: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        h2 = h.reshape(-1, h.shape[-1])
        y = labels.reshape(-1)
        chunk = self.cfg.loss_chunk
        if FUSED_OPS and h2.is_cuda and model_ops.kernels_apply(h2) and self.lm_head.weight.dtype == h2.dtype:
            return model_ops.linear_cross_entropy(h2, self.lm_head.weight, y, chunk)
        if chunk <= 0 or h2.shape[0] <= chunk:
            return F.cross_entropy(self.lm_head(h2).float(), y)
        total = h2.new_zeros((), dtype=torch.float32)
        for lo in range(0, h2.shape[0], chunk):
            total = total + _ce_chunk(self.lm_head.weight, h2[lo : lo + chunk], y[lo : lo + chunk])
        return total / h2.shape[0]


def _ce_chunk(weight: torch.Tensor, h: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Summed cross-entropy of one token chunk; checkpointed so the fp32 logits
    of a chunk are alive only while that chunk is differentiated."""
    from torch.utils.checkpoint import checkpoint

    def fn(w, hh, yy):
        return F.cross_entropy(F.linear(hh, w).float(), yy, reduction="sum")

    if torch.is_grad_enabled():
        return checkpoint(fn, weight, h, y, use_reentrant=False)
    return fn(weight, h, y)

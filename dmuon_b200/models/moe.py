"""Mixture-of-experts decoder: the Llama-style block with its MLP replaced by a
routed set of SwiGLU experts (top-k token choice, softmax gates renormalised
over the chosen experts, optional load-balancing term).

It exists to exercise what a mixture of experts asks of dedicated ownership
(the reference names MoE as a use of custom hook boundaries,
docs/guides/custom-hook-boundaries.md:125-164, and ships no model):

* every expert's ``gate_proj`` / ``up_proj`` / ``down_proj`` is a Muon matrix, so
  one layer holds ``3 * n_experts + 4`` dedicated matrices of three shapes -- many
  small same-shape matrices, which is what the shape-batched Newton-Schulz path
  is for;
* the hook boundary is the decoder layer (``layers.N``): the router runs inside
  it on every rank, whichever experts the rank's tokens choose;
* an expert that received no token on a rank has no gradient there.  Experts are
  made of dedicated matrices only, so ``DMUON_ZERO_FILL_MISSING_GRADS=1`` (zeros
  for what is missing) keeps every rank's reduce identical; the router is an
  ordinary FSDP2 parameter and always has a gradient.

Tokens are dispatched with index operations (no capacity limit, no token
dropping), which is exact and good enough for tests and small runs; a fused
grouped GEMM would be the next step for a production MoE.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .llama import Attention, LlamaConfig, RMSNorm, RopeTables, rope_tables


@dataclass
class MoEConfig(LlamaConfig):
    n_experts: int = 8
    top_k: int = 2
    expert_hidden: int = 0            # 0: ffn_hidden // top_k (keeps the active width of the dense model)
    balance_coef: float = 0.0         # weight of the load-balancing term added to the loss

    def __post_init__(self):
        super().__post_init__()
        if self.expert_hidden <= 0:
            self.expert_hidden = max(8, self.ffn_hidden // max(1, self.top_k))
        if not 1 <= self.top_k <= self.n_experts:
            raise ValueError(f"top_k={self.top_k} must lie in 1..n_experts={self.n_experts}")

    @staticmethod
    def tiny(**kw) -> "MoEConfig":
        """2 layers, width 128, 4 heads, 4 experts of hidden 256, top-2, vocab 512."""
        base = dict(vocab_size=512, d_model=128, n_layers=2, n_heads=4, n_kv_heads=4, head_dim=32, ffn_hidden=512,
                    rope_theta=10000.0, n_experts=4, top_k=2, expert_hidden=256, loss_chunk=0)
        base.update(kw)
        return MoEConfig(**base)


class Expert(nn.Module):
    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.gate_proj = nn.Linear(d_model, hidden, bias=False)
        self.up_proj = nn.Linear(d_model, hidden, bias=False)
        self.down_proj = nn.Linear(hidden, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class MoEFeedForward(nn.Module):
    """Token-choice routing.  ``forward`` returns the mixed expert outputs and the
    load-balancing statistic of the layer (fraction of tokens per expert times mean
    gate probability per expert, summed and scaled by ``n_experts``: 1 when
    perfectly balanced)."""

    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.top_k = cfg.top_k
        self.router = nn.Linear(cfg.d_model, cfg.n_experts, bias=False)          # not a "proj": stays with FSDP2 / AdamW
        self.experts = nn.ModuleList(Expert(cfg.d_model, cfg.expert_hidden) for _ in range(cfg.n_experts))

    def forward(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        shape = x.shape
        tokens = x.reshape(-1, shape[-1])
        probs = F.softmax(self.router(tokens).float(), dim=-1)
        gate, choice = probs.topk(self.top_k, dim=-1)
        gate = (gate / gate.sum(dim=-1, keepdim=True)).to(tokens.dtype)
        out = torch.zeros_like(tokens)
        n_exp = len(self.experts)
        for e, expert in enumerate(self.experts):
            rows, slot = (choice == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue                        # no token chose this expert here: its weights get no gradient on this rank
            out = out.index_add(0, rows, expert(tokens[rows]) * gate[rows, slot].unsqueeze(-1))
        load = torch.zeros(n_exp, dtype=probs.dtype, device=probs.device)
        load = load.index_add(0, choice.reshape(-1), torch.ones(choice.numel(), dtype=probs.dtype, device=probs.device))
        balance = n_exp * ((load / choice.numel()) * probs.mean(dim=0)).sum()
        return out.reshape(shape), balance


class MoEDecoderLayer(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.mlp = MoEFeedForward(cfg)

    def forward(self, x: torch.Tensor, rope: RopeTables) -> tuple[torch.Tensor, torch.Tensor]:
        x = x + self.self_attn(self.input_layernorm(x), rope)
        y, balance = self.mlp(self.post_attention_layernorm(x))
        return x + y, balance


class MoEModel(nn.Module):
    """``forward(input_ids, labels=None)`` returns logits, or the mean next-token
    cross-entropy (plus ``balance_coef`` times the mean load-balancing statistic)
    when ``labels`` is given."""

    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(MoEDecoderLayer(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                m.weight.normal_(0.0, self.cfg.init_std)
            elif isinstance(m, RMSNorm):
                m.weight.fill_(1.0)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.embed_tokens(input_ids)
        rope = RopeTables(*rope_tables(input_ids.shape[1], self.cfg.head_dim, self.cfg.rope_theta, x.device))
        balance = x.new_zeros((), dtype=torch.float32)
        for layer in self.layers:
            x, b = layer(x, rope)
            balance = balance + b
        h = self.norm(x)
        logits = self.lm_head(h)
        if labels is None:
            return logits
        loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1))
        if self.cfg.balance_coef:
            loss = loss + self.cfg.balance_coef * balance / len(self.layers)
        return loss

"""A Llama-style decoder in stock PyTorch (RMSNorm, rotary embeddings,
grouped-query attention through ``scaled_dot_product_attention``, SwiGLU MLP,
tied input/output embeddings).

The reference's end-to-end run fine-tunes the Hugging Face Llama-3.2-1B
checkpoint (implementation/custom_backend/dp.py:99-100).  There is no network
on the benchmark machines, so the same architecture is built here with random
weights; ``LlamaConfig.llama32_1b()`` is that shape: 16 layers, hidden 2048,
32 heads with 8 KV heads, FFN 8192, vocabulary 128256.  The model compute is
deliberately plain PyTorch: the subject of this library is the gradient
AllReduce, not the model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 2048
    intermediate_size: int = 8192
    num_layers: int = 16
    num_heads: int = 32
    num_kv_heads: int = 8
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    tie_embeddings: bool = True
    max_seq_len: int = 8192

    @classmethod
    def llama32_1b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(vocab_size=512, hidden_size=128, intermediate_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                   max_seq_len=256)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    def num_parameters(self) -> int:
        h, f, v, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_layers
        kv = self.num_kv_heads * self.head_dim
        per_layer = h * h * 2 + h * kv * 2 + 3 * h * f + 2 * h
        return L * per_layer + v * h * (1 if self.tie_embeddings else 2) + h


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        dtype = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return (x.to(dtype)) * self.weight


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    freqs = torch.outer(t, inv)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rope(x, cos, sin):
    # x: [B, H, S, D]; rotate pairs (first half, second half), the Llama convention
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    cos, sin = cos[None, None, : x.shape[2]], sin[None, None, : x.shape[2]]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        kv = cfg.num_kv_heads * cfg.head_dim
        self.q_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)
        self.k_proj = nn.Linear(cfg.hidden_size, kv, bias=False)
        self.v_proj = nn.Linear(cfg.hidden_size, kv, bias=False)
        self.o_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        c = self.cfg
        q = self.q_proj(x).view(B, S, c.num_heads, c.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(B, S, c.num_kv_heads, c.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(B, S, c.num_kv_heads, c.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=c.num_kv_heads != c.num_heads)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, c.hidden_size))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.mlp = MLP(cfg)

    def forward(self, x, cos, sin):
        x = x + self.self_attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.num_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.lm_head = None if cfg.tie_embeddings else nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def forward(self, input_ids, labels: Optional[torch.Tensor] = None):
        """Returns the logits, or the mean next-token cross-entropy when
        ``labels`` is given (shifted inside, as Hugging Face models do)."""
        B, S = input_ids.shape
        x = self.embed_tokens(input_ids)
        cos, sin = rope_tables(S, self.cfg.head_dim, self.cfg.rope_theta, x.device, x.dtype)
        for layer in self.layers:
            x = layer(x, cos, sin)
        x = self.norm(x)
        w = self.embed_tokens.weight if self.lm_head is None else self.lm_head.weight
        if labels is None:
            return F.linear(x, w)
        logits = F.linear(x[:, :-1], w)
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1))

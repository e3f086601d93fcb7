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

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, Optional

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
    # Llama-3 frequency scaling of the rotary embedding ({"factor", "low_freq_factor", "high_freq_factor",
    # "original_max_position_embeddings"}); None = plain rotary embedding
    rope_scaling: Optional[dict] = None

    @classmethod
    def llama32_1b(cls) -> "LlamaConfig":
        """The shape (and rotary scaling) of the Llama-3.2-1B checkpoint."""
        return cls(max_seq_len=131072, rope_scaling={"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                      "original_max_position_embeddings": 8192})

    @classmethod
    def from_hf(cls, d: dict) -> "LlamaConfig":
        """From the ``config.json`` of a Hugging Face Llama checkpoint."""
        rs = d.get("rope_scaling")
        if rs is not None and rs.get("rope_type", rs.get("type")) not in ("llama3",):
            rs = None
        return cls(vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], intermediate_size=d["intermediate_size"],
                   num_layers=d["num_hidden_layers"], num_heads=d["num_attention_heads"],
                   num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
                   rope_theta=float(d.get("rope_theta", 10000.0)), rms_eps=float(d.get("rms_norm_eps", 1e-5)),
                   tie_embeddings=bool(d.get("tie_word_embeddings", False)),
                   max_seq_len=int(d.get("max_position_embeddings", 8192)), rope_scaling=rs)

    def to_hf(self) -> dict:
        d = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": self.vocab_size,
             "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
             "num_hidden_layers": self.num_layers, "num_attention_heads": self.num_heads,
             "num_key_value_heads": self.num_kv_heads, "head_dim": self.head_dim, "hidden_act": "silu",
             "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_eps, "tie_word_embeddings": self.tie_embeddings,
             "max_position_embeddings": self.max_seq_len, "attention_bias": False, "mlp_bias": False}
        if self.rope_scaling is not None:
            d["rope_scaling"] = dict(self.rope_scaling, rope_type="llama3")
        return d

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


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype=torch.float32, scaling: Optional[dict] = None):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    if scaling is not None:
        # Llama-3 scaling: long wavelengths are stretched by `factor`, short ones kept, the band between blended
        factor, lo, hi = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = ((orig / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)
        inv = (1.0 - smooth) * inv / factor + smooth * inv
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

    def forward(self, input_ids, labels: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None):
        """Returns the logits, or the mean next-token cross-entropy when
        ``labels`` is given (shifted inside, as Hugging Face models do; label -100 is ignored).
        ``attention_mask`` is accepted for batches that carry one and not needed: attention is causal and the
        padding sits on the right, so no real token attends to padding, and padded positions have label -100."""
        B, S = input_ids.shape
        x = self.embed_tokens(input_ids)
        cos, sin = rope_tables(S, self.cfg.head_dim, self.cfg.rope_theta, x.device, x.dtype, self.cfg.rope_scaling)
        for layer in self.layers:
            x = layer(x, cos, sin)
        x = self.norm(x)
        w = self.embed_tokens.weight if self.lm_head is None else self.lm_head.weight
        if labels is None:
            return F.linear(x, w)
        logits = F.linear(x[:, :-1], w)
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1))

    # ---- Hugging Face checkpoint layout (config.json + model.safetensors), so that a directory written by
    # ``AutoModelForCausalLM.save_pretrained`` (motivation/load_model.py) can be loaded and vice versa
    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        out = {}
        for k, v in self.state_dict().items():
            out[k if k.startswith("lm_head.") else "model." + k] = v.detach().contiguous()
        return out

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        own = {}
        for k, v in sd.items():
            if k == "lm_head.weight":
                if self.lm_head is not None:
                    own[k] = v
                continue               # tied: the head is the embedding
            own[k[len("model."):] if k.startswith("model.") else k] = v
        missing, unexpected = self.load_state_dict(own, strict=False)
        missing = [m for m in missing if not (m == "lm_head.weight" and "embed_tokens.weight" in own)]
        if "lm_head.weight" in self.state_dict() and "lm_head.weight" not in own:
            self.lm_head.weight.data.copy_(self.embed_tokens.weight.data)   # checkpoint with tied weights
        if missing or unexpected:
            raise KeyError(f"checkpoint does not match the model: missing {missing}, unexpected {list(unexpected)}")

    def save_pretrained(self, directory: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump(dict(self.cfg.to_hf(), torch_dtype=str(next(self.parameters()).dtype).replace("torch.", "")), f, indent=1)
        save_file(self.hf_state_dict(), os.path.join(directory, "model.safetensors"), metadata={"format": "pt"})

    @classmethod
    def from_pretrained(cls, directory: str, dtype: Optional[torch.dtype] = None) -> "LlamaForCausalLM":
        """Loads ``config.json`` and the weights (``*.safetensors``, sharded or not, else ``pytorch_model.bin``)."""
        with open(os.path.join(directory, "config.json")) as f:
            cfg = LlamaConfig.from_hf(json.load(f))
        with torch.device("meta"):
            model = cls(cfg)
        model = model.to_empty(device="cpu")
        sd: Dict[str, torch.Tensor] = {}
        shards = sorted(fn for fn in os.listdir(directory) if fn.endswith(".safetensors"))
        if shards:
            from safetensors.torch import load_file
            for fn in shards:
                sd.update(load_file(os.path.join(directory, fn)))
        else:
            sd = torch.load(os.path.join(directory, "pytorch_model.bin"), map_location="cpu", weights_only=True)
        model.load_hf_state_dict(sd)
        return model.to(dtype) if dtype is not None else model

"""Llama-3-architecture decoder in plain PyTorch (benchmark / test model).

RMSNorm, rotary position embedding, grouped-query attention through
``F.scaled_dot_product_attention``, SwiGLU feed-forward, untied embedding and
output head.  Forward and backward are stock PyTorch on purpose: the library's
subject is the optimizer and its collectives, and the same model runs under
the reference for comparisons.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    max_seq_len: int = 4096
    activation_checkpointing: bool = False

    @classmethod
    def llama3_8b(cls, **kw) -> "LlamaConfig":
        return cls(**kw)

    @classmethod
    def llama3_70b(cls, **kw) -> "LlamaConfig":
        return cls(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_dim=28672, **kw)

    @classmethod
    def tiny(cls, **kw) -> "LlamaConfig":
        d = dict(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256, max_seq_len=128)
        d.update(kw)
        return cls(**d)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    ang = torch.outer(t, inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [B, H, S, D]; rotate pairs (even, odd halves)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    cos = cos[None, None, :, :]
    sin = sin[None, None, :, :]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_heads, self.n_kv = cfg.n_heads, cfg.n_kv_heads
        self.hd = cfg.dim // cfg.n_heads
        self.wq = nn.Linear(cfg.dim, cfg.n_heads * self.hd, bias=False)
        self.wk = nn.Linear(cfg.dim, cfg.n_kv_heads * self.hd, bias=False)
        self.wv = nn.Linear(cfg.dim, cfg.n_kv_heads * self.hd, bias=False)
        self.wo = nn.Linear(cfg.n_heads * self.hd, cfg.dim, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        q = self.wq(x).view(b, s, self.n_heads, self.hd).transpose(1, 2)
        k = self.wk(x).view(b, s, self.n_kv, self.hd).transpose(1, 2)
        v = self.wv(x).view(b, s, self.n_kv, self.hd).transpose(1, 2)
        q = apply_rope(q, cos, sin)
        k = apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.n_kv != self.n_heads)
        return self.wo(o.transpose(1, 2).reshape(b, s, -1))


class FeedForward(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.w1 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
        self.w3 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
        self.w2 = nn.Linear(cfg.ffn_dim, cfg.dim, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.attention = Attention(cfg)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.feed_forward = FeedForward(cfg)

    def forward(self, x, cos, sin):
        x = x + self.attention(self.attention_norm(x), cos, sin)
        return x + self.feed_forward(self.ffn_norm(x))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.output = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)

    @torch.no_grad()
    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device=self.tok_embeddings.weight.device).manual_seed(seed)
        for p in self.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, std, generator=g)
            else:
                p.fill_(1.0)

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None):
        b, s = tokens.shape
        h = self.tok_embeddings(tokens)
        cos, sin = rope_tables(s, self.cfg.dim // self.cfg.n_heads, self.cfg.rope_theta, tokens.device, h.dtype)
        for layer in self.layers:
            if self.cfg.activation_checkpointing and self.training:
                h = checkpoint(layer, h, cos, sin, use_reentrant=False)
            else:
                h = layer(h, cos, sin)
        logits = self.output(self.norm(h))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(b * s, -1), targets.reshape(-1))


def num_params(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters())

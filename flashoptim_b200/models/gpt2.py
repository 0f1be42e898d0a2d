"""GPT-2-architecture decoder in plain PyTorch (benchmark / test model).

Learned position embedding, pre-LayerNorm blocks, fused-QKV attention through
``F.scaled_dot_product_attention``, GELU MLP, output head tied to the token
embedding (as in GPT-2).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    d_mlp: int = 4096
    max_seq_len: int = 1024
    tie_weights: bool = True

    @classmethod
    def medium(cls, **kw) -> "GPT2Config":
        return cls(**kw)

    @classmethod
    def tiny(cls, **kw) -> "GPT2Config":
        d = dict(vocab_size=257, n_layer=2, n_head=4, d_model=64, d_mlp=256, max_seq_len=64)
        d.update(kw)
        return cls(**d)


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head = cfg.n_head
        self.ln_1 = nn.LayerNorm(cfg.d_model)
        self.c_attn = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.c_proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln_2 = nn.LayerNorm(cfg.d_model)
        self.c_fc = nn.Linear(cfg.d_model, cfg.d_mlp)
        self.c_out = nn.Linear(cfg.d_mlp, cfg.d_model)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.c_attn(self.ln_1(x)).split(d, dim=2)
        shape = (b, s, self.n_head, d // self.n_head)
        o = F.scaled_dot_product_attention(
            q.view(shape).transpose(1, 2), k.view(shape).transpose(1, 2), v.view(shape).transpose(1, 2),
            is_causal=True,
        )
        x = x + self.c_proj(o.transpose(1, 2).reshape(b, s, d))
        return x + self.c_out(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq_len, cfg.d_model)
        self.h = nn.ModuleList(GPT2Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_weights:
            self.lm_head.weight = self.wte.weight

    @torch.no_grad()
    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device=self.wte.weight.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, std, generator=g)
            elif name.endswith("bias"):
                p.zero_()
            else:
                p.fill_(1.0)

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None):
        b, s = tokens.shape
        pos = torch.arange(s, device=tokens.device)
        x = self.wte(tokens) + self.wpe(pos)[None]
        for blk in self.h:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(b * s, -1), targets.reshape(-1))

"""GPT-2 (decoder-only transformer, learned positions, pre-LayerNorm, tied output embedding).

Not part of the reference repository; it is the fifth benchmark configuration (GPT-2 medium:
24 layers, d = 1024, 16 heads, vocabulary 50 257, sequence 1024, bf16 autocast with float32
gradients). Attention uses PyTorch's scaled-dot-product kernel; gradient compression is
independent of the sequence length, so no sequence parallelism is involved.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 1024
    n_layer: int = 24
    n_head: int = 16
    dropout: float = 0.0

    @classmethod
    def medium(cls) -> "GPT2Config":
        return cls()

    @classmethod
    def small(cls) -> "GPT2Config":
        return cls(n_embd=768, n_layer=12, n_head=12)

    @classmethod
    def tiny(cls) -> "GPT2Config":
        return cls(vocab_size=512, n_positions=64, n_embd=64, n_layer=2, n_head=4)


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln_1 = nn.LayerNorm(cfg.n_embd)
        self.attn_qkv = nn.Linear(cfg.n_embd, 3 * cfg.n_embd)
        self.attn_proj = nn.Linear(cfg.n_embd, cfg.n_embd)
        self.ln_2 = nn.LayerNorm(cfg.n_embd)
        self.mlp_fc = nn.Linear(cfg.n_embd, 4 * cfg.n_embd)
        self.mlp_proj = nn.Linear(4 * cfg.n_embd, cfg.n_embd)
        self.n_head, self.dropout = cfg.n_head, cfg.dropout

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, t, c = x.shape
        q, k, v = self.attn_qkv(self.ln_1(x)).split(c, dim=2)
        shape = (b, t, self.n_head, c // self.n_head)
        q, k, v = (z.view(shape).transpose(1, 2) for z in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=self.dropout if self.training else 0.0)
        x = x + self.attn_proj(y.transpose(1, 2).reshape(b, t, c))
        return x + self.mlp_proj(F.gelu(self.mlp_fc(self.ln_2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config = GPT2Config()):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = nn.Embedding(cfg.n_positions, cfg.n_embd)
        self.h = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.n_embd)
        self.apply(self._init)
        for block in self.h:  # scaled init of the residual projections
            for proj in (block.attn_proj, block.mlp_proj):
                nn.init.normal_(proj.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(module: nn.Module) -> None:
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, std=0.02)
        if isinstance(module, nn.Linear) and module.bias is not None:
            nn.init.zeros_(module.bias)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        _, t = tokens.shape
        pos = torch.arange(t, device=tokens.device)
        x = self.wte(tokens) + self.wpe(pos)
        for block in self.h:
            x = block(x)
        return F.linear(self.ln_f(x), self.wte.weight)  # tied output embedding

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        logits = self(tokens)
        return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))

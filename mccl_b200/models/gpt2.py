"""GPT-2 (decoder-only transformer); ``gpt2_medium()`` is the 24-layer, d_model 1024, 16-head config."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d: int, heads: int):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.fc = nn.Linear(d, 4 * d)
        self.out = nn.Linear(4 * d, d)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, D))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, vocab: int = 50257, d_model: int = 1024, layers: int = 24, heads: int = 16, max_seq: int = 1024):
        super().__init__()
        self.wte = nn.Embedding(vocab, d_model)
        self.wpe = nn.Embedding(max_seq, d_model)
        self.blocks = nn.ModuleList(Block(d_model, heads) for _ in range(layers))
        self.ln_f = nn.LayerNorm(d_model)
        self.apply(self._init)
        for b in self.blocks:  # scaled residual projections, as in GPT-2
            for lin in (b.proj, b.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * layers))

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, idx, targets=None):
        B, T = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)  # tied output embedding
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.view(-1))


def gpt2_medium(**kw) -> GPT2:
    return GPT2(d_model=1024, layers=24, heads=16, **kw)


def gpt2_tiny(**kw) -> GPT2:
    """4 layers, d_model 128: the shape used by tests."""
    return GPT2(vocab=kw.pop("vocab", 1024), d_model=128, layers=4, heads=4, max_seq=kw.pop("max_seq", 128), **kw)

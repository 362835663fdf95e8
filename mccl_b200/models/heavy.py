"""A ~96 M parameter mixed conv / attention / MLP classifier.

Stand-in for the dummy model behind the reference's headline throughput numbers (a
convolutional trunk feeding self-attention and an MLP head, ~96.5 M parameters at
hidden=1024; reference examples/ddp_utils.py:105-147): flat feature vectors in, class
logits out, so the synthetic Gaussian-cluster dataset can drive it.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class _ConvStage(nn.Module):
    def __init__(self, cin, cout, k):
        super().__init__()
        self.a = nn.Conv2d(cin, cout, k, padding=k // 2)
        self.b = nn.Conv2d(cout, cout, 3, padding=1)
        self.na, self.nb = nn.BatchNorm2d(cout), nn.BatchNorm2d(cout)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x):
        y = F.relu(self.na(self.a(x)))
        return F.gelu(self.nb(self.b(y)) + self.skip(x))


class _SelfAttention(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.h = heads
        self.qkv, self.o, self.norm = nn.Linear(d, 3 * d), nn.Linear(d, d), nn.LayerNorm(d)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.norm(x)).view(B, T, 3, self.h, D // self.h).permute(2, 0, 3, 1, 4)
        return x + self.o(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, D))


class HeavyDummyModel(nn.Module):
    def __init__(self, input_dim: int = 512, num_classes: int = 10, hidden: int = 1024, depth: int = 4,
                 grid: int = 64, tokens: int = 16):
        super().__init__()
        if depth < 1:
            raise ValueError("depth must be >= 1")
        self.grid, self.tokens, self.hidden = grid, tokens, hidden
        self.inp = nn.Linear(input_dim, hidden)
        self.to_image = nn.Linear(hidden, 16 * grid * grid)          # the bulk of the parameters
        self.trunk = nn.Sequential(_ConvStage(16, 32, 7), _ConvStage(32, 64, 5), _ConvStage(64, 64, 5),
                                   nn.Conv2d(64, 64, 3, padding=2, dilation=2), nn.BatchNorm2d(64), nn.ReLU(),
                                   nn.Conv2d(64, 64, 3, padding=4, dilation=4), nn.BatchNorm2d(64), nn.GELU(),
                                   nn.AdaptiveAvgPool2d(16))
        self.to_seq = nn.Linear(64 * 16 * 16, hidden)
        self.pos = nn.Parameter(torch.randn(tokens, hidden) * 0.02)
        self.attn = nn.ModuleList(_SelfAttention(hidden, 8) for _ in range(2))
        head = []
        for _ in range(max(depth - 2, 1)):
            head += [nn.Linear(hidden, hidden), nn.LayerNorm(hidden), nn.ReLU(), nn.Dropout(0.1)]
        self.head = nn.Sequential(*head, nn.Linear(hidden, num_classes))

    def forward(self, x):
        B = x.shape[0]
        h = self.inp(x)
        img = self.to_image(h).view(B, 16, self.grid, self.grid)
        feat = self.trunk(img).flatten(1)
        seq = self.to_seq(feat).unsqueeze(1).expand(B, self.tokens, self.hidden) + self.pos
        for a in self.attn:
            seq = a(seq)
        return self.head(seq.mean(1))

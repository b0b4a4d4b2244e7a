"""Small fixtures: a tied-weight MLP (layers 1 and 3 share weight and bias, as in the
reference's toy, benchmark_mp.py:35-49) and a skip-connection net whose early activations are
consumed several stages later (the UNet pattern)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class TiedMLP(nn.Module):
    def __init__(self, dim: int = 10, depth_between: int = 1):
        super().__init__()
        self.first = nn.Linear(dim, dim)
        self.middle = nn.ModuleList([nn.Linear(dim, dim) for _ in range(depth_between)])
        self.last = nn.Linear(dim, dim)
        self.last.weight = self.first.weight
        self.last.bias = self.first.bias

    def forward(self, x):
        x = torch.relu(self.first(x))
        for m in self.middle:
            x = torch.relu(m(x))
        return self.last(x)


class SkipNet(nn.Module):
    """down_i outputs are added back in reverse order on the way up."""

    def __init__(self, dim: int = 16, depth: int = 3):
        super().__init__()
        self.down = nn.ModuleList([nn.Linear(dim, dim) for _ in range(depth)])
        self.mid = nn.Linear(dim, dim)
        self.up = nn.ModuleList([nn.Linear(dim, dim) for _ in range(depth)])
        self.out = nn.Linear(dim, dim)

    def forward(self, x):
        skips = []
        for d in self.down:
            x = torch.tanh(d(x))
            skips.append(x)
        x = torch.tanh(self.mid(x))
        for u in self.up:
            x = torch.tanh(u(x + skips.pop()))
        return self.out(x)


class DeepMLP(nn.Module):
    def __init__(self, dim: int = 32, depth: int = 8, out_dim: int = 10):
        super().__init__()
        self.layers = nn.ModuleList([nn.Linear(dim, dim) for _ in range(depth)])
        self.head = nn.Linear(dim, out_dim)

    def forward(self, x):
        for l in self.layers:
            x = x + F.gelu(l(x))
        return self.head(x)

"""Vision Transformer (ViT-Tiny/L/g) on the native ops.

Pre-norm encoder as in the reference's benchmark model (HF ``ViTForImageClassification``,
bench_models/models/train_vit.py:150-169): patch embedding, [CLS] token, learned position
embedding, ``depth`` x (LN -> MHSA -> residual, LN -> MLP(GELU) -> residual), final LN, linear
head on the [CLS] token.  Per block the hot path is 4 GEMM launches (fused QKV, attention
output, and the two MLP GEMMs, the first with bias+GELU in its epilogue), one flash-attention
launch and two LayerNorm launches.

The residual stream travels between blocks as a pair (x, delta): the sum x + delta is formed
inside the next LayerNorm launch, which returns both the sum and its normalised form.  Every
tensor of the stream then has exactly one consumer, so the backward pass of the LayerNorm adds
the gradient that arrives through the sum in the same launch and autograd never has to add two
gradient contributions with a separate kernel.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops


@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    mlp_dim: int = 3072
    num_classes: int = 1000
    layer_norm_eps: float = 1e-12

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @property
    def seq_len(self) -> int:
        return self.num_patches + 1


VIT_CONFIGS = {
    "vit_tiny": ViTConfig(hidden_size=192, num_layers=12, num_heads=3, mlp_dim=768, num_classes=10),
    "vit_base": ViTConfig(),
    "vit_large": ViTConfig(hidden_size=1024, num_layers=24, num_heads=16, mlp_dim=4096),
    "vit_g14": ViTConfig(patch_size=14, hidden_size=1408, num_layers=40, num_heads=16,
                         mlp_dim=6144),
}


def vit_config(name: str, **overrides) -> ViTConfig:
    cfg = VIT_CONFIGS[name]
    return ViTConfig(**{**cfg.__dict__, **overrides})


class ViTBlock(nn.Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        d = cfg.hidden_size
        self.num_heads = cfg.num_heads
        self.eps = cfg.layer_norm_eps
        self.ln1 = nn.LayerNorm(d, eps=cfg.layer_norm_eps)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d, eps=cfg.layer_norm_eps)
        self.fc1 = nn.Linear(d, cfg.mlp_dim)
        self.fc2 = nn.Linear(cfg.mlp_dim, d)

    def forward(self, x: torch.Tensor, delta: torch.Tensor):
        """(x, delta) -> (x', delta'): the stream entering the block is x + delta, the stream
        leaving it x' + delta'."""
        B, S, d = x.shape
        H = self.num_heads
        y, x = ops.layer_norm(delta, self.ln1.weight, self.ln1.bias, self.eps, residual=x)
        qkv = ops.linear(y, self.qkv.weight, self.qkv.bias).view(B, S, 3, H, d // H)
        a = ops.attention_qkv(qkv).view(B, S, d)
        delta = ops.linear(a, self.proj.weight, self.proj.bias)
        y, x = ops.layer_norm(delta, self.ln2.weight, self.ln2.bias, self.eps, residual=x)
        return x, ops.mlp(y, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias,
                          "gelu")


class ViT(nn.Module):
    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.hidden_size
        self.patch = nn.Linear(cfg.num_channels * cfg.patch_size ** 2, d)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, d))
        self.pos_embed = nn.Parameter(torch.zeros(1, cfg.seq_len, d))
        self.blocks = nn.ModuleList([ViTBlock(cfg) for _ in range(cfg.num_layers)])
        self.ln = nn.LayerNorm(d, eps=cfg.layer_norm_eps)
        self.head = nn.Linear(d, cfg.num_classes)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=0.02)
                nn.init.zeros_(m.bias)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        nn.init.trunc_normal_(self.cls_token, std=0.02)

    def patchify(self, pixel_values: torch.Tensor) -> torch.Tensor:
        B, C, Hh, Ww = pixel_values.shape
        p = self.cfg.patch_size
        x = pixel_values.view(B, C, Hh // p, p, Ww // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(B, (Hh // p) * (Ww // p), C * p * p)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        x = ops.linear(self.patchify(pixel_values), self.patch.weight, self.patch.bias)
        B = x.shape[0]
        cls = self.cls_token.to(x.dtype).expand(B, -1, -1)
        x = torch.cat([cls, x], dim=1)
        delta = self.pos_embed.to(x.dtype).expand(B, -1, -1).contiguous()
        for blk in self.blocks:
            x, delta = blk(x, delta)
        y, _ = ops.layer_norm(delta, self.ln.weight, self.ln.bias, self.cfg.layer_norm_eps,
                              residual=x)
        return ops.linear(y[:, 0], self.head.weight, self.head.bias)

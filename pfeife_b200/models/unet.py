"""SDXL-shaped UNet (2.6 B parameters at the default configuration) on the native ops,
channels-last throughout.

Structure of diffusers' ``UNet2DConditionModel`` as configured for SDXL (the reference trains it
in bench_models/models/train_sdxl.py:805-810): conv_in 4->320; time embedding plus the "text +
time ids" additive embedding; down path (320: 2 ResNets | 640: 2x[ResNet + 2 transformer
layers] | 1280: 2x[ResNet + 10 transformer layers]) with stride-2 convolutions between levels;
middle (ResNet, 10 transformer layers, ResNet); mirrored up path with 3 blocks per level whose
inputs are concatenated with the stored skip activations (the long skip edges that cross many
pipeline stages); GroupNorm + SiLU + conv_out.  Transformer layers: LayerNorm, self-attention,
LayerNorm, cross-attention over the 77x2048 text states, LayerNorm, GEGLU feed-forward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Tuple

import torch
import torch.nn as nn

from .. import ops


@dataclass
class UNetConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_channels: Tuple[int, ...] = (320, 640, 1280)
    transformer_depth: Tuple[int, ...] = (0, 2, 10)
    layers_per_block: int = 2
    head_dim: int = 64
    cross_dim: int = 2048
    pooled_dim: int = 1280
    time_id_count: int = 6
    time_id_dim: int = 256
    groups: int = 32


UNET_CONFIGS = {
    "sdxl": UNetConfig(),
    "unet_tiny": UNetConfig(block_channels=(32, 64), transformer_depth=(0, 1), head_dim=16,
                            cross_dim=32, pooled_dim=16, time_id_dim=8, groups=8),
}


def unet_config(name: str, **kw) -> UNetConfig:
    return UNetConfig(**{**UNET_CONFIGS[name].__dict__, **kw})


def sinusoidal(t: torch.Tensor, dim: int) -> torch.Tensor:
    """t [N] -> [N, dim] (cos | sin halves, flipped as in diffusers' Timesteps)."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device,
                                                        dtype=torch.float32) / half)
    ang = t.float()[:, None] * freqs[None]
    return torch.cat([ang.cos(), ang.sin()], -1)


class Conv(nn.Module):
    def __init__(self, cin, cout, k=3, stride=1):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, cin, k, k))
        self.bias = nn.Parameter(torch.zeros(cout))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        self.stride, self.pad = stride, k // 2

    def forward(self, x):
        return ops.conv2d(x, self.weight, self.bias, self.stride, self.pad)


class GroupNorm(nn.Module):
    def __init__(self, groups, c, eps=1e-5, silu=False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(c))
        self.bias = nn.Parameter(torch.zeros(c))
        self.groups, self.eps, self.silu = groups, eps, silu

    def forward(self, x):
        return ops.group_norm(x, self.weight, self.bias, self.groups, self.eps, self.silu)


class ResBlock(nn.Module):
    def __init__(self, cin, cout, emb_dim, groups):
        super().__init__()
        self.norm1 = GroupNorm(groups, cin, silu=True)
        self.conv1 = Conv(cin, cout)
        self.emb = nn.Linear(emb_dim, cout)
        self.norm2 = GroupNorm(groups, cout, silu=True)
        self.conv2 = Conv(cout, cout)
        self.short = Conv(cin, cout, k=1) if cin != cout else None

    def forward(self, x, emb_act):
        h = self.conv1(self.norm1(x))
        h = h + ops.linear(emb_act, self.emb.weight, self.emb.bias)[:, None, None, :]
        h = self.conv2(self.norm2(h))
        return h + (self.short(x) if self.short is not None else x)


class TransformerLayer(nn.Module):
    def __init__(self, dim, heads, cross_dim):
        super().__init__()
        self.heads = heads
        self.n1, self.n2, self.n3 = nn.LayerNorm(dim), nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.o1 = nn.Linear(dim, dim)
        self.q2 = nn.Linear(dim, dim, bias=False)
        self.kv2 = nn.Linear(cross_dim, 2 * dim, bias=False)
        self.o2 = nn.Linear(dim, dim)
        self.ff1 = nn.Linear(dim, 8 * dim)      # GEGLU: gate | up, 4*dim each
        self.ff2 = nn.Linear(4 * dim, dim)

    def forward(self, x, delta, ctx):
        """(x, delta) -> (x', delta'): the token stream is x + delta; the sum is formed inside
        the next LayerNorm launch, so each tensor of the stream has a single consumer and its
        gradient needs no separate add."""
        B, S, d = x.shape
        H = self.heads
        if delta is None:
            y = ops.layer_norm(x, self.n1.weight, self.n1.bias, 1e-5)
        else:
            y, x = ops.layer_norm(delta, self.n1.weight, self.n1.bias, 1e-5, residual=x)
        a = ops.attention_qkv(ops.linear(y, self.qkv.weight).view(B, S, 3, H, d // H))
        delta = ops.linear(a.view(B, S, d), self.o1.weight, self.o1.bias)
        y, x = ops.layer_norm(delta, self.n2.weight, self.n2.bias, 1e-5, residual=x)
        q = ops.linear(y, self.q2.weight).view(B, S, H, d // H)
        kv = ops.linear(ctx, self.kv2.weight).view(B, ctx.shape[1], 2, H, d // H)
        a = ops.attention(q, kv[:, :, 0], kv[:, :, 1])
        delta = ops.linear(a.view(B, S, d), self.o2.weight, self.o2.bias)
        y, x = ops.layer_norm(delta, self.n3.weight, self.n3.bias, 1e-5, residual=x)
        g = ops.geglu(ops.linear(y, self.ff1.weight, self.ff1.bias))
        return x, ops.linear(g, self.ff2.weight, self.ff2.bias)


class SpatialTransformer(nn.Module):
    def __init__(self, dim, depth, head_dim, cross_dim, groups):
        super().__init__()
        self.norm = GroupNorm(groups, dim, eps=1e-6)
        self.proj_in = nn.Linear(dim, dim)
        self.layers = nn.ModuleList([TransformerLayer(dim, dim // head_dim, cross_dim)
                                     for _ in range(depth)])
        self.proj_out = nn.Linear(dim, dim)

    def forward(self, x, ctx):
        B, Hh, Ww, C = x.shape
        h = ops.linear(self.norm(x).view(B, Hh * Ww, C), self.proj_in.weight, self.proj_in.bias)
        delta = None
        for layer in self.layers:
            h, delta = layer(h, delta, ctx)
        if delta is not None:
            h = h + delta
        h = ops.linear(h, self.proj_out.weight, self.proj_out.bias)
        return h.view(B, Hh, Ww, C) + x


class UNet(nn.Module):
    def __init__(self, cfg: UNetConfig):
        super().__init__()
        self.cfg = cfg
        ch = cfg.block_channels
        emb = ch[0] * 4
        g = cfg.groups
        self.conv_in = Conv(cfg.in_channels, ch[0])
        self.time1, self.time2 = nn.Linear(ch[0], emb), nn.Linear(emb, emb)
        add_in = cfg.pooled_dim + cfg.time_id_count * cfg.time_id_dim
        self.add1, self.add2 = nn.Linear(add_in, emb), nn.Linear(emb, emb)

        self.down_res, self.down_attn, self.down_sample = nn.ModuleList(), nn.ModuleList(), \
            nn.ModuleList()
        skip_ch: List[int] = [ch[0]]
        cur = ch[0]
        self.down_plan: List[Tuple[str, int]] = []
        for lvl, c in enumerate(ch):
            for _ in range(cfg.layers_per_block):
                self.down_res.append(ResBlock(cur, c, emb, g))
                depth = cfg.transformer_depth[lvl]
                self.down_attn.append(SpatialTransformer(c, depth, cfg.head_dim, cfg.cross_dim, g)
                                      if depth else nn.Identity())
                cur = c
                skip_ch.append(cur)
            if lvl < len(ch) - 1:
                self.down_sample.append(Conv(cur, cur, stride=2))
                skip_ch.append(cur)
        self.mid1 = ResBlock(cur, cur, emb, g)
        self.mid_attn = SpatialTransformer(cur, cfg.transformer_depth[-1], cfg.head_dim,
                                           cfg.cross_dim, g)
        self.mid2 = ResBlock(cur, cur, emb, g)

        self.up_res, self.up_attn, self.up_sample = nn.ModuleList(), nn.ModuleList(), \
            nn.ModuleList()
        for lvl in reversed(range(len(ch))):
            c = ch[lvl]
            for _ in range(cfg.layers_per_block + 1):
                self.up_res.append(ResBlock(cur + skip_ch.pop(), c, emb, g))
                depth = cfg.transformer_depth[lvl]
                self.up_attn.append(SpatialTransformer(c, depth, cfg.head_dim, cfg.cross_dim, g)
                                    if depth else nn.Identity())
                cur = c
            if lvl > 0:
                self.up_sample.append(Conv(cur, cur))
        self.norm_out = GroupNorm(g, cur, silu=True)
        self.conv_out = Conv(cur, cfg.out_channels)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, latents, timesteps, text_states, pooled, time_ids):
        """latents [B, 4, H, W] (NCHW as in diffusers), timesteps [B], text_states [B, 77, 2048],
        pooled [B, 1280], time_ids [B, 6] -> predicted noise [B, 4, H, W]."""
        cfg = self.cfg
        B = latents.shape[0]
        x = latents.permute(0, 2, 3, 1).contiguous()
        dtype = x.dtype
        t = sinusoidal(timesteps, cfg.block_channels[0]).to(dtype)
        emb = ops.linear(ops.linear(t, self.time1.weight, self.time1.bias, activation="silu"),
                         self.time2.weight, self.time2.bias)
        ids = sinusoidal(time_ids.reshape(-1), cfg.time_id_dim).view(B, -1).to(dtype)
        add = torch.cat([pooled.to(dtype), ids], -1)
        emb = emb + ops.linear(ops.linear(add, self.add1.weight, self.add1.bias, activation="silu"),
                               self.add2.weight, self.add2.bias)
        emb_act = ops.silu(emb)
        ctx = text_states.to(dtype)

        x = self.conv_in(x)
        skips = [x]
        i = s = 0
        for lvl in range(len(cfg.block_channels)):
            for _ in range(cfg.layers_per_block):
                x = self.down_res[i](x, emb_act)
                if cfg.transformer_depth[lvl]:
                    x = self.down_attn[i](x, ctx)
                skips.append(x)
                i += 1
            if lvl < len(cfg.block_channels) - 1:
                x = self.down_sample[s](x)
                skips.append(x)
                s += 1
        x = self.mid2(self.mid_attn(self.mid1(x, emb_act), ctx), emb_act)
        i = s = 0
        for lvl in reversed(range(len(cfg.block_channels))):
            for _ in range(cfg.layers_per_block + 1):
                x = self.up_res[i](torch.cat([x, skips.pop()], -1), emb_act)
                if cfg.transformer_depth[lvl]:
                    x = self.up_attn[i](x, ctx)
                i += 1
            if lvl > 0:
                x = self.up_sample[s](ops.upsample_nearest2x(x))
                s += 1
        x = self.conv_out(self.norm_out(x))
        return x.permute(0, 3, 1, 2)

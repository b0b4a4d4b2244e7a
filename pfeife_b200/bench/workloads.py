"""Benchmark workloads: the model, synthetic batch, loss and default layout of every training
configuration the project is measured on (the reference ships one trainer script per model:
bench_models/train_vit.py, train_llama.py, train_sdxl.py; here they share one harness).

A workload only describes; ``bench.py`` drives it through the public API.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass
class Workload:
    name: str
    model_name: str
    build_model: Callable[[], torch.nn.Module]
    # n samples -> CPU tensors (model inputs..., loss targets...); floats are cast to the
    # compute dtype before they are pinned
    make_batch: Callable[[int, torch.Generator], Tuple[torch.Tensor, ...]]
    # (callable model, *device batch) -> scalar loss
    loss: Callable[..., torch.Tensor]
    micro_batch: int
    batch_cnt: int
    precision: Optional[str]            # "fp16" | "bf16" | None (fp32)
    config: Dict[str, Any] = field(default_factory=dict)
    mesh_for_8: Optional[str] = None    # the layout named by the configuration (8 GPUs)
    option: Dict[str, Any] = field(default_factory=dict)   # extra PipeOption fields
    data: str = "synthetic, random-init weights"
    n_model_inputs: int = 1             # leading tensors of the batch that the model consumes


def _vit(name, model_name, cfg_name, micro_batch, batch_cnt, mesh8=None, option=None, **over):
    from ..models.vit import ViT, vit_config
    from .. import ops
    cfg = vit_config(cfg_name, **over)

    def batch(n, g):
        return (torch.randn(n, 3, cfg.image_size, cfg.image_size, generator=g),
                torch.randint(0, cfg.num_classes, (n,), generator=g))

    def loss(model, x, y):
        return ops.cross_entropy(model(x), y)

    return Workload(name, model_name, lambda: ViT(cfg), batch, loss, micro_batch, batch_cnt, "fp16",
                    config={"layers": cfg.num_layers, "hidden": cfg.hidden_size,
                            "heads": cfg.num_heads, "mlp": cfg.mlp_dim, "patch": cfg.patch_size,
                            "seq_len": cfg.seq_len, "optimizer": "AdamW"},
                    mesh_for_8=mesh8, option=option or {},
                    data="synthetic (N(0,1) images, uniform labels), random-init weights")


def _llama(name, cfg_name, micro_batch, batch_cnt, seq, mesh8, option, **over):
    from ..models.llama import Llama, causal_lm_loss, llama_config
    cfg = llama_config(cfg_name, **over)

    def batch(n, g):
        return (torch.randint(0, cfg.vocab_size, (n, seq), generator=g),)

    def loss(model, ids):
        return causal_lm_loss(model(ids), ids)

    return Workload(name, "Llama-2-7B" if cfg_name == "llama2_7b" else cfg_name,
                    lambda: Llama(cfg), batch, loss, micro_batch, batch_cnt, "bf16",
                    config={"layers": cfg.num_layers, "hidden": cfg.hidden_size,
                            "heads": cfg.num_heads, "ffn": cfg.intermediate_size,
                            "vocab": cfg.vocab_size, "seq_len": seq, "optimizer": "AdamW"},
                    mesh_for_8=mesh8, option=option,
                    data="synthetic (uniform token ids), random-init weights")


def _unet(name, cfg_name, micro_batch, batch_cnt, hw, mesh8, **over):
    from ..models.unet import UNet, unet_config
    from .. import ops
    cfg = unet_config(cfg_name, **over)

    def batch(n, g):
        r = lambda *s: torch.randn(*s, generator=g)
        return (r(n, cfg.in_channels, hw, hw), torch.randint(0, 1000, (n,), generator=g),
                r(n, 77, cfg.cross_dim), r(n, cfg.pooled_dim),
                torch.rand(n, cfg.time_id_count, generator=g) * 1024,
                r(n, cfg.out_channels, hw, hw))

    def loss(model, lat, t, txt, pooled, ids, noise):
        return ops.mse_loss(model(lat, t, txt, pooled, ids), noise)

    return Workload(name, "SDXL UNet" if cfg_name == "sdxl" else cfg_name,
                    lambda: UNet(cfg), batch, loss, micro_batch, batch_cnt, "bf16",
                    config={"block_channels": list(cfg.block_channels),
                            "transformer_depth": list(cfg.transformer_depth),
                            "latents": [cfg.in_channels, hw, hw], "optimizer": "AdamW"},
                    mesh_for_8=mesh8, n_model_inputs=5,
                    data="synthetic (N(0,1) latents / text states / noise, uniform timesteps), "
                         "random-init weights")


def get_workload(name: str, args=None) -> Workload:
    """`args` (bench.py's namespace) may override the ViT-g/14 shape and the batch sizes."""
    g = lambda k, d: getattr(args, k, None) if (args is not None and getattr(args, k, None)
                                                 is not None) else d
    if name == "vitg":
        return _vit("vitg", g("model_name", "ViT-g/14"), "vit_g14", g("batch_size", 24),
                    g("batch_cnt", 8), num_layers=g("layers", 40), hidden_size=g("hidden", 1408),
                    num_heads=g("heads", 16), mlp_dim=g("mlp", 6144), patch_size=g("patch", 14),
                    num_classes=1000)
    if name == "vitl":          # PP=4 x DP=2, prefetch_fwd 2
        return _vit("vitl", "ViT-L/16", "vit_large", 16, 8, mesh8="-2,4",
                    option={"prefetch_fwd": 2}, num_classes=1000)
    # --layers / --batch_cnt shorten a run of the big configurations (plumbing checks on few GPUs)
    over = {"num_layers": g("layers", None)} if g("layers", None) else {}
    if name == "llama7b":       # looped pipeline: 16 stages on 8 ranks
        return _llama("llama7b", "llama2_7b", 1, g("batch_cnt", 16), 2048, "8", {"loop_cnt": 2},
                      **over)
    if name == "llama7b_fsdp":  # PP=4 x DP=2, row-sharded weights between optimizer steps
        return _llama("llama7b_fsdp", "llama2_7b", 1, g("batch_cnt", 16), 2048, "-2,4",
                      {"use_fsdp": True}, **over)
    if name == "sdxl":
        return _unet("sdxl", "sdxl", 4, g("batch_cnt", 8), 128, "2,-4")
    # reduced shapes for plumbing checks (CPU / few GPUs)
    if name == "vit_tiny":
        return _vit("vit_tiny", "ViT-Tiny", "vit_tiny", g("batch_size", 4), g("batch_cnt", 4),
                    num_layers=4, image_size=32, patch_size=8)
    if name == "llama_tiny":
        return _llama("llama_tiny", "llama_tiny", g("batch_size", 2), g("batch_cnt", 4), 16, None,
                      {})
    if name == "unet_tiny":
        return _unet("unet_tiny", "unet_tiny", g("batch_size", 2), g("batch_cnt", 2), 16, None)
    raise ValueError(f"unknown workload {name!r}")


WORKLOADS = ("vitg", "vitl", "llama7b", "llama7b_fsdp", "sdxl", "vit_tiny", "llama_tiny",
             "unet_tiny")

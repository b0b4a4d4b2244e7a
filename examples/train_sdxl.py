"""Text-to-image diffusion trainer for the SDXL UNet: DDPM forward process, epsilon / v / sample
targets, optional min-SNR loss weights, noise offset, empty-prompt dropout; bf16 by default.

    python mp_launch.py --world_size 8 --dp_mesh "2,-4" examples/train_sdxl.py \\
        --resolution 1024 --train_batch_size 4 --batch_cnt 8

Counterpart of the reference's bench_models/models/train_sdxl.py (the per-micro-batch function at
:1303-1455).  The reference encodes images with the SDXL VAE and prompts with two CLIP text
encoders, all pretrained and fetched from the network; this trainer starts where those frozen
models end: VAE latents [N,4,R/8,R/8], text states [N,77,2048], pooled text embedding [N,1280],
original sizes and crop offsets [N,4] — random by default, or read from a local ``--data_file``
holding those four tensors in that order.
"""
from __future__ import annotations

import argparse

import torch

from common import (DevicePrefetcher, SyntheticDataset, TensorFileDataset, add_train_arguments,
                    make_loader, option_from_args, train_loop)

from pfeife_b200 import PartialRunner, initialize_pfeife, ops, partial_compiler
from pfeife_b200.models.unet import UNet, unet_config
from pfeife_b200.utils import set_seed


class DDPMSchedule:
    """The forward process of DDPM with the "scaled linear" betas SDXL was trained with
    (beta from 0.00085 to 0.012 in sqrt space, 1000 steps)."""

    def __init__(self, device, steps: int = 1000, beta_start: float = 0.00085,
                 beta_end: float = 0.012):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, steps, dtype=torch.float64) ** 2
        ac = torch.cumprod(1.0 - betas, 0)
        self.steps = steps
        self.sqrt_ac = ac.sqrt().float().to(device)
        self.sqrt_1mac = (1.0 - ac).sqrt().float().to(device)

    def _coef(self, table, t, like):
        return table[t].view(-1, *([1] * (like.ndim - 1))).to(like.dtype)

    def add_noise(self, x0, noise, t):
        return self._coef(self.sqrt_ac, t, x0) * x0 + self._coef(self.sqrt_1mac, t, x0) * noise

    def velocity(self, x0, noise, t):
        return self._coef(self.sqrt_ac, t, x0) * noise - self._coef(self.sqrt_1mac, t, x0) * x0

    def snr(self, t):
        return (self.sqrt_ac[t] / self.sqrt_1mac[t]) ** 2


def main():
    state = initialize_pfeife()

    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default="sdxl", choices=["sdxl", "unet_tiny"])
    parser.add_argument("--resolution", type=int, default=1024, help="image side; latents are 1/8")
    parser.add_argument("--train_batch_size", type=int, default=None,
                        help="samples per micro-batch (same as --batch_size)")
    parser.add_argument("--prediction_type", default="epsilon",
                        choices=["epsilon", "v_prediction", "sample"])
    parser.add_argument("--snr_gamma", type=float, default=None,
                        help="min-SNR loss weighting (5.0 is the usual choice)")
    parser.add_argument("--noise_offset", type=float, default=0.0)
    parser.add_argument("--proportion_empty_prompts", type=float, default=0.0,
                        help="fraction of samples trained with the text conditioning zeroed")
    add_train_arguments(parser)
    parser.set_defaults(learning_rate=1e-6, weight_decay=1e-2)
    args = parser.parse_args()
    if args.train_batch_size is not None:
        args.batch_size = args.train_batch_size
    if args.mixed_precision is None and state.device.type == "cuda":
        args.mixed_precision = "bf16"
    option = option_from_args(args)
    set_seed(args.seed)

    cfg = unet_config(args.model)
    model = UNet(cfg).to(state.device)
    side = args.resolution // 8
    dtype = option.mixed_precision or torch.float32

    def item(g):
        r = lambda *s: torch.randn(*s, generator=g)
        # integers: the loader casts floating tensors to the compute dtype, and bf16 would round sizes
        size = torch.tensor([args.resolution, args.resolution, 0, 0], dtype=torch.int64)
        return (r(cfg.in_channels, side, side) * 0.18, r(77, cfg.cross_dim), r(cfg.pooled_dim), size)

    dataset = TensorFileDataset(args.data_file, 4) if args.data_file else \
        SyntheticDataset(item, args.dataset_len, args.seed)
    loader = make_loader(dataset, option.batch_size * option.batch_cnt, args, state.dp_rank,
                         state.dp_size)
    batches = DevicePrefetcher(loader, state.device, option.mixed_precision)
    ddpm = DDPMSchedule(state.device)
    target_size = torch.tensor([args.resolution, args.resolution], dtype=torch.float32,
                               device=state.device)

    # ---- the integration
    optimizer = torch.optim.AdamW(model.parameters(), lr=args.learning_rate,
                                  weight_decay=args.weight_decay)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def iter_fn(latents, text_states, pooled, sizes):
        n = latents.shape[0]
        noise = torch.randn_like(latents)
        if args.noise_offset:
            noise = noise + args.noise_offset * torch.randn(n, latents.shape[1], 1, 1,
                                                            device=latents.device, dtype=noise.dtype)
        t = torch.randint(0, ddpm.steps, (n,), device=latents.device)
        noisy = ddpm.add_noise(latents, noise, t)
        if args.proportion_empty_prompts > 0:
            keep = (torch.rand(n, device=latents.device) >= args.proportion_empty_prompts)
            text_states = text_states * keep.view(n, 1, 1).to(text_states.dtype)
            pooled = pooled * keep.view(n, 1).to(pooled.dtype)
        # original size (h, w), crop offset (top, left), target size (h, w)
        time_ids = torch.cat([sizes.float(), target_size.expand(n, 2)], 1)[:, :cfg.time_id_count]

        pred = cmodel(noisy.to(dtype), t, text_states, pooled, time_ids)
        if args.prediction_type == "epsilon":
            target = noise
        elif args.prediction_type == "v_prediction":
            target = ddpm.velocity(latents, noise, t)
        else:
            target, pred = latents, pred - noise
        if args.snr_gamma is None:
            loss = ops.mse_loss(pred, target)
        else:
            snr = ddpm.snr(t)
            w = torch.minimum(snr, torch.full_like(snr, args.snr_gamma))
            if args.prediction_type == "epsilon":
                w = w / snr
            elif args.prediction_type == "v_prediction":
                w = w / (snr + 1)
            per = (pred.float() - target.float()).pow(2).flatten(1).mean(1)
            loss = (per * w).mean()
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(iter_fn)
    train_loop(args, runner, model, batches)


if __name__ == "__main__":
    main()

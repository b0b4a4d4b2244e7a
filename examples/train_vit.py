"""Image-classification trainer: ViT-g/14 (default), ViT-L/16 or smaller, 10 classes, AdamW,
fp16 autocast with the job-wide loss scaler.

    python mp_launch.py --world_size 8 examples/train_vit.py --batch_size 24 --batch_cnt 8

Counterpart of the reference's bench_models/models/train_vit.py (model shape at :148-160, the
integration at :45-64).  Data: random images and labels of CIFAR-10's shape after the 224-pixel
resize, or a local ``--data_file`` holding ``(pixel_values [N,3,H,W], labels [N])``.
"""
from __future__ import annotations

import argparse

import torch

from common import (DevicePrefetcher, SyntheticDataset, TensorFileDataset, add_train_arguments,
                    make_loader, option_from_args, train_loop)

from pfeife_b200 import PartialRunner, initialize_pfeife, ops, partial_compiler
from pfeife_b200.models.vit import ViT, vit_config
from pfeife_b200.utils import set_seed


def main():
    state = initialize_pfeife()

    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default="vit_g14",
                        choices=["vit_g14", "vit_large", "vit_base", "vit_tiny"])
    parser.add_argument("--num_labels", type=int, default=10)
    parser.add_argument("--image_size", type=int, default=224)
    parser.add_argument("--num_layers", type=int, default=None, help="override the model's depth")
    add_train_arguments(parser)
    args = parser.parse_args()
    if args.mixed_precision is None and state.device.type == "cuda":
        args.mixed_precision = "fp16"
    option = option_from_args(args)
    set_seed(args.seed)

    over = {"num_classes": args.num_labels, "image_size": args.image_size}
    if args.num_layers:
        over["num_layers"] = args.num_layers
    if args.model == "vit_g14" and args.num_layers is None:
        over["num_layers"] = 32        # the depth of the reference's trainer (its ViTConfig)
    cfg = vit_config(args.model, **over)
    if args.image_size % cfg.patch_size:
        raise SystemExit(f"--image_size must be a multiple of the patch size {cfg.patch_size}")
    model = ViT(cfg).to(state.device)

    def item(g):
        return (torch.randn(3, cfg.image_size, cfg.image_size, generator=g),
                torch.randint(0, cfg.num_classes, (), generator=g))

    dataset = TensorFileDataset(args.data_file, 2) if args.data_file else \
        SyntheticDataset(item, args.dataset_len, args.seed)
    loader = make_loader(dataset, option.batch_size * option.batch_cnt, args, state.dp_rank,
                         state.dp_size)
    batches = DevicePrefetcher(loader, state.device, option.mixed_precision)

    # ---- the integration: an optimizer over the whole model, a runner, a compiled model and a
    # per-micro-batch function that ends in backward()
    optimizer = torch.optim.AdamW(model.parameters(), lr=args.learning_rate * state.dp_size,
                                  weight_decay=args.weight_decay)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def iter_fn(pixel_values, labels):
        loss = ops.cross_entropy(cmodel(pixel_values), labels)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(iter_fn)
    train_loop(args, runner, model, batches)


if __name__ == "__main__":
    main()

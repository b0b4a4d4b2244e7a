"""Causal language-model trainer: Llama-2-7B shape (default) or a reduced one, bf16, AdamW with
decay on the matrices only, a linear learning-rate schedule with warm-up.

    python mp_launch.py --world_size 8 examples/train_llama.py \\
        --block_size 2048 --per_device_train_batch_size 1 --batch_cnt 16 --loop_cnt 2

Counterpart of the reference's bench_models/models/train_llama.py (grouped texts of
``block_size`` tokens at :560-576, the two weight-decay groups at :610-630, the integration at
:754-789).  Data: uniform random token ids, or a local ``--data_file`` holding one tensor
``input_ids [N, block_size]`` (already tokenised and grouped); labels are the ids shifted by one.
"""
from __future__ import annotations

import argparse

import torch

from common import (DevicePrefetcher, SyntheticDataset, TensorFileDataset, add_train_arguments,
                    make_loader, option_from_args, train_loop)

from pfeife_b200 import PartialRunner, initialize_pfeife, partial_compiler
from pfeife_b200.models.llama import Llama, causal_lm_loss, llama_config
from pfeife_b200.utils import set_seed


def decay_groups(model: torch.nn.Module, weight_decay: float):
    """Matrices decay; norm gains and biases do not."""
    decay = [p for p in model.parameters() if p.requires_grad and p.ndim >= 2]
    rest = [p for p in model.parameters() if p.requires_grad and p.ndim < 2]
    groups = [{"params": decay, "weight_decay": weight_decay}]
    if rest:
        groups.append({"params": rest, "weight_decay": 0.0})
    return groups


def linear_schedule(optimizer, warmup: int, total: int):
    def factor(step: int) -> float:
        if step < warmup:
            return (step + 1) / max(1, warmup)
        return max(0.0, (total - step) / max(1, total - warmup))
    return torch.optim.lr_scheduler.LambdaLR(optimizer, factor)


def main():
    state = initialize_pfeife()

    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default="llama2_7b", choices=["llama2_7b", "llama_tiny"])
    parser.add_argument("--block_size", type=int, default=2048, help="tokens per sample")
    parser.add_argument("--per_device_train_batch_size", type=int, default=None,
                        help="samples per micro-batch (same as --batch_size)")
    parser.add_argument("--num_layers", type=int, default=None, help="override the model's depth")
    parser.add_argument("--tie_embeddings", action="store_true",
                        help="share the embedding with the output projection (its gradient is then "
                             "summed across the stages that hold a copy)")
    parser.add_argument("--lr_scheduler_type", default="linear", choices=["linear", "constant"])
    parser.add_argument("--num_warmup_steps", type=int, default=0)
    add_train_arguments(parser)
    parser.set_defaults(learning_rate=5e-5, weight_decay=0.0)
    args = parser.parse_args()
    if args.per_device_train_batch_size is not None:
        args.batch_size = args.per_device_train_batch_size
    if args.mixed_precision is None and state.device.type == "cuda":
        args.mixed_precision = "bf16"
    option = option_from_args(args)
    set_seed(args.seed)

    over = {"max_seq_len": args.block_size, "tie_embeddings": args.tie_embeddings}
    if args.num_layers:
        over["num_layers"] = args.num_layers
    cfg = llama_config(args.model, **over)
    model = Llama(cfg).to(state.device)

    def item(g):
        return (torch.randint(0, cfg.vocab_size, (args.block_size,), generator=g),)

    dataset = TensorFileDataset(args.data_file, 1) if args.data_file else \
        SyntheticDataset(item, args.dataset_len, args.seed)
    loader = make_loader(dataset, option.batch_size * option.batch_cnt, args, state.dp_rank,
                         state.dp_size)
    batches = DevicePrefetcher(loader, state.device)

    # ---- the integration
    optimizer = torch.optim.AdamW(decay_groups(model, args.weight_decay), lr=args.learning_rate)
    scheduler = linear_schedule(optimizer, args.num_warmup_steps, args.iter_cnt) \
        if args.lr_scheduler_type == "linear" else None
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def iter_fn(input_ids):
        loss = causal_lm_loss(cmodel(input_ids), input_ids)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(iter_fn)
    train_loop(args, runner, model, batches, scheduler)


if __name__ == "__main__":
    main()

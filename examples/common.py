"""What the three example trainers share: synthetic datasets, a loader that keeps the next batch
in flight to the device, the training loop with its throughput lines, and checkpoints.

The reference's trainers (bench_models/models/train_vit.py, train_llama.py, train_sdxl.py) read
HuggingFace datasets and pretrained weights from the network; these examples run anywhere:
random data of the same shapes by default, or tensors from a local ``--data_file``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import DataLoader, Dataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from pfeife_b200 import PipeOption, get_state  # noqa: E402


class SyntheticDataset(Dataset):
    """``length`` samples drawn on demand; item ``i`` is a pure function of ``(seed, i)``, so every
    epoch, every loader worker and every resumed run sees the same sample at the same index."""

    def __init__(self, make_item: Callable[[torch.Generator], Sequence[torch.Tensor]], length: int,
                 seed: int = 0):
        self.make_item, self.length, self.seed = make_item, length, seed

    def __len__(self) -> int:
        return self.length

    def __getitem__(self, i: int):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        return tuple(self.make_item(g))


class TensorFileDataset(Dataset):
    """A ``torch.save``d tuple/list of tensors with a common leading dimension (one entry per
    element of the batch the trainer expects)."""

    def __init__(self, path: str, n_fields: int):
        obj = torch.load(path, map_location="cpu")
        if isinstance(obj, dict):
            obj = list(obj.values())
        if len(obj) != n_fields:
            raise ValueError(f"{path}: expected {n_fields} tensors, found {len(obj)}")
        n = {int(t.shape[0]) for t in obj}
        if len(n) != 1:
            raise ValueError(f"{path}: tensors disagree on the number of samples: {sorted(n)}")
        self.fields = list(obj)

    def __len__(self) -> int:
        return int(self.fields[0].shape[0])

    def __getitem__(self, i: int):
        return tuple(t[i] for t in self.fields)


class ResumableSampler(torch.utils.data.Sampler):
    """A shuffled pass over the data per epoch; the order is a function of ``(seed, epoch)`` alone
    and every data-parallel replica takes its own stride of it, so a resumed run can be put back
    at the exact sample where the checkpoint was taken."""

    def __init__(self, n: int, seed: int, dp_rank: int = 0, dp_size: int = 1):
        self.n, self.seed, self.dp_rank, self.dp_size = n, seed, dp_rank, dp_size
        self.epoch, self.skip = 0, 0

    def __len__(self) -> int:
        return self.n // self.dp_size

    def set_position(self, epoch: int, skip_samples: int = 0) -> None:
        self.epoch, self.skip = epoch, skip_samples

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed * 7919 + self.epoch)
        order = torch.randperm(self.n, generator=g)[self.dp_rank::self.dp_size][:len(self)]
        skip, self.skip = self.skip, 0
        return iter(order[skip:].tolist())


def make_loader(dataset: Dataset, batch: int, args, dp_rank: int, dp_size: int) -> DataLoader:
    sampler = ResumableSampler(len(dataset), args.seed, dp_rank, dp_size)
    if len(sampler) < batch:
        raise SystemExit(f"{len(dataset)} samples are fewer than one step needs "
                         f"({batch} per replica x {dp_size} replicas)")
    return DataLoader(dataset, batch_size=batch, sampler=sampler, drop_last=True,
                      num_workers=args.num_workers,
                      pin_memory=torch.cuda.is_available() and not args.cpu)


class DevicePrefetcher:
    """Iterates a loader for ever (epoch after epoch) and returns batches that already live on
    the device: the copy of batch i+1 is issued on a side stream while step i runs."""

    def __init__(self, loader: DataLoader, device: torch.device, cast: Optional[torch.dtype] = None):
        self.loader, self.device, self.cast = loader, device, cast
        self.stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self.epoch = 0
        self._it = None
        self._next = None

    def seek(self, step: int) -> None:
        """Positions the stream of batches at optimizer step ``step`` (before the first ``next``)."""
        per_epoch = len(self.loader)
        self.epoch = step // per_epoch
        self.loader.sampler.set_position(self.epoch, (step % per_epoch) * self.loader.batch_size)
        self._it, self._next = None, None

    def _epochs(self) -> Iterator:
        first = True
        while True:
            if not first:
                self.loader.sampler.set_position(self.epoch)
            first = False
            yield from self.loader
            self.epoch += 1

    def _move(self, t: torch.Tensor) -> torch.Tensor:
        t = t.to(self.device, non_blocking=True)
        return t.to(self.cast) if (self.cast is not None and t.is_floating_point()) else t

    def _issue(self):
        batch = next(self._it)
        if self.stream is None:
            return [self._move(t) for t in batch], None
        with torch.cuda.stream(self.stream):
            moved = [self._move(t) for t in batch]
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return moved, ev

    def next(self) -> List[torch.Tensor]:
        if self._it is None:
            self._it = self._epochs()
            self._next = self._issue()
        batch, ev = self._next
        self._next = self._issue()
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for t in batch:
                t.record_stream(cur)
        return batch


def add_train_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    parser.add_argument("--iter_cnt", type=int, default=300, help="optimizer steps to run")
    parser.add_argument("--learning_rate", type=float, default=3e-4)
    parser.add_argument("--weight_decay", type=float, default=0.1)
    parser.add_argument("--warmup_iters", type=int, default=20,
                        help="steps left out of the throughput figure")
    parser.add_argument("--log_every", type=int, default=20)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--num_workers", type=int, default=0, help="data loader workers")
    parser.add_argument("--dataset_len", type=int, default=4096, help="synthetic samples per epoch")
    parser.add_argument("--data_file", default=None,
                        help="torch.save'd tuple of tensors to train on instead of random data")
    parser.add_argument("--output_dir", default=None, help="where checkpoints go")
    parser.add_argument("--checkpointing_steps", type=int, default=0,
                        help="write a checkpoint every this many steps (0: only at the end, and "
                             "only with --output_dir)")
    parser.add_argument("--resume_from", default=None, help="checkpoint file to continue from")
    PipeOption.add_arguments(parser)
    return parser


def option_from_args(args) -> PipeOption:
    """The pipeline depth is the mesh's: ``--device_cnt`` follows the launcher's ``--dp_mesh``."""
    state = get_state()
    args.device_cnt = state.pp_size
    if state.device.type == "cpu":      # launched with ``mp_launch.py --cpu``
        args.cpu = True
    return PipeOption.from_args(args)


def save_checkpoint(path: str, runner, model: torch.nn.Module, step: int, extra: Dict = None):
    """``gather_params`` brings every stage's parameters back into the user's module, so the file
    holds an ordinary ``state_dict`` plus the optimizer moments keyed by parameter name."""
    opt = runner.gather_params(with_optimizer=True)
    state = get_state()
    if state.is_main_process:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        tmp = path + ".tmp"
        torch.save({"model": {k: v.detach().cpu() for k, v in model.state_dict().items()},
                    "optimizer": opt, "step": step, **(extra or {})}, tmp)
        os.replace(tmp, path)


def load_checkpoint(path: str, runner, lr_scheduler=None) -> int:
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    runner.load_params(ckpt["model"], ckpt.get("optimizer"))
    if lr_scheduler is not None and ckpt.get("lr_scheduler") is not None:
        lr_scheduler.load_state_dict(ckpt["lr_scheduler"])
    if ckpt.get("rng_cpu") is not None:
        torch.set_rng_state(ckpt["rng_cpu"])
    if ckpt.get("rng_cuda") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(ckpt["rng_cuda"])
    return int(ckpt.get("step", 0))


def _train_state(lr_scheduler) -> Dict:
    """What a resumed run needs beside the weights: where the schedule stands and the generators
    that draw the noise and timesteps of the diffusion trainer."""
    return {"lr_scheduler": lr_scheduler.state_dict() if lr_scheduler is not None else None,
            "rng_cpu": torch.get_rng_state(),
            "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}


def train_loop(args, runner, model: torch.nn.Module, batches: DevicePrefetcher,
               lr_scheduler=None) -> Dict[str, float]:
    """Runs ``--iter_cnt`` optimizer steps; prints the running and the recent throughput every
    ``--log_every`` steps after the warm-up, in the reference trainers' "it/s" format, and the
    samples per second of the whole job beside it."""
    state = get_state()
    option = runner.option
    per_step = option.batch_size * option.batch_cnt * state.dp_size
    step0 = load_checkpoint(args.resume_from, runner, lr_scheduler) if args.resume_from else 0
    if step0:
        batches.seek(step0)
    ckpt = (lambda s: os.path.join(args.output_dir, f"checkpoint-{s}.pt")) if args.output_dir else None

    counted, start, last, loss = 0, time.time(), time.time(), float("nan")
    for it in range(step0, args.iter_cnt):
        losses = runner.step(*batches.next())
        if lr_scheduler is not None:
            lr_scheduler.step()
        done = it - step0 + 1
        if done <= args.warmup_iters:
            if done == args.warmup_iters or done == args.iter_cnt - step0:
                loss = float(torch.stack([l.float() for l in losses]).mean())
            start = last = time.time()
        else:
            counted += 1
            if counted % args.log_every == 0:
                # one host read per logging interval; the steps in between stay asynchronous
                loss = float(torch.stack([l.float() for l in losses]).mean())
                now = time.time()
                if state.is_main_process:
                    print(f"throughput {counted}: {counted / (now - start):7.5f} it/s, "
                          f"{args.log_every / (now - last):7.5f} it/s, "
                          f"{per_step * counted / (now - start):9.2f} samples/s, loss {loss:.4f}",
                          flush=True)
                last = now
        if ckpt and args.checkpointing_steps and (it + 1) % args.checkpointing_steps == 0:
            save_checkpoint(ckpt(it + 1), runner, model, it + 1, _train_state(lr_scheduler))
    loss = float(torch.stack([l.float() for l in losses]).mean()) if args.iter_cnt > step0 else loss
    end = time.time()
    its = counted / (end - start) if counted else 0.0
    if state.is_main_process:
        print(f"throughput: {its:7.5f} it/s, {per_step * its:9.2f} samples/s, final loss {loss:.4f}",
              flush=True)
    if ckpt:
        save_checkpoint(ckpt(args.iter_cnt), runner, model, args.iter_cnt,
                        _train_state(lr_scheduler))
    runner.close()
    return {"it_per_s": its, "samples_per_s": per_step * its, "loss": loss}

"""Benchmark / validity driver for the process-per-GPU runtime.

    python mp_launch.py --world_size 4 benchmark_mp.py --model hf_Bert --batch_size 8 --batch_cnt 8
    python mp_launch.py --world_size 2 benchmark_mp.py --model toy --check_valid
    python mp_launch.py --world_size 2 --cpu benchmark_mp.py --model tv:resnet18 --repeat 5

``--check_valid`` trains the pipelined model and an un-pipelined copy side by side (same
micro-batches, same Adam) and prints how far the summed losses are apart after every step;
the default run times ``--repeat`` optimizer steps; ``--profile`` writes a Chrome trace of three
steps.  Counterpart of the reference's benchmark_mp.py (models at :158-184, validity check at
:186-327, timing at :380-405, trace at :52-99); models come from ``pfeife_b200.bench.zoo``.
"""
from __future__ import annotations

import argparse
import copy
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, partial_compiler  # noqa: E402
from pfeife_b200.bench.zoo import prepare_model, replace_batch_norm  # noqa: E402
from pfeife_b200.loss import RescaleLoss  # noqa: E402
from pfeife_b200.utils import set_seed  # noqa: E402
from pfeife_b200.utils.batch import split_args_kwargs  # noqa: E402


def _to(x, device, dtype=None):
    if torch.is_tensor(x):
        x = x.to(device)
        return x.to(dtype) if (dtype is not None and x.is_floating_point()) else x
    if isinstance(x, (tuple, list)):
        return type(x)(_to(e, device, dtype) for e in x)
    if isinstance(x, dict):
        return {k: _to(v, device, dtype) for k, v in x.items()}
    return x


def build(args, option, state):
    n = option.batch_size * option.batch_cnt
    model, vargs, kwargs, loss_fn, target = prepare_model(args.model, n)
    model.train()
    dev, cd = state.device, option.mixed_precision
    vargs, kwargs, target = _to(vargs, dev, cd), _to(kwargs, dev, cd), _to(target, dev, cd)
    return model, vargs, kwargs, loss_fn, target


def make_runner(option, model, loss_fn, lr_kwargs):
    optimizer = torch.optim.Adam(model.parameters(), **lr_kwargs)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def exec_fn(target, *a, **k):
        loss = loss_fn(cmodel(*a, **k), target, model)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(exec_fn)
    return runner


def run_valid(args, option, state) -> int:
    """Pipelined against un-pipelined, step by step; returns the number of steps out of
    tolerance."""
    set_seed(option.bench_seed)
    model, vargs, kwargs, loss_fn, target = build(args, option, state)
    replace_batch_norm(model)           # statistics per micro-batch would be equal, dropout not
    loss_fn = RescaleLoss(loss_fn, 1 / 1000)
    lr_kwargs = dict(option.optimizer_kwargs or {})
    lr_kwargs.setdefault("lr", 1e-5)
    local = copy.deepcopy(model)
    model.to(state.device)
    local.to(state.device)
    runner = make_runner(option, model, loss_fn, lr_kwargs)
    optim = torch.optim.Adam(local.parameters(), **lr_kwargs)
    bad = 0
    for step in range(args.valid_steps):
        pipe = float(sum(l.float() for l in runner.step(target, *vargs, **kwargs)))
        a_all, k_all = split_args_kwargs((target, *vargs), kwargs, option.batch_cnt)
        optim.zero_grad()
        plain = 0.0
        for a, k in zip(a_all, k_all):
            with torch.autocast(state.device.type, dtype=option.mixed_precision,
                                enabled=option.mixed_precision is not None):
                loss = loss_fn(local(*a[1:], **k), a[0], local)
            loss.backward()
            plain += float(loss.detach())
        optim.step()
        diff = (pipe - plain) / plain * 100 if plain else 0.0
        print(f"#{step} pipe output (sum): {pipe:.8g}\n#{step} vanilla output (sum): {plain:.8g}\n"
              f"#{step} diff percentage: {diff:.3f}%", flush=True)
        if abs(diff) > args.valid_tol:
            bad += 1
    runner.close()
    return bad


def timed_steps(runner, state, target, vargs, kwargs, times: int):
    out = []
    for _ in range(times):
        if state.device.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        losses = runner.step(target, *vargs, **kwargs)
        float(torch.stack([l.float() for l in losses]).sum())      # the step's result on the host
        out.append(time.perf_counter() - t0)
    return out


def run_model(args, option, state) -> None:
    set_seed(option.bench_seed)
    model, vargs, kwargs, loss_fn, target = build(args, option, state)
    model.to(state.device)
    runner = make_runner(option, model, loss_fn, dict(option.optimizer_kwargs or {"lr": 1e-4}))
    timed_steps(runner, state, target, vargs, kwargs, 3)            # compile + warm-up
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if state.device.type == "cuda" else [])
        os.makedirs(args.result_dir, exist_ok=True)
        path = os.path.join(args.result_dir, f"trace-{args.model.replace(':', '_')}-rank{state.rank}.json.gz")
        with profile(activities=acts, record_shapes=True) as prof:
            timed_steps(runner, state, target, vargs, kwargs, 3)
        prof.export_chrome_trace(path)
        print(f"trace written to {path}", flush=True)
    else:
        if state.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats()
        times = timed_steps(runner, state, target, vargs, kwargs, args.repeat)
        mean = sum(times) / len(times)
        std = (sum((t - mean) ** 2 for t in times) / len(times)) ** 0.5
        n = option.batch_size * option.batch_cnt * state.dp_size
        print(f"mean latency {mean} / std.dev. {std} across {args.repeat} runs "
              f"({n / mean:.2f} samples/s)", flush=True)
        runner.log_memory_usage()
    runner.close()


def main() -> int:
    state = initialize_pfeife()
    parser = argparse.ArgumentParser()
    parser.add_argument("--profile", action="store_true")
    parser.add_argument("--check_valid", action="store_true")
    parser.add_argument("--valid_steps", type=int, default=6)
    parser.add_argument("--valid_tol", type=float, default=1.0, help="percent")
    parser.add_argument("--repeat", default=30, type=int, help="Repeats for timing run")
    parser.add_argument("--result_dir", default="result")
    parser.add_argument("--model", default="toy",
                        help="toy | hf_<Name> | tv:<torchvision name> | timm:<name> | a workload "
                             "of pfeife_b200.bench.workloads (vitg, vitl, llama7b, sdxl, ...)")
    PipeOption.add_arguments(parser)
    args = parser.parse_args()
    args.device_cnt = state.pp_size
    if state.device.type == "cpu":
        args.cpu = True
    option = PipeOption.from_args(args)
    if not state.is_main_rank:          # only under ``mp_launch.py --all_main``
        from pfeife_b200.runtime.partial import worker_loop
        worker_loop()
        return 0
    if args.check_valid:
        bad = run_valid(args, option, state)
        if bad:
            print(f"{bad} step(s) differ by more than {args.valid_tol}%", flush=True)
        return 1 if bad else 0
    run_model(args, option, state)
    return 0


if __name__ == "__main__":
    sys.exit(main())

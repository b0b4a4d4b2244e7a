"""Benchmark / validity driver for the single-process runtime (one thread per device).

    python benchmark_local.py --model hf_GPT2 --device_cnt 4 --batch_size 4 --batch_cnt 8
    python benchmark_local.py --model toy --device_cnt 2 --check_valid --cpu
    python benchmark_local.py --model tv:resnet50 --device_cnt 2 --memory_snapshot

The framework owns the loss here (``PipeManager(model, loss_fn, option).run(target, *inputs)``).
Counterpart of the reference's benchmark_local.py (manager API at :196-260, per-stage timing
records at :300-330, memory snapshot at :346-357); models come from ``pfeife_b200.bench.zoo``.
"""
from __future__ import annotations

import argparse
import copy
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from benchmark_mp import _to  # noqa: E402
from pfeife_b200 import PipeOption  # noqa: E402
from pfeife_b200.bench.zoo import prepare_model, replace_batch_norm  # noqa: E402
from pfeife_b200.loss import RescaleLoss  # noqa: E402
from pfeife_b200.runtime.manager import LocalPipeManager  # noqa: E402
from pfeife_b200.utils import set_seed  # noqa: E402
from pfeife_b200.utils.batch import split_args_kwargs  # noqa: E402


def build(args, option):
    n = option.batch_size * option.batch_cnt
    model, vargs, kwargs, loss_fn, target = prepare_model(args.model, n)
    model.train()
    cpu = option.cpu_test or not torch.cuda.is_available()
    first = torch.device("cpu") if cpu else torch.device(option.device_map[0])
    last = torch.device("cpu") if cpu else torch.device(option.device_map[option.device_cnt - 1])
    cd = option.mixed_precision
    # the graph is captured with the model's own tensors: they sit with the inputs (the first
    # device) until the stages are cut and every device takes its share
    model.to(first)
    return model, _to(vargs, first, cd), _to(kwargs, first, cd), loss_fn, _to(target, last, cd), last


def run_valid(args, option) -> int:
    set_seed(option.bench_seed)
    model, vargs, kwargs, loss_fn, target, last = build(args, option)
    replace_batch_norm(model)
    loss_fn = RescaleLoss(loss_fn, 1 / 1000)
    opt_kwargs = dict(option.optimizer_kwargs or {})
    opt_kwargs.setdefault("lr", 1e-5)
    local = copy.deepcopy(model).to("cpu")       # the plain loop runs on the host
    manager = LocalPipeManager(model, loss_fn, option,
                               optimizer=torch.optim.Adam(model.parameters(), **opt_kwargs))
    optim = torch.optim.Adam(local.parameters(), **opt_kwargs)
    bad = 0
    for step in range(args.valid_steps):
        pipe = float(sum(l.float().cpu() for l in manager.run(target, *vargs, **kwargs)))
        a_all, k_all = split_args_kwargs((target, *vargs), kwargs, option.batch_cnt)
        optim.zero_grad()
        plain = 0.0
        for a, k in zip(a_all, k_all):
            a, k = _to(a, torch.device("cpu")), _to(k, torch.device("cpu"))
            loss = loss_fn(local(*a[1:], **k), a[0], local)
            loss.backward()
            plain += float(loss.detach())
        optim.step()
        diff = (pipe - plain) / plain * 100 if plain else 0.0
        print(f"#{step} pipe output (sum): {pipe:.8g}\n#{step} vanilla output (sum): {plain:.8g}\n"
              f"#{step} diff percentage: {diff:.3f}%", flush=True)
        bad += abs(diff) > args.valid_tol
    manager.close()
    return bad


def run_model(args, option) -> None:
    set_seed(option.bench_seed)
    model, vargs, kwargs, loss_fn, target, last = build(args, option)
    manager = LocalPipeManager(model, loss_fn, option)
    cuda = last.type == "cuda"

    def steps(n):
        out = []
        for _ in range(n):
            if cuda:
                for d in option.device_map[:option.device_cnt]:
                    torch.cuda.synchronize(d)
            t0 = time.perf_counter()
            losses = manager.run(target, *vargs, **kwargs)
            float(torch.stack([l.float() for l in losses]).sum())
            out.append(time.perf_counter() - t0)
        return out

    steps(3)
    manager.clear_record()
    if cuda and args.memory_snapshot:
        torch.cuda.memory._record_memory_history(max_entries=100000)
    if cuda:
        for d in option.device_map[:option.device_cnt]:
            torch.cuda.reset_peak_memory_stats(d)
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if cuda else [])
        os.makedirs(args.result_dir, exist_ok=True)
        path = os.path.join(args.result_dir, f"trace-local-{args.model.replace(':', '_')}.json.gz")
        with profile(activities=acts, record_shapes=True) as prof:
            steps(3)
        prof.export_chrome_trace(path)
        print(f"trace written to {path}", flush=True)
    else:
        times = steps(args.repeat)
        mean = sum(times) / len(times)
        std = (sum((t - mean) ** 2 for t in times) / len(times)) ** 0.5
        n = option.batch_size * option.batch_cnt
        print(f"mean latency {mean} / std.dev. {std} across {args.repeat} runs "
              f"({n / mean:.2f} samples/s)", flush=True)
        for stage, (fw, bw) in sorted(manager.runner.record_times().items()):
            print(f"stage {stage}: forward {fw:.3f} ms, backward {bw:.3f} ms", flush=True)
    if cuda:
        for d in option.device_map[:option.device_cnt]:
            print(f"[Device {d}] max alloc: {torch.cuda.max_memory_allocated(d) / 2**20:.1f} MiB, "
                  f"reserved: {torch.cuda.max_memory_reserved(d) / 2**20:.1f} MiB", flush=True)
        if args.memory_snapshot:
            os.makedirs(args.result_dir, exist_ok=True)
            path = os.path.join(args.result_dir, f"memory-{args.model.replace(':', '_')}.pickle")
            torch.cuda.memory._dump_snapshot(path)
            torch.cuda.memory._record_memory_history(enabled=None)
            print(f"memory snapshot written to {path}", flush=True)
    manager.close()


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--profile", action="store_true")
    parser.add_argument("--check_valid", action="store_true")
    parser.add_argument("--memory_snapshot", action="store_true",
                        help="record the allocator history of the timed steps (CUDA only)")
    parser.add_argument("--valid_steps", type=int, default=6)
    parser.add_argument("--valid_tol", type=float, default=1.0, help="percent")
    parser.add_argument("--repeat", default=30, type=int, help="Repeats for timing run")
    parser.add_argument("--result_dir", default="result")
    parser.add_argument("--model", default="toy",
                        help="toy | hf_<Name> | tv:<torchvision name> | timm:<name> | a workload "
                             "of pfeife_b200.bench.workloads")
    PipeOption.add_arguments(parser)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        args.cpu = True
    option = PipeOption.from_args(args)
    if args.check_valid:
        bad = run_valid(args, option)
        if bad:
            print(f"{bad} step(s) differ by more than {args.valid_tol}%", flush=True)
        return 1 if bad else 0
    run_model(args, option)
    return 0


if __name__ == "__main__":
    sys.exit(main())

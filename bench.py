#!/usr/bin/env python
"""Flagship benchmark: training samples/s of ViT-g/14 (40 layers, hidden 1408, 16 heads, MLP
6144, patch 14, 224x224 images, 1000 classes, AdamW, fp16 compute with fp32 master weights,
micro-batch 24 x batch_cnt 8 per pipeline) on N GPUs of one node, driven through the public API
(``initialize_pfeife`` / ``PipeOption`` / ``PartialRunner.step`` / ``partial_compiler``).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...          # the unmodified reference, same harness

Prints ONE JSON line on the global main process.  ``value`` is whole-job samples/s from a
device-timed loop (CUDA events, barrier + synchronize on both sides, max over ranks) with the
inputs resident on the device; ``e2e.value`` repeats the measurement with every step copying
its inputs from pinned host memory and reading the loss back.  With more than one GPU the
PPxDP mesh is chosen by the planner from a profile taken on rank 0 before the process groups
are built (``--dp_mesh`` overrides; the table it chose from is reported as
``planner_mesh_table``).
Synthetic data, random-init weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# ------------------------------------------------------------------------------ shared harness
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def baseline_number():
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            pub = json.load(f).get("published") or {}
        v = pub.get("value")
        return float(v) if v else None
    except Exception:
        return None


def emit_result(args, impl, n_gpus, ms, ms_e2e, samples, clocks, launches, parallelism, h2d, d2h,
                extra=None):
    value = samples / ms * 1e3
    base = baseline_number()
    rec = {
        "metric": "train samples/sec", "value": value, "unit": "samples/s", "impl": impl,
        "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / base) if base else None,
        "dtype": "fp16", "data": "synthetic (N(0,1) images, uniform labels), random-init weights",
        "config": {"model": args.model_name, "layers": args.layers, "hidden": args.hidden,
                   "heads": args.heads, "mlp": args.mlp, "patch": args.patch,
                   "micro_batch": args.batch_size, "batch_cnt": args.batch_cnt,
                   "global_batch": samples, "seq_len": (224 // args.patch) ** 2 + 1,
                   "optimizer": "AdamW", "parallelism": parallelism,
                   "l2": "per-step working set (weights + activations, several GB) exceeds L2"},
        "clocks": clocks,
        "e2e": {"value": samples / ms_e2e * 1e3, "unit": "samples/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    if extra:
        rec.update(extra)
    print(json.dumps(rec), flush=True)


# ------------------------------------------------------------------------------ native arm
def _planned_mesh(args, cfg, world, rank, cpu):
    """The PP x DP mesh for `world` GPUs, chosen by the planner: rank 0 profiles one micro-batch
    of the model on its GPU and evaluates every factorisation of the world size; the others read
    its answer from a key-value store (the process groups do not exist yet -- they depend on
    the answer).  Falls back to pure data parallelism if planning fails on rank 0."""
    import datetime
    import torch
    import torch.distributed as dist
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    store = dist.TCPStore(host, port, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=1200))
    if rank == 0:
        mesh, table = f"-{world},1", None
        try:
            from pfeife_b200 import PipeOption
            from pfeife_b200.models.vit import ViT
            from pfeife_b200.parallel.mesh_plan import plan_mesh
            dev = torch.device("cpu") if cpu else torch.device(
                "cuda", int(os.environ.get("LOCAL_RANK", "0")))
            if not cpu:
                torch.cuda.set_device(dev)
            torch.manual_seed(0)
            model = ViT(cfg).to(dev)
            opt = PipeOption(device_cnt=1, batch_size=args.batch_size, batch_cnt=args.batch_cnt,
                             mixed_precision=None if cpu else "fp16", cpu_test=cpu,
                             no_bench_optimizer=True, verbosity="warning")
            x = torch.randn(args.batch_size, 3, 224, 224, device=dev,
                            dtype=torch.float32 if cpu else torch.float16)
            choice = plan_mesh(model, (x,), opt, world, dev)
            mesh = choice.dp_mesh
            table = [{"pp": a, "dp": b, "step_ms": round(c, 2), "samples_per_s": round(d, 1),
                      "fits": bool(e)} for a, b, c, d, e in choice.table]
            del model, choice, x
            if not cpu:
                torch.cuda.empty_cache()
        except Exception as exc:   # planning must never take the benchmark down
            print(f"[bench] mesh planning failed ({type(exc).__name__}: {exc}); "
                  f"using pure data parallelism", file=sys.stderr, flush=True)
        store.set("mesh", json.dumps({"mesh": mesh, "table": table}))
    got = json.loads(store.get("mesh").decode())
    # every rank has read the answer before rank 0 (the store's server) moves on
    store.add("mesh_read", 1)
    if rank == 0:
        deadline = time.time() + 600
        while int(store.add("mesh_read", 0)) < world and time.time() < deadline:
            time.sleep(0.05)
    return got["mesh"], got["table"]


def run_native(args) -> int:
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, partial_compiler
    from pfeife_b200 import ops
    from pfeife_b200.models.vit import ViT, ViTConfig
    from pfeife_b200.ops import _lib
    from pfeife_b200.runtime.partial import worker_loop
    from pfeife_b200.utils import get_logger, set_logger_level

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cpu = args.cpu or not torch.cuda.is_available()
    set_logger_level(20 if args.verbose else 30)

    cfg = ViTConfig(image_size=224, patch_size=args.patch, hidden_size=args.hidden,
                    num_layers=args.layers, num_heads=args.heads, mlp_dim=args.mlp,
                    num_classes=1000)
    dp_mesh = args.dp_mesh
    planned = None
    if dp_mesh in (None, "auto") and world > 1:
        dp_mesh, planned = _planned_mesh(args, cfg, world, rank, cpu)
    state = initialize_pfeife(dp_mesh=dp_mesh, cpu=cpu)
    dev = state.device
    mp = None if cpu else "fp16"
    option = PipeOption(device_cnt=state.pp_size, batch_size=args.batch_size,
                        batch_cnt=args.batch_cnt, mixed_precision=mp, cpu_test=cpu,
                        no_bench_optimizer=True, optimizer={"type": "adamw", "lr": 1e-4},
                        fused_dp=not args.nccl_dp, cuda_graphs=not args.no_graphs, verbosity="info" if args.verbose else "warning")
    if not state.is_main_rank:
        worker_loop()
        return 0

    torch.manual_seed(0)
    model = ViT(cfg).to(dev)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def exec_fn(pixel_values, labels):
        logits = cmodel(pixel_values)
        loss = ops.cross_entropy(logits, labels)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(exec_fn)
    n = args.batch_size * args.batch_cnt
    g = torch.Generator(device="cpu").manual_seed(1 + state.dp_rank)
    host_x = torch.randn(n, 3, 224, 224, generator=g)
    host_y = torch.randint(0, 1000, (n,), generator=g)
    if not cpu:
        host_x, host_y = host_x.pin_memory(), host_y.pin_memory()
        host_x16 = host_x.to(torch.float16).pin_memory()
    else:
        host_x16 = host_x
    x_dev, y_dev = host_x16.to(dev), host_y.to(dev)

    def one_step(e2e: bool):
        if e2e:
            x = host_x16.to(dev, non_blocking=True)
            y = host_y.to(dev, non_blocking=True)
        else:
            x, y = x_dev, y_dev
        losses = runner.step(x, y)
        if e2e:
            return float(torch.stack([l.float() for l in losses]).sum().cpu())
        return losses

    def sync():
        if not cpu:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if not cpu:
                torch.cuda.synchronize()

    def timed(e2e: bool) -> float:
        sync()
        if cpu:
            t0 = time.perf_counter()
            for _ in range(args.steps):
                one_step(e2e)
            ms = (time.perf_counter() - t0) * 1e3 / args.steps
        else:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(args.steps):
                one_step(e2e)
            e.record()
            sync()
            ms = s.elapsed_time(e) / args.steps
        if world > 1:   # max over ranks
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    for _ in range(max(args.warmup, 1)):
        one_step(False)
    sampler = ClockSampler(dev.index or 0)
    if state.is_main_process and not cpu:
        sampler.start()
    l0 = _lib.launch_count()
    ms = timed(False)
    launches = _lib.launch_count() - l0
    ms_e2e = timed(True)
    clocks = sampler.stop() if (state.is_main_process and not cpu) else None
    if not cpu:
        from pfeife_b200.ops import kernels as kx
        kx.check_status()
    bubble = 0.0
    for m in runner.modules:
        if m.plan is not None and m.plan.sim is not None:
            bubble = m.plan.sim.bubble_fraction
    if state.is_main_process:
        samples = n * state.dp_size
        emit_result(args, impl="pfeife_b200", n_gpus=world, ms=ms, ms_e2e=ms_e2e, samples=samples,
                    clocks=clocks, launches=launches,
                    parallelism=f"pp{state.pp_size}xdp{state.dp_size}",
                    h2d=host_x16.numel() * host_x16.element_size() + host_y.numel() * 8, d2h=4,
                    extra={"dp_impl": ("fused_p2p" if option.fused_dp else "nccl")
                           if state.dp_size > 1 else None,
                           "planner_mesh_table": planned,
                           "optimizer_and_dp_exposed_ms": runner.worker.last_optimizer_ms(),
                           "pipeline_bubble_pct": 100.0 * bubble})
    runner.close()
    if world > 1:
        dist.barrier()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--dp_mesh", type=str, default=None)
    ap.add_argument("--nccl_dp", action="store_true", help="NCCL all-reduce DP baseline")
    ap.add_argument("--no_graphs", action="store_true",
                    help="run stages eagerly instead of replaying captured CUDA graphs")
    ap.add_argument("--cpu", action="store_true", help="plumbing check without a GPU")
    ap.add_argument("--verbose", action="store_true")
    # model shape (defaults: ViT-g/14 of the headline configuration)
    ap.add_argument("--model_name", default="ViT-g/14")
    ap.add_argument("--layers", type=int, default=40)
    ap.add_argument("--hidden", type=int, default=1408)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--mlp", type=int, default=6144)
    ap.add_argument("--patch", type=int, default=14)
    ap.add_argument("--batch_size", type=int, default=24)
    ap.add_argument("--batch_cnt", type=int, default=8)
    args = ap.parse_args(argv)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        try:
            return reference_arm.run(args)
        except SystemExit:
            raise
        except BaseException as e:   # the arm must always print a line and exit 0
            import traceback
            traceback.print_exc()
            return reference_arm.unavailable(f"{type(e).__name__}: {e}")
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())

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
its inputs from pinned host memory (prefetched one step ahead on a side stream, as a data
loader would) and reading the loss back.  With more than one GPU the
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
                extra=None, workload=None):
    value = samples / ms * 1e3
    base = baseline_number()
    if workload is not None:
        config = {"model": workload.model_name, **workload.config,
                  "micro_batch": workload.micro_batch, "batch_cnt": workload.batch_cnt}
        dtype, data = workload.precision or "fp32", workload.data
    else:
        config = {"model": args.model_name, "layers": args.layers, "hidden": args.hidden,
                  "heads": args.heads, "mlp": args.mlp, "patch": args.patch,
                  "micro_batch": args.batch_size, "batch_cnt": args.batch_cnt,
                  "seq_len": (224 // args.patch) ** 2 + 1, "optimizer": "AdamW"}
        dtype, data = "fp16", "synthetic (N(0,1) images, uniform labels), random-init weights"
    config.update({"global_batch": samples, "parallelism": parallelism,
                   "l2": "per-step working set (weights + activations, several GB) exceeds L2"})
    rec = {
        "metric": "train samples/sec", "value": value, "unit": "samples/s", "impl": impl,
        "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / base) if base else None,
        "dtype": dtype, "data": data,
        "config": config,
        "clocks": clocks,
        "e2e": {"value": samples / ms_e2e * 1e3, "unit": "samples/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    if extra:
        rec.update(extra)
    print(json.dumps(rec), flush=True)


# ------------------------------------------------------------------------------ native arm
def _compute_dtype(torch, precision):
    return {"fp16": torch.float16, "bf16": torch.bfloat16}.get(precision, torch.float32)


def _to_compute(t, dtype):
    return t.to(dtype) if t.is_floating_point() else t


def _planned_mesh(args, wl, world, rank, cpu):
    """The PP x DP mesh for `world` GPUs, chosen by the planner.  The job's default process
    group is created first and two of its ranks measure the link (latency and bandwidth of
    point-to-point transfers, the ``--device_bench`` measurement); rank 0 then profiles one
    micro-batch of the model on its GPU, evaluates every factorisation of the world size with
    the measured link and broadcasts its choice.  Falls back to pure data parallelism if
    planning fails on rank 0."""
    import datetime
    import torch
    import torch.distributed as dist
    from pfeife_b200.parallel.device_bench import NCCLDeviceBench
    dev = torch.device("cpu") if cpu else torch.device(
        "cuda", int(os.environ.get("LOCAL_RANK", "0")) % max(1, torch.cuda.device_count()))
    if not cpu:
        torch.cuda.set_device(dev)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "24446")
        kw = {} if cpu else {"device_id": dev}
        dist.init_process_group("gloo" if cpu else "nccl", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=1800), **kw)
    link = None
    if not cpu:
        bench = NCCLDeviceBench(rank, list(range(world)), dev, dist.group.WORLD)
        bench.run_bench(args.device_bench, uniform=True)
        if bench.params:
            link = tuple(float(v) for v in next(iter(bench.params.values())))
    box = [None]
    if rank == 0:
        mesh, table, pred = f"-{world},1", None, None
        try:
            from pfeife_b200 import PipeOption
            from pfeife_b200.parallel.mesh_plan import NVSWITCH_LINK, plan_mesh
            torch.manual_seed(0)
            with torch.device(dev):
                model = wl.build_model()
            model = model.to(dev)
            extra = {k: v for k, v in wl.option.items() if k in ("prefetch_fwd", "loop_batch")}
            opt = PipeOption(device_cnt=1, batch_size=wl.micro_batch, batch_cnt=wl.batch_cnt,
                             mixed_precision=None if cpu else wl.precision, cpu_test=cpu,
                             no_bench_optimizer=True, verbosity="warning",
                             cuda_graphs=not (cpu or args.no_graphs), **extra)
            cd = _compute_dtype(torch, None if cpu else wl.precision)
            mb = wl.make_batch(wl.micro_batch, torch.Generator().manual_seed(0))
            x = tuple(_to_compute(t, cd).to(dev) for t in mb[:wl.n_model_inputs])
            choice = plan_mesh(model, x, opt, world, dev, link=link or NVSWITCH_LINK)
            mesh = choice.dp_mesh
            # a pure data-parallel layout within 2 % of the best prediction wins the tie (no
            # stage hand-offs, no bubble: fewer things that the cost model leaves out)
            dp_only = [row for row in choice.table if row[0] == 1 and row[4]]
            if dp_only and dp_only[0][3] >= 0.98 * choice.samples_per_s:
                mesh = f"-{world},1"
            table = [{"pp": a, "dp": b, "step_ms": round(c, 2), "samples_per_s": round(d, 1),
                      "fits": bool(e)} for a, b, c, d, e in choice.table]
            del model, choice, x, mb
            if not cpu:
                torch.cuda.empty_cache()
        except Exception as exc:   # planning must never take the benchmark down
            print(f"[bench] mesh planning failed ({type(exc).__name__}: {exc}); "
                  f"using pure data parallelism", file=sys.stderr, flush=True)
        box = [{"mesh": mesh, "table": table}]
    dist.broadcast_object_list(box, src=0)
    got = box[0]
    got["link"] = None if link is None else {
        "latency_ms": round(link[0], 4), "gb_per_s": round((1 << 20) / 1e9 / (link[1] / 1e3), 1)
        if link[1] > 0 else None}
    return got["mesh"], got


def _predicted_ms(table, pp, dp):
    for row in table or []:
        if row["pp"] == pp and row["dp"] == dp:
            return row["step_ms"]
    return None


def run_native(args) -> int:
    import torch
    import torch.distributed as dist

    from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, partial_compiler
    from pfeife_b200.bench.workloads import get_workload
    from pfeife_b200.ops import _lib
    from pfeife_b200.runtime.partial import worker_loop
    from pfeife_b200.utils import set_logger_level

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cpu = args.cpu or not torch.cuda.is_available()
    set_logger_level(20 if args.verbose else 30)

    wl = get_workload(args.workload, args)
    dp_mesh = args.dp_mesh
    planned = None
    if dp_mesh is None and world == 8 and wl.mesh_for_8:
        dp_mesh = wl.mesh_for_8             # the layout the configuration names
    if dp_mesh in (None, "auto") and world > 1:
        dp_mesh, planned = _planned_mesh(args, wl, world, rank, cpu)
    state = initialize_pfeife(dp_mesh=dp_mesh, cpu=cpu)
    dev = state.device
    mp = None if cpu else wl.precision
    extra_opt = dict(wl.option)
    for k in ("loop_cnt", "loop_batch", "prefetch_fwd", "split_points", "scheduler",
              "schedule_picture"):
        if getattr(args, k, None) is not None:
            extra_opt[k] = getattr(args, k)
    if state.pp_size == 1:
        for k in ("loop_cnt", "loop_batch", "prefetch_fwd"):
            extra_opt.pop(k, None)
    if args.use_fsdp:
        extra_opt["use_fsdp"] = True
    option = PipeOption(device_cnt=state.pp_size, batch_size=wl.micro_batch,
                        batch_cnt=wl.batch_cnt, mixed_precision=mp, cpu_test=cpu,
                        no_bench_optimizer=True, optimizer={"type": "adamw", "lr": 1e-4},
                        fused_dp=not args.nccl_dp, cuda_graphs=not args.no_graphs,
                        device_bench=args.device_bench,
                        verbosity="info" if args.verbose else "warning", **extra_opt)
    if not state.is_main_rank:
        worker_loop()
        if world > 1:
            dist.barrier()      # the job ends together (the main ranks wait here after closing)
        return 0

    torch.manual_seed(0)
    with torch.device(dev):     # initialised on the device: seconds instead of minutes at 7B
        model = wl.build_model()
    model = model.to(dev)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def exec_fn(*batch):
        loss = wl.loss(cmodel, *batch)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(exec_fn)
    n = wl.micro_batch * wl.batch_cnt
    g = torch.Generator(device="cpu").manual_seed(args.data_seed + 1 + state.dp_rank)
    cd = _compute_dtype(torch, mp)
    # the host holds what a data loader would hand over: fp32 tensors in pinned memory
    host = list(wl.make_batch(n, g))
    if not cpu:
        host = [t.pin_memory() for t in host]

    def to_compute(t):
        if not t.is_floating_point() or t.dtype == cd:
            return t
        if t.is_cuda and cd in (torch.float16, torch.bfloat16):
            from pfeife_b200.ops import kernels as kx
            return kx.cast(t, cd)
        return t.to(cd)

    resident = [to_compute(t.to(dev)) for t in host]

    # End-to-end steps read their inputs from pinned host memory and bring the loss back.  Like
    # a prefetching data loader, the copy of step i+1's inputs is issued on a side stream
    # before step i is launched, so it travels while step i computes; every step still makes
    # its own host-to-device copy inside the timed region, followed by the cast to the compute
    # dtype on the device.  The reference arm loads its inputs the same way.
    copy_stream = None if cpu else torch.cuda.Stream(device=dev)
    pending = []
    last_loss = [None]

    def fetch():
        if cpu:
            return list(host), None
        with torch.cuda.stream(copy_stream):
            batch = [t.to(dev, non_blocking=True) for t in host]
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return batch, ev

    def one_step(e2e: bool, last: bool = False):
        if not e2e:
            last_loss[0] = runner.step(*resident)   # read back after the timed region
            return 0.0
        batch, ev = pending.pop() if pending else fetch()
        if not last:
            pending.append(fetch())
        if ev is not None:
            torch.cuda.current_stream(dev).wait_event(ev)
            for t in batch:
                t.record_stream(torch.cuda.current_stream(dev))
        losses = runner.step(*[to_compute(t) for t in batch])
        last_loss[0] = losses
        return float(torch.stack([l.float() for l in losses]).sum().cpu())

    def sync():
        """Every rank of the job is idle: the other ranks of this pipeline answer a control
        round trip after synchronising their devices, and the pipelines' main ranks (one
        data-parallel group) meet at a barrier."""
        if state.pp_size > 1:
            runner.time_report(reset=False)
        if not cpu:
            torch.cuda.synchronize()
        if state.dp_size > 1:
            dist.barrier(group=state.dp_group)
            if not cpu:
                torch.cuda.synchronize()

    def timed(e2e: bool) -> float:
        sync()
        if cpu:
            t0 = time.perf_counter()
            for i in range(args.steps):
                one_step(e2e, last=(i == args.steps - 1))
            ms = (time.perf_counter() - t0) * 1e3 / args.steps
        else:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(args.steps):
                one_step(e2e, last=(i == args.steps - 1))
            if state.pp_size > 1:
                # the earlier stages finish a step after the last one: the timed region ends
                # when every rank of the pipeline has finished its work
                runner.time_report(reset=False)
            e.record()
            sync()
            ms = s.elapsed_time(e) / args.steps
        if world > 1:   # max over the ranks that time (the main rank of every pipeline)
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=state.dp_group) \
                if state.dp_size > 1 else None
            ms = float(t)
        return ms

    for _ in range(max(args.warmup, 1)):
        one_step(False)
    runner.time_report(reset=True)          # per-stage event records restart with the timed steps
    sampler = ClockSampler(dev.index or 0)
    if state.is_main_process and not cpu:
        sampler.start()
    if not cpu:
        torch.cuda.profiler.start()         # capture range for an external profiler
    l0 = _lib.launch_count()
    ms = timed(False)
    launches = _lib.launch_count() - l0
    if not cpu:
        torch.cuda.profiler.stop()
    bubble = runner.bubble_report(ms)
    # the end-to-end path has first-use costs of its own (copy stream, staging buffers of the
    # allocator): warm it up as well
    for _ in range(min(max(args.warmup, 1), 2)):
        one_step(True, last=True)
    ms_e2e = timed(True)
    clocks = sampler.stop() if (state.is_main_process and not cpu) else None
    if not cpu:
        from pfeife_b200.ops import kernels as kx
        kx.check_status()
    sim_bubble, predicted = 0.0, None
    for m in runner.modules:
        if m.plan is not None and m.plan.sim is not None:
            sim_bubble = m.plan.sim.bubble_fraction
            predicted = m.plan.time
    # every pipeline's main rank reports its own bubble; the line carries the worst pipeline
    if state.dp_size > 1:
        allb = [None] * state.dp_size
        dist.all_gather_object(allb, bubble, group=state.ctrl_dp)
        bubble = max(allb, key=lambda b: b["max_pct"])
    if state.is_main_process:
        samples = n * state.dp_size
        table = (planned or {}).get("table")
        pred_mesh = _predicted_ms(table, state.pp_size, state.dp_size)
        emit_result(args, impl="pfeife_b200", n_gpus=world, ms=ms, ms_e2e=ms_e2e, samples=samples,
                    clocks=clocks, launches=launches,
                    parallelism=f"pp{state.pp_size}xdp{state.dp_size}",
                    h2d=sum(t.numel() * t.element_size() for t in host), d2h=4, workload=wl,
                    extra={"loss_mean_last_step": (None if last_loss[0] is None else float(
                               torch.stack([l.float() for l in last_loss[0]]).mean().cpu())),
                           "dp_impl": ("fused_p2p" if option.fused_dp else "nccl")
                           if state.dp_size > 1 else None,
                           "planner_mesh_table": table,
                           "planner_link": (planned or {}).get("link"),
                           "planner_predicted_step_ms": pred_mesh if pred_mesh is not None
                           else predicted,
                           "planner_error_pct": None if not (pred_mesh or predicted) else round(
                               100.0 * ((pred_mesh or predicted) - ms) / ms, 2),
                           "use_fsdp": bool(option.use_fsdp),
                           "optimizer_and_dp_exposed_ms": runner.worker.last_optimizer_ms(),
                           "dp_phases_ms": runner.worker.dp.phase_ms()
                           if getattr(runner.worker.dp, "fused", False) else None,
                           "pipeline_bubble_pct": bubble["max_pct"],
                           "pipeline_bubble_mean_pct": bubble["mean_pct"],
                           "pipeline_bubble_simulated_pct": 100.0 * sim_bubble,
                           "per_rank": [{k: (round(v, 3) if isinstance(v, float) else v)
                                         for k, v in r.items()} for r in bubble["per_rank"]]})
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
    ap.add_argument("--use_fsdp", action="store_true",
                    help="keep weight matrices row-sharded between optimizer steps; the first "
                         "GEMM that reads one gathers the other ranks' rows (needs DP > 1)")
    ap.add_argument("--loop_cnt", type=int, default=None, help="stages per pipeline rank")
    ap.add_argument("--loop_batch", type=int, default=None)
    ap.add_argument("--prefetch_fwd", type=int, default=None)
    ap.add_argument("--scheduler", type=str, default=None)
    ap.add_argument("--device_bench", type=str, default=None,
                    help="link-model file (measured and written when it does not exist)")
    ap.add_argument("--schedule_picture", type=str, default=None,
                    help="write the planned schedule as an SVG chart to FILE")
    ap.add_argument("--data_seed", type=int, default=0,
                    help="offset of the synthetic batch's seed (replica r draws with seed + 1 + r)")
    ap.add_argument("--cpu", action="store_true", help="plumbing check without a GPU")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--workload", default="vitg",
                    help="vitg (headline, default) | vitl | llama7b | llama7b_fsdp | sdxl | "
                         "vit_tiny | llama_tiny | unet_tiny; on 8 GPUs a workload runs on the "
                         "mesh its configuration names unless --dp_mesh is given")
    # shape of the vitg workload (defaults: ViT-g/14 of the headline configuration)
    ap.add_argument("--model_name", default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=None)
    ap.add_argument("--heads", type=int, default=None)
    ap.add_argument("--mlp", type=int, default=None)
    ap.add_argument("--patch", type=int, default=None)
    ap.add_argument("--batch_size", type=int, default=None)
    ap.add_argument("--batch_cnt", type=int, default=None)
    args = ap.parse_args(argv)
    if args.impl == "reference":
        # the reference arm runs the headline configuration (or the shape given on the command
        # line) of the ViT workload
        for k, v in (("model_name", "ViT-g/14"), ("layers", 40), ("hidden", 1408), ("heads", 16),
                     ("mlp", 6144), ("patch", 14), ("batch_size", 24), ("batch_cnt", 8)):
            if getattr(args, k) is None:
                setattr(args, k, v)
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

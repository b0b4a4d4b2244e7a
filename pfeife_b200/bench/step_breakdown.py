"""Where a training step's device time goes: runs a benchmark workload on one GPU through the
public API, records ONE steady-state step with ``torch.profiler`` (kernel activity only) and
prints the kernels grouped by name with their share of the step.

    python -m pfeife_b200.bench.step_breakdown --workload vitg [--top 30] [--out FILE]

Times under a profiler are a little longer than unprofiled ones: read the SHARES; the step time
to quote is ``bench.py``'s.
"""
from __future__ import annotations

import argparse
import collections
import json
import re
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--workload", default="vitg")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--out", default=None, help="also write the table as JSON lines here")
    for k in ("layers", "hidden", "heads", "mlp", "patch", "batch_size", "batch_cnt"):
        ap.add_argument(f"--{k}", type=int, default=None)
    ap.add_argument("--model_name", default=None)
    ap.add_argument("--no_graphs", action="store_true")
    args = ap.parse_args(argv)

    import torch
    from torch.profiler import ProfilerActivity, profile

    from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, partial_compiler
    from pfeife_b200.bench.workloads import get_workload
    from pfeife_b200.utils import set_logger_level

    set_logger_level(30)
    wl = get_workload(args.workload, args)
    state = initialize_pfeife(dp_mesh=None)
    dev = state.device
    option = PipeOption(device_cnt=1, batch_size=wl.micro_batch, batch_cnt=wl.batch_cnt,
                        mixed_precision=wl.precision, no_bench_optimizer=True,
                        optimizer={"type": "adamw", "lr": 1e-4}, cuda_graphs=not args.no_graphs,
                        verbosity="warning")
    torch.manual_seed(0)
    model = wl.build_model().to(dev)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)

    def exec_fn(*batch):
        loss = wl.loss(cmodel, *batch)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(exec_fn)
    cd = {"fp16": torch.float16, "bf16": torch.bfloat16}.get(wl.precision, torch.float32)
    g = torch.Generator().manual_seed(1)
    batch = [t.to(dev).to(cd) if t.is_floating_point() else t.to(dev)
             for t in wl.make_batch(wl.micro_batch * wl.batch_cnt, g)]
    for _ in range(max(args.warmup, 3)):
        runner.step(*batch)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        s.record()
        runner.step(*batch)
        e.record()
        torch.cuda.synchronize()
    step_ms = s.elapsed_time(e)
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        dur = getattr(ev, "device_time_total", 0) or getattr(ev, "cuda_time_total", 0)
        if dur <= 0:
            continue
        name = re.sub(r"<.*", "", ev.name)          # template arguments off
        name = re.sub(r"^void\s+", "", name)
        agg[name][0] += 1
        agg[name][1] += dur / 1e3
    rows = sorted(agg.items(), key=lambda kv: -kv[1][1])
    total = sum(v[1] for v in agg.values())
    print(f"workload {wl.name}: step {step_ms:.2f} ms under the profiler, kernels sum "
          f"{total:.2f} ms")
    print(f"{'kernel':60s} {'calls':>7s} {'ms':>9s} {'share':>7s}")
    out = []
    for name, (calls, ms) in rows[:args.top]:
        print(f"{name[:60]:60s} {calls:7d} {ms:9.3f} {100.0 * ms / total:6.2f}%")
        out.append({"kernel": name, "calls": calls, "ms": round(ms, 3),
                    "share_pct": round(100.0 * ms / total, 2)})
    if args.out:
        with open(args.out, "w") as f:
            f.write(json.dumps({"workload": wl.name, "step_ms": step_ms, "kernel_ms": total}) + "\n")
            for r in out:
                f.write(json.dumps(r) + "\n")
    runner.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Reference arm of bench.py: runs the UNMODIFIED reference package installed under
``baseline/_ref`` through its own public API (``initialize_pfeife``, ``PipeOption``,
``PartialRunner``, ``partial_compiler``) and its stock worker / planner / NCCL code path, on
the benchmark's model shape with synthetic data.  None of this framework's models, kernels or
runtime is imported here.

Environment shims, all outside the reference's sources: (1) torch 2.11 lifts parameters to
graph inputs, which silently disables the reference's pipelining, so
``torch._dynamo.config.inline_inbuilt_nn_modules`` is switched off to give it the
``call_module`` graphs it was written for; (2) an import stand-in for matplotlib; (3) the
model is HuggingFace ``ViTForImageClassification`` built from a config (random weights), as in
the reference's own ViT trainer.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def unavailable(reason: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}),
          flush=True)
    return 0


def _candidate_meshes(world: int):
    """The reference's own mesh options for `world` GPUs (its ``--dp_mesh``), most promising
    first: data-parallel replicas of short pipelines, then one pipeline over everything.  It has
    no single-stage mode (its planner raises with one device), so pure data parallelism is not
    among them."""
    meshes = []
    pp = 2
    while pp < world:
        if world % pp == 0:
            meshes.append(f"-{world // pp},{pp}")
        pp *= 2
    meshes.append(str(world))
    return meshes


def _mesh_name(mesh: str) -> str:
    parts = [int(v) for v in mesh.split(",")]
    if len(parts) == 1:
        return f"pp{parts[0]}"
    dp = -min(parts)
    return f"pp{max(parts)}xdp{dp}"


def run(args) -> int:
    """Parent of the arm (one per rank the launcher started): runs the reference once per mesh
    in child processes with ``DP_MESH`` set as its launcher would set it, and reports the
    reference's BEST mesh, listing all of them.  The children are the processes that touch the
    GPUs."""
    if os.environ.get("PFEIFE_REF_CHILD"):
        return run_one(args)
    ref_root = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_root, "pfeife")):
        return unavailable("baseline/_ref is not installed")
    import subprocess
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    time_limit = float(os.environ.get("PFEIFE_REF_TIMEOUT", "780"))
    t_begin = time.time()
    base_port = int(os.environ.get("MASTER_PORT", "24446"))
    forced = os.environ.get("PFEIFE_REF_MESH")
    meshes = [forced] if forced else _candidate_meshes(world)
    tag = f"/tmp/pfeife_ref_{base_port}_{os.getppid() if world > 1 else os.getpid()}"
    if world > 1:
        tag = f"/tmp/pfeife_ref_{base_port}"
    root = os.path.dirname(HERE)
    results = []
    for i, mesh in enumerate(meshes):
        left = time_limit - (time.time() - t_begin)
        share = left / (len(meshes) - i)
        if share < 60:
            results.append({"mesh": _mesh_name(mesh), "unavailable": "no time left in the arm"})
            continue
        out = f"{tag}_{i}"
        for r in range(world):
            try:
                os.remove(f"{out}.{r}")
            except OSError:
                pass
        env = dict(os.environ, PFEIFE_REF_CHILD="1", DP_MESH=mesh, PFEIFE_REF_OUT=out,
                   MASTER_PORT=str(base_port + 101 + i), PFEIFE_REF_LIMIT=str(share - 15))
        # the children rendezvous on a port of their own, where no launcher agent serves a
        # store: without these variables rank 0 of the child job creates it, as under the
        # reference's own launcher
        for k in [k for k in env if k.startswith("TORCHELASTIC_") or k.startswith("TORCH_NCCL_ASYNC")]:
            env.pop(k, None)
        cmd = [sys.executable, os.path.join(root, "bench.py"), "--impl", "reference",
               "--gpus", str(world), "--steps", str(args.steps), "--warmup", str(args.warmup),
               "--layers", str(args.layers), "--hidden", str(args.hidden), "--heads",
               str(args.heads), "--mlp", str(args.mlp), "--patch", str(args.patch),
               "--batch_size", str(args.batch_size), "--batch_cnt", str(args.batch_cnt)]
        log = open(f"{out}.log.{rank}", "w")
        proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, cwd=root,
                                start_new_session=True)
        try:
            proc.wait(timeout=share)
        except subprocess.TimeoutExpired:
            try:
                os.killpg(proc.pid, 9)      # the process group this arm started, nothing else
            except OSError:
                pass
            proc.wait()
        log.close()
        if rank != 0:
            continue
        # the main rank of every pipeline of the child job wrote one record
        recs = []
        deadline = time.time() + 20
        while time.time() < deadline:
            recs = []
            for r in range(world):
                try:
                    with open(f"{out}.{r}") as f:
                        recs.append(json.load(f))
                except (OSError, ValueError):
                    pass
            if recs and len(recs) >= recs[0].get("dp", 1):
                break
            time.sleep(0.5)
        if not recs or "ms" not in recs[0]:
            why = recs[0].get("unavailable") if recs else None
            if why is None:
                try:
                    with open(f"{out}.log.0") as f:
                        tail = [ln.strip() for ln in f.read().splitlines() if ln.strip()]
                    why = tail[-1][:200] if tail else "no output"
                except OSError:
                    why = "no output"
            results.append({"mesh": _mesh_name(mesh), "unavailable": why})
            continue
        dp = recs[0]["dp"]
        ms = max(r["ms"] for r in recs)
        ms_e2e = max(r["ms_e2e"] for r in recs)
        n = recs[0]["samples"] * dp
        clocks = next((r["clocks"] for r in recs if r.get("clocks")), None)
        results.append({"mesh": _mesh_name(mesh), "samples_per_s": n / ms * 1e3,
                        "e2e_samples_per_s": n / ms_e2e * 1e3, "ms_per_step": ms,
                        "ms_e2e": ms_e2e, "samples": n, "clocks": clocks,
                        "h2d": recs[0]["h2d"]})
    if rank != 0:
        return 0
    ok = [r for r in results if "samples_per_s" in r]
    if not ok:
        why = "; ".join(f"{r['mesh']}: {r.get('unavailable')}" for r in results)
        return unavailable(why or "no mesh ran")
    best = max(ok, key=lambda r: r["e2e_samples_per_s"])
    import bench as harness
    listing = [{k: (round(v, 2) if isinstance(v, float) else v) for k, v in r.items()
                if k in ("mesh", "samples_per_s", "e2e_samples_per_s", "ms_per_step",
                         "unavailable")} for r in results]
    harness.emit_result(args, impl="reference", n_gpus=world, ms=best["ms_per_step"],
                        ms_e2e=best["ms_e2e"], samples=best["samples"], clocks=best["clocks"],
                        launches=None, parallelism=best["mesh"], h2d=best["h2d"], d2h=4,
                        extra={"reference_meshes": listing})
    return 0


def _write(rec) -> None:
    out = os.environ.get("PFEIFE_REF_OUT")
    if out:
        with open(f"{out}.{os.environ.get('RANK', '0')}.tmp", "w") as f:
            json.dump(rec, f)
        os.replace(f"{out}.{os.environ.get('RANK', '0')}.tmp",
                   f"{out}.{os.environ.get('RANK', '0')}")


def _start_watchdog(rank: int) -> None:
    """The reference profiles every graph node before its first step, which at full size can
    take minutes; past the limit the parent gave this mesh (PFEIFE_REF_LIMIT seconds) every rank
    leaves and the mesh is reported as unavailable instead of running into the caller's own
    time limit without a line."""
    import threading
    limit = float(os.environ.get("PFEIFE_REF_LIMIT", "1500"))

    def fire():
        _write({"unavailable": f"the reference did not finish profiling and its steps in "
                               f"{limit:.0f} s (its node-by-node profiling pass dominates)"})
        os._exit(0)

    t = threading.Timer(limit, fire)
    t.daemon = True
    t.start()


def run_one(args) -> int:
    """One run of the reference on the mesh in ``DP_MESH`` (child process, one per rank)."""
    ref_root = os.path.join(HERE, "_ref")
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    import bench as harness   # timing / reporting helpers only (standard library code)
    # the reference package must win over this repository's compatibility package `pfeife`
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(HERE)]
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, ref_root)
    for k in [k for k in sys.modules if k == "pfeife" or k.startswith("pfeife.")]:
        del sys.modules[k]

    import torch
    if not torch.cuda.is_available():
        _write({"unavailable": "no CUDA device"})
        return 0
    import torch._dynamo
    torch._dynamo.config.inline_inbuilt_nn_modules = False

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    _start_watchdog(rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "24446")
    os.environ.setdefault("LOCAL_RANK", str(rank))
    try:
        from pfeife.mp import initialize_pfeife, PartialRunner, partial_compiler
        from pfeife.mp.worker import ProcessWorker
        from pfeife.option import PipeOption
        import pfeife
        assert os.path.abspath(pfeife.__file__).startswith(ref_root), pfeife.__file__
    except Exception as e:  # import problems are reported, not raised
        _write({"unavailable": f"reference import failed: {type(e).__name__}: {e}"})
        return 0

    try:
        return _run_reference(args, harness, torch, initialize_pfeife, PartialRunner,
                              partial_compiler, ProcessWorker, PipeOption, world, rank)
    except BaseException as e:      # e.g. its planner's IndexError with one device
        import traceback
        traceback.print_exc()
        _write({"unavailable": f"{type(e).__name__}: {e}"[:300]})
        sys.stdout.flush()
        os._exit(0)


def _run_reference(args, harness, torch, initialize_pfeife, PartialRunner, partial_compiler,
                   ProcessWorker, PipeOption, world, rank) -> int:
    state = initialize_pfeife()      # reads DP_MESH, as under the reference's launcher
    dev = state.device
    if not state.is_main_rank:
        # stock worker body of the reference launcher (mp_launch.py:157-172)
        worker = ProcessWorker()
        worker.wait_for_init()
        worker.run_loop()
        return 0

    from transformers import ViTConfig, ViTForImageClassification
    cfg = ViTConfig(hidden_size=args.hidden, num_hidden_layers=args.layers,
                    num_attention_heads=args.heads, intermediate_size=args.mlp,
                    image_size=224, patch_size=args.patch, num_labels=1000,
                    hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    model = ViTForImageClassification(cfg).to(dev)
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    mesh_tag = os.environ.get("DP_MESH", str(world)).replace(",", "_")
    option = PipeOption(device_cnt=state.pp_size, batch_size=args.batch_size,
                        batch_cnt=args.batch_cnt, mixed_precision="fp16",
                        optimizer={"type": "adamw", "lr": 1e-4}, no_bench_optimizer=True,
                        verbosity="info",
                        device_bench=os.path.join("/tmp", f"pfeife_ref_dev{mesh_tag}.bench"))
    runner = PartialRunner(option, optimizer)
    cmodel = torch.compile(model, backend=partial_compiler)
    scaler = torch.GradScaler(enabled=True)
    criterion = torch.nn.CrossEntropyLoss()

    def exec_fn(pixel_values, labels):
        with torch.autocast(dtype=torch.float16, device_type="cuda"):
            logits = cmodel(pixel_values=pixel_values).logits
            loss = criterion(logits.view(-1, 1000).float(), labels)
        scaler.scale(loss).backward()
        return loss

    runner.set_exec_fn(exec_fn)
    n = args.batch_size * args.batch_cnt
    g = torch.Generator(device="cpu").manual_seed(1 + state.rank)
    host = [torch.randn(n, 3, 224, 224, generator=g).pin_memory(),
            torch.randint(0, 1000, (n,), generator=g).pin_memory()]
    resident = [t.to(dev) for t in host]

    # the same loader as the other arm: fp32 tensors in pinned host memory, the copy of the
    # next step's inputs issued on a side stream before the current step is launched
    copy_stream = torch.cuda.Stream(device=dev)
    pending = []

    def fetch():
        with torch.cuda.stream(copy_stream):
            batch = [t.to(dev, non_blocking=True) for t in host]
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return batch, ev

    def one_step(e2e: bool, last: bool = False):
        if not e2e:
            return runner.step(*resident)
        batch, ev = pending.pop() if pending else fetch()
        if not last:
            pending.append(fetch())
        torch.cuda.current_stream(dev).wait_event(ev)
        for t in batch:
            t.record_stream(torch.cuda.current_stream(dev))
        losses = runner.step(*batch)
        return float(sum(l.detach().float() for l in losses).cpu())

    dp_group = getattr(state, "dp_group", None) if state.dp_size > 1 else None

    def sync():
        torch.cuda.synchronize()
        if dp_group is not None:
            torch.distributed.barrier(group=dp_group)
            torch.cuda.synchronize()

    def timed(e2e: bool) -> float:
        sync()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(args.steps):
            one_step(e2e, last=(i == args.steps - 1))
        e.record()
        sync()
        return s.elapsed_time(e) / args.steps

    for _ in range(max(args.warmup, 3)):
        one_step(False)
    sampler = harness.ClockSampler(dev.index or 0)
    if state.is_main_process:
        sampler.start()
    ms = timed(False)
    one_step(True, last=True)
    ms_e2e = timed(True)
    clocks = sampler.stop() if state.is_main_process else None
    _write({"ms": ms, "ms_e2e": ms_e2e, "samples": n, "dp": state.dp_size, "pp": state.pp_size,
            "clocks": clocks, "h2d": sum(t.numel() * t.element_size() for t in host)})
    sys.stdout.flush()
    try:
        runner.worker.destroy_workers()   # the reference's own shutdown broadcast (its atexit hook)
    except Exception:
        pass
    os._exit(0)

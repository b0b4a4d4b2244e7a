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


def _start_watchdog(rank: int) -> None:
    """The reference profiles every graph node before its first step, which at full size can
    take tens of minutes; past the limit (PFEIFE_REF_TIMEOUT seconds, default 1500) every rank
    leaves and rank 0 reports the arm as unavailable instead of running into the caller's own
    time limit without a line."""
    import threading
    limit = float(os.environ.get("PFEIFE_REF_TIMEOUT", "1500"))

    def fire():
        if rank == 0:
            unavailable(f"the reference did not finish profiling and {limit:.0f} s of steps "
                        f"(its node-by-node profiling pass dominates)")
        os._exit(0)

    t = threading.Timer(limit + (0.0 if rank == 0 else 5.0), fire)
    t.daemon = True
    t.start()


def run(args) -> int:
    ref_root = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_root, "pfeife")):
        return unavailable("baseline/_ref is not installed")
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
        return unavailable("no CUDA device")
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
        return unavailable(f"reference import failed: {type(e).__name__}: {e}")

    state = initialize_pfeife()
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
    option = PipeOption(device_cnt=world, batch_size=args.batch_size, batch_cnt=args.batch_cnt,
                        mixed_precision="fp16", optimizer={"type": "adamw", "lr": 1e-4},
                        no_bench_optimizer=True, verbosity="info",
                        device_bench=os.path.join("/tmp", f"pfeife_ref_dev{world}.bench"))
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
    g = torch.Generator(device="cpu").manual_seed(1)
    host_x = torch.randn(n, 3, 224, 224, generator=g).pin_memory()
    host_y = torch.randint(0, 1000, (n,), generator=g).pin_memory()
    x_dev, y_dev = host_x.to(dev), host_y.to(dev)

    ClockSampler, emit_result = harness.ClockSampler, harness.emit_result

    def one_step(e2e: bool):
        if e2e:
            x = host_x.to(dev, non_blocking=True)
            y = host_y.to(dev, non_blocking=True)
        else:
            x, y = x_dev, y_dev
        losses = runner.step(x, y)
        if e2e:
            return float(sum(l.detach().float() for l in losses).cpu())
        return losses

    for _ in range(max(args.warmup, 3)):
        one_step(False)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        one_step(False)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    s.record()
    for _ in range(args.steps):
        one_step(True)
    e.record()
    torch.cuda.synchronize()
    ms_e2e = s.elapsed_time(e) / args.steps
    clocks = sampler.stop()
    emit_result(args, impl="reference", n_gpus=world, ms=ms, ms_e2e=ms_e2e, samples=n,
                clocks=clocks, launches=None, parallelism=f"pp{world}",
                h2d=host_x.numel() * 4 + host_y.numel() * 8, d2h=4)
    sys.stdout.flush()
    try:
        runner.worker.destroy_workers()   # the reference's own shutdown broadcast (its atexit hook)
    except Exception:
        pass
    os._exit(0)

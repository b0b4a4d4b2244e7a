"""End-to-end training on one GPU through the public API: mixed precision with the native
kernels, eager versus CUDA-graph replay, against fp32 PyTorch training of the same model."""
import copy
import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _train(cuda_graphs, steps=4, precision="bf16"):
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("MASTER_PORT", "29877")
    from pfeife_b200 import PartialRunner, PipeOption, initialize_pfeife, ops, partial_compiler
    from pfeife_b200.models.vit import ViT, vit_config
    from pfeife_b200.ops import _lib
    from pfeife_b200.ops import kernels as kx

    state = initialize_pfeife()
    dev = state.device
    torch.manual_seed(0)
    cfg = vit_config("vit_tiny", num_layers=3, image_size=64, patch_size=16, num_classes=16)
    model = ViT(cfg).to(dev)
    ref = copy.deepcopy(model).float()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.01)
    option = PipeOption(device_cnt=1, batch_size=8, batch_cnt=2, mixed_precision=precision,
                        no_bench_optimizer=True, cuda_graphs=cuda_graphs, verbosity="warning")
    runner = PartialRunner(option, opt)
    torch._dynamo.reset()
    cm = torch.compile(model, backend=partial_compiler)

    def fn(x, y):
        loss = ops.cross_entropy(cm(x), y)
        runner.scaler.scale(loss).backward()
        return loss.detach()

    runner.set_exec_fn(fn)
    g = torch.Generator().manual_seed(3)
    losses, ref_losses = [], []
    before = _lib.launch_count()
    for _ in range(steps):
        x = torch.randn(16, 3, 64, 64, generator=g).to(dev)
        y = torch.randint(0, 16, (16,), generator=g).to(dev)
        out = runner.step(x.to(torch.bfloat16 if precision == "bf16" else torch.float16), y)
        losses.append(sum(float(l) for l in out))
        ropt.zero_grad()
        cur = 0.0
        for xs, ys in zip(x.chunk(2), y.chunk(2)):
            l = F.cross_entropy(ref(xs), ys)
            l.backward()
            cur += float(l)
        ropt.step()
        ref_losses.append(cur)
    torch.cuda.synchronize()
    kx.check_status()
    launched = _lib.launch_count() - before
    runner.gather_params()
    diff = max(float((p.detach().float() - q.detach()).abs().max())
               for p, q in zip(model.parameters(), ref.parameters()))
    graphs = len(runner.worker.graphs)
    runner.close()
    return losses, ref_losses, diff, launched, graphs


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_vit_training_matches_fp32_reference(cuda_graphs):
    losses, ref_losses, diff, launched, graphs = _train(cuda_graphs)
    assert launched > 100, "native kernels did not run"
    for a, b in zip(losses, ref_losses):
        assert a == pytest.approx(b, rel=3e-2, abs=3e-2)
    assert diff < 2e-2
    assert (graphs > 0) == cuda_graphs


@pytest.mark.parametrize("workload", ["vit_tiny", "llama_tiny", "unet_tiny"])
def test_bench_workloads_run_natively(workload):
    """The benchmark harness drives every model family through the public API on the GPU (CUDA
    graphs on): one JSON line with a positive rate and kernels of this library launched."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # a rendezvous port of its own: this process may still hold the default one
    port = 29741 + ["vit_tiny", "llama_tiny", "unet_tiny"].index(workload)
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--workload", workload,
                        "--steps", "2", "--warmup", "3"], stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=600, cwd=root, env=env)
    assert r.returncode == 0, r.stdout[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    rec = json.loads(line)
    assert rec["value"] > 0 and rec["e2e"]["value"] > 0
    assert rec["gpu_launches"] > 0
    assert rec["e2e"]["h2d_bytes_per_step"] > 0
    assert rec["loss_mean_last_step"] is not None and \
        rec["loss_mean_last_step"] == rec["loss_mean_last_step"]      # finite, not NaN

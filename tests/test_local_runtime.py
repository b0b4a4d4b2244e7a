"""Single-process thread-per-device runtime on CPU devices, and the manager-style API."""
import copy

import pytest
import torch
import torch.nn.functional as F

from pfeife_b200.loss import CrossEntropyLoss
from pfeife_b200.models.toy import DeepMLP, TiedMLP
from pfeife_b200.option import PipeOption
from pfeife_b200.runtime.manager import LocalPipeManager


@pytest.mark.parametrize("model_fn,dim,devices", [
    (lambda: DeepMLP(16, 8, 10), 16, 2),
    (lambda: TiedMLP(10, 3), 10, 2),
    (lambda: DeepMLP(16, 9, 10), 16, 3),
])
def test_local_pipeline_matches_plain_training(model_fn, dim, devices):
    torch.manual_seed(0)
    torch._dynamo.reset()
    model = model_fn()
    ref = copy.deepcopy(model)
    option = PipeOption(device_cnt=devices, batch_size=2, batch_cnt=4, cpu_test=True,
                        no_bench_optimizer=True, verbosity="warning", ctrl_timeout=60,
                        optimizer={"type": "sgd", "lr": 0.05})
    mgr = LocalPipeManager(model, CrossEntropyLoss(10), option)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(1)
    try:
        for _ in range(3):
            x = torch.randn(8, dim, generator=g)
            y = torch.randint(0, 10, (8,), generator=g)
            losses = mgr.run(y, x)
            ropt.zero_grad()
            want = []
            for xs, ys in zip(x.chunk(4), y.chunk(4)):
                l = F.cross_entropy(ref(xs), ys)
                l.backward()
                want.append(float(l.detach()))
            ropt.step()
            assert [float(l) for l in losses] == pytest.approx(want, abs=1e-5)
        mgr.gather_params()
        for p, q in zip(model.parameters(), ref.parameters()):
            assert torch.allclose(p, q, atol=1e-5)
        assert len(mgr.runner.workers) == devices
    finally:
        mgr.close()


@pytest.mark.timeout(120)
def test_a_failing_stage_stops_the_whole_pipeline_at_once():
    """Whichever device thread fails, the step raises that error within moments (the other
    stages stop waiting for its tensors) and the runner refuses further steps."""
    import time

    import torch

    from pfeife_b200 import PipeOption
    from pfeife_b200.loss import SumLoss
    from pfeife_b200.runtime.manager import LocalPipeManager

    torch.manual_seed(0)
    model = torch.nn.Sequential(*[torch.nn.Linear(8, 8) for _ in range(6)])
    option = PipeOption(device_cnt=2, batch_size=2, batch_cnt=2, cpu_test=True,
                        no_bench_optimizer=True, ctrl_timeout=60)
    mgr = LocalPipeManager(model, SumLoss(), option)
    x = torch.randn(4, 8)
    mgr.run(None, x)

    def boom(*a, **k):
        raise ValueError("stage 0 broke")

    mgr.runner.workers[0].forward = boom
    t0 = time.time()
    with pytest.raises(ValueError, match="stage 0 broke"):
        mgr.run(None, x)
    assert time.time() - t0 < 20
    with pytest.raises(RuntimeError, match="stopped after a failed step"):
        mgr.run(None, x)
    mgr.close()

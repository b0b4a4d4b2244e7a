"""The fused data-parallel step on one device: the single-rank form against torch's AdamW over
two optimizer groups, the job-wide skip flag, the applied-step counter, and a wait that runs
out (a replica that never arrives) leaving the weights untouched and the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tables(*tensors_per_rank):
    from pfeife_b200.parallel.dp_fused import _table
    return _table([t.data_ptr() for t in tensors_per_rank])


def _setup(n, world=1, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda: torch.randn(n, device="cuda", generator=g)
    st = {
        "grad": [mk() * 0.01 for _ in range(world)],
        "master": [mk() for _ in range(world)],
        "lp": [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(world)],
        "flags": [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(world)],
        "local_sync": torch.zeros(4, dtype=torch.int32, device="cuda"),
        "found": torch.zeros(1, device="cuda"),
        "applied": torch.zeros(1, dtype=torch.int32, device="cuda"),
    }
    for r in range(1, world):
        st["master"][r].copy_(st["master"][0])
    return st


def _launch(st, rank, world, shard, total, groups, hyper, m, v, **kw):
    from pfeife_b200.parallel.dp_fused import launch_fused_step
    return launch_fused_step(
        rank, world, _tables(*st["grad"]), _tables(*st["master"]), _tables(*st["lp"]),
        _tables(*st["flags"]), m, v, st["local_sync"], shard, total, groups, hyper,
        st["applied"], kw.get("host_step", 1), kw.get("grad_scale", 1.0), st["lp"][0].dtype,
        check_inf=kw.get("check_inf", False), found_given=kw.get("found_given", False),
        loss_scale=kw.get("loss_scale"), found_inf=st["found"], epoch=kw.get("epoch", 1),
        arrivals=kw.get("arrivals", 0), device=torch.device("cuda", 0))


@pytest.mark.parametrize("n", [1 << 20, (1 << 20) + 4])      # whole 8-element groups / 4 left over
def test_single_rank_two_groups_match_torch_adamw_over_three_steps(n):
    from pfeife_b200.ops import kernels as kx
    cut = 3 << 18
    st = _setup(n)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ref = st["master"][0].clone()
    p0, p1 = ref[:cut].clone().requires_grad_(), ref[cut:].clone().requires_grad_()
    opt = torch.optim.AdamW([{"params": [p0], "lr": 1e-2, "weight_decay": 0.1},
                             {"params": [p1], "lr": 3e-3, "weight_decay": 0.0,
                              "betas": (0.8, 0.95)}], eps=1e-8)
    groups = [(0, cut, 0, 0), (cut, n, cut, cut)]
    hyper = [(1e-2, 0.9, 0.999, 1e-8, 0.1, True), (3e-3, 0.8, 0.95, 1e-8, 0.0, True)]
    epoch = arrivals = 0
    epoch = 1
    for step in range(3):
        g = torch.randn(n, device="cuda") * 0.02
        st["grad"][0].copy_(g)
        p0.grad, p1.grad = g[:cut].clone(), g[cut:].clone()
        opt.step()
        nbar, grid = _launch(st, 0, 1, (0, n), n, groups, hyper, m, v, epoch=epoch,
                             arrivals=arrivals)
        kx.step_advance(st["applied"], None)
        epoch += nbar
        arrivals += nbar * grid
    torch.cuda.synchronize()
    kx.check_status()
    want = torch.cat([p0.detach(), p1.detach()])
    assert torch.allclose(st["master"][0], want, atol=2e-6, rtol=2e-6)
    assert torch.equal(st["lp"][0], want.to(torch.bfloat16)) or \
        torch.allclose(st["lp"][0].float(), want, atol=1e-2, rtol=1e-2)
    assert int(st["grad"][0].abs().max()) == 0          # the bucket was cleared
    assert int(st["applied"]) == 3


def test_agreed_skip_flag_leaves_weights_and_step_count_alone():
    from pfeife_b200.ops import kernels as kx
    n = 1 << 18
    st = _setup(n, dtype=torch.float16)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    before = st["master"][0].clone()
    groups, hyper = [(0, n, 0, 0)], [(1e-2, 0.9, 0.999, 1e-8, 0.0, True)]
    scale = torch.tensor([1024.0], device="cuda")
    st["found"].fill_(1.0)                               # decided elsewhere: skip this step
    nbar, grid = _launch(st, 0, 1, (0, n), n, groups, hyper, m, v, found_given=True,
                         loss_scale=scale)
    kx.step_advance(st["applied"], st["found"])
    torch.cuda.synchronize()
    assert torch.equal(st["master"][0], before) and float(m.abs().max()) == 0.0
    assert int(st["applied"]) == 0 and float(st["grad"][0].abs().max()) == 0.0
    # the next step is applied with the bias correction of a FIRST step
    st["found"].zero_()
    g = torch.randn(n, device="cuda") * 0.5
    st["grad"][0].copy_(g * 1024.0)
    _launch(st, 0, 1, (0, n), n, groups, hyper, m, v, found_given=True, loss_scale=scale,
            epoch=1 + nbar, arrivals=nbar * grid, host_step=2)
    kx.step_advance(st["applied"], st["found"])
    torch.cuda.synchronize()
    kx.check_status()
    want = before - 1e-2 * g / (g.abs() + 1e-8)          # Adam's first step: lr * sign(g)
    assert torch.allclose(st["master"][0], want, atol=1e-5, rtol=1e-5)
    assert int(st["applied"]) == 1


def test_in_kernel_overflow_check_skips_every_group():
    n, cut = 1 << 18, 1 << 17
    st = _setup(n, dtype=torch.float16)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    before = st["master"][0].clone()
    st["grad"][0][n - 5] = float("inf")                  # only the second group overflows
    groups = [(0, cut, 0, 0), (cut, n, cut, cut)]
    hyper = [(1e-2, 0.9, 0.999, 1e-8, 0.0, True)] * 2
    _launch(st, 0, 1, (0, n), n, groups, hyper, m, v, check_inf=True,
            loss_scale=torch.tensor([2.0], device="cuda"))
    torch.cuda.synchronize()
    assert float(st["found"]) == 1.0
    assert torch.equal(st["master"][0], before)          # neither group moved
    assert float(st["grad"][0].abs().max()) == 0.0


def test_a_replica_that_never_arrives_runs_the_wait_out_and_nothing_is_written():
    """World of two with both buffers on this device and rank 1 never launched: rank 0's entry
    barrier gives up after the (shortened) limit, reports TIMEOUT_PEER_FLAG, skips the reduce,
    the update and every store to its peer, and the device keeps working."""
    from pfeife_b200.ops import _lib
    from pfeife_b200.ops import kernels as kx
    n = 1 << 18
    st = _setup(n, world=2)
    m, v = torch.zeros(n // 2, device="cuda"), torch.zeros(n // 2, device="cuda")
    snap = {k: [t.clone() for t in st[k]] for k in ("grad", "master", "lp")}
    groups, hyper = [(0, n, 0, 0)], [(1e-2, 0.9, 0.999, 1e-8, 0.0, True)]
    torch.cuda.synchronize()
    kx.check_status()
    kx.set_wait_limit(2_000_000)                         # about a millisecond
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        _launch(st, 0, 2, (0, n // 2), n, groups, hyper, m, v)
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 2000.0              # gave up quickly
        with pytest.raises(_lib.KernelError, match="TIMEOUT_PEER_FLAG"):
            kx.check_status()
    finally:
        kx.set_wait_limit(None)
    for k in ("grad", "master", "lp"):
        for a, b in zip(st[k], snap[k]):
            assert torch.equal(a, b)
    assert float(st["found"]) == 1.0                     # the step counts as skipped
    # the context is intact: an ordinary kernel runs and the status word is clean again
    x = torch.randn(256, 1408, device="cuda", dtype=torch.bfloat16)
    y, *_ = kx.norm_fwd(x, torch.ones(1408, device="cuda"), None, 1e-5, True)
    torch.cuda.synchronize()
    kx.check_status()
    assert torch.isfinite(y.float()).all()


def test_status_poll_reports_one_call_later():
    from pfeife_b200.ops import _lib
    from pfeife_b200.ops import kernels as kx
    kx.check_status()
    kx.poll_status()
    kx.status_word()[0] = 5
    kx.poll_status()                                     # starts the copy that sees the code
    with pytest.raises(_lib.KernelError):
        kx.poll_status()
    kx.poll_status()
    kx.check_status()

"""Memory-bound kernels (norms, activations, optimizer, losses, embedding, RoPE) against plain
PyTorch fp32 references of the same op."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _t(*shape, dtype=torch.bfloat16, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


def _tol(dtype):
    return {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,N", [(37, 1408), (64, 1024), (9, 4096), (130, 640)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(dtype, rows, N, rms):
    from pfeife_b200.ops import kernels as kx
    x = _t(rows, N, dtype=dtype)
    res = _t(rows, N, dtype=dtype, seed=1)
    gamma = torch.randn(N, device="cuda") * 0.5 + 1.0
    beta = None if rms else torch.randn(N, device="cuda") * 0.1
    dy = _t(rows, N, dtype=dtype, seed=2)
    dres = _t(rows, N, dtype=dtype, seed=3)
    y, h, mean, rstd = kx.norm_fwd(x, gamma, beta, 1e-5, rms, residual=res)
    dx, dg, db = kx.norm_bwd(dy, h, gamma, mean, rstd, rms, dres=dres)

    hf = (x.float() + res.float()).to(dtype).float().requires_grad_()
    gf = gamma.clone().requires_grad_()
    if rms:
        yr = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
        bf = None
    else:
        bf = beta.clone().requires_grad_()
        yr = F.layer_norm(hf, (N,), gf, bf, 1e-5)
    yr.backward(dy.float())
    t = _tol(dtype)
    assert torch.allclose(h.float(), hf.detach(), atol=t, rtol=t)
    assert torch.allclose(y.float(), yr.detach(), atol=4 * t, rtol=t)
    assert torch.allclose(dx.float(), hf.grad + dres.float(), atol=8 * t, rtol=4 * t)
    assert torch.allclose(dg, gf.grad, atol=rows ** 0.5 * 8 * t, rtol=4 * t)
    if not rms:
        assert torch.allclose(db, bf.grad, atol=rows ** 0.5 * 8 * t, rtol=4 * t)


@pytest.mark.parametrize("rms", [False, True])
def test_norm_bwd_adds_into_existing_gradients(rms):
    """accumulate=True: the weight / bias gradients are added to what the buffers already hold
    (the framework's gradient bucket), two calls in a row."""
    from pfeife_b200.ops import kernels as kx
    rows, N, dtype = 3000, 1408, torch.bfloat16
    x = _t(rows, N, dtype=dtype)
    gamma = torch.randn(N, device="cuda") * 0.5 + 1.0
    beta = None if rms else torch.zeros(N, device="cuda")
    dy = _t(rows, N, dtype=dtype, seed=2)
    y, h, mean, rstd = kx.norm_fwd(x, gamma, beta, 1e-5, rms)
    _, dg_ref, db_ref = kx.norm_bwd(dy, x, gamma, mean, rstd, rms)
    dg = torch.full((N,), 2.0, device="cuda")
    db = None if rms else torch.full((N,), -1.0, device="cuda")
    for _ in range(2):
        kx.norm_bwd(dy, x, gamma, mean, rstd, rms, dgamma=dg, dbeta=db, accumulate=True,
                    want_dbeta=not rms)
    torch.cuda.synchronize()
    assert torch.allclose(dg, 2.0 + 2.0 * dg_ref, atol=0.05, rtol=1e-3)
    if not rms:
        assert torch.allclose(db, -1.0 + 2.0 * db_ref, atol=0.05, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_elementwise_family(dtype):
    from pfeife_b200.ops import kernels as kx
    x = _t(1000, 77, dtype=dtype)
    y = _t(1000, 77, dtype=dtype, seed=1)
    t = _tol(dtype)
    xf, yf = x.float(), y.float()
    assert torch.allclose(kx.elementwise(kx.EW_GELU, x).float(), F.gelu(xf), atol=t, rtol=t)
    assert torch.allclose(kx.elementwise(kx.EW_GELU_TANH, x).float(),
                          F.gelu(xf, approximate="tanh"), atol=t, rtol=t)
    assert torch.allclose(kx.elementwise(kx.EW_SILU, x).float(), F.silu(xf), atol=t, rtol=t)
    assert torch.allclose(kx.elementwise(kx.EW_ADD, x, y).float(), xf + yf, atol=t, rtol=t)
    assert torch.allclose(kx.elementwise(kx.EW_SILU_MUL, x, y).float(), F.silu(xf) * yf,
                          atol=2 * t, rtol=2 * t)
    xr = xf.clone().requires_grad_()
    F.gelu(xr).backward(yf)
    assert torch.allclose(kx.elementwise(kx.EW_DGELU, y, x).float(), xr.grad, atol=2 * t, rtol=2 * t)


@pytest.mark.parametrize("gelu", [False, True])
def test_glu(gelu):
    from pfeife_b200.ops import kernels as kx
    H = 256
    gu = _t(33, 2 * H)
    dout = _t(33, H, seed=1)
    out = kx.glu_fwd(gu, gelu)
    dgu = kx.glu_bwd(gu, dout, gelu)
    g = gu.float().requires_grad_()
    act = F.gelu if gelu else F.silu
    ref = act(g[:, :H]) * g[:, H:]
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref.detach(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(dgu.float(), g.grad, atol=5e-2, rtol=3e-2)


def test_colsum_transpose_cast_axpy():
    from pfeife_b200.ops import kernels as kx
    x = _t(777, 200)
    assert torch.allclose(kx.colsum(x), x.float().sum(0), atol=0.5, rtol=1e-2)
    assert torch.equal(kx.transpose16(x), x.t().contiguous())
    f = torch.randn(5001, device="cuda")
    assert torch.equal(kx.cast(f, torch.bfloat16), f.to(torch.bfloat16))
    dst = torch.ones(777 * 200, device="cuda")
    kx.axpy_f32(dst, x, scale=0.5, accumulate=True)
    assert torch.allclose(dst, 1 + 0.5 * x.float().view(-1))


@pytest.mark.parametrize("decoupled", [True, False])
def test_adamw_matches_torch(decoupled):
    from pfeife_b200.ops import kernels as kx
    n = 100003
    p0 = torch.randn(n, device="cuda")
    ref = p0.clone().requires_grad_()
    cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    opt = cls([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.1)
    p, m, v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    found = torch.zeros(1, device="cuda")
    scale = torch.full((1,), 8.0, device="cuda")
    for step in range(1, 4):
        grad = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(step))
        ref.grad = grad.clone()
        opt.step()
        g = grad * 8.0
        kx.nonfinite(g, found)
        kx.adamw(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-6, weight_decay=0.1,
                 step=step, decoupled=decoupled, lp=lp, found_inf=found, loss_scale=scale)
        assert float(g.abs().max()) == 0.0  # gradient zeroed in the same pass
    assert torch.allclose(p, ref.detach(), atol=1e-5, rtol=1e-5)
    assert torch.equal(lp, p.to(torch.bfloat16))
    # a non-finite gradient skips the update
    g = torch.full((n,), float("inf"), device="cuda")
    before = p.clone()
    kx.nonfinite(g, found)
    kx.adamw(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-6, weight_decay=0.1, step=4,
             found_inf=found)
    assert float(found) == 1.0 and torch.equal(p, before)
    state = torch.tensor([8.0, 0.0], device="cuda")
    kx.loss_scale_update(state, found, 2.0, 0.5, 2)
    assert state.tolist() == [4.0, 0.0] and float(found) == 0.0


def test_sgd_matches_torch():
    from pfeife_b200.ops import kernels as kx
    n = 4099
    p0 = torch.randn(n, device="cuda")
    ref = p0.clone().requires_grad_()
    opt = torch.optim.SGD([ref], lr=0.01, momentum=0.9, weight_decay=0.01)
    p, mom = p0.clone(), torch.zeros(n, device="cuda")
    for step in range(3):
        grad = torch.randn(n, device="cuda")
        ref.grad = grad.clone()
        opt.step()
        kx.sgd(p, grad.clone(), mom, lr=0.01, momentum=0.9, weight_decay=0.01,
               first_step=(step == 0))
    assert torch.allclose(p, ref.detach(), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [1000, 32000, 10])
def test_cross_entropy(dtype, V):
    from pfeife_b200.ops import kernels as kx
    rows = 64
    logits = _t(rows, V, dtype=dtype, scale=3.0)
    target = torch.randint(0, V, (rows,), device="cuda")
    target[3] = -100
    loss, lse = kx.ce_fwd(logits, target)
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, target, reduction="none", ignore_index=-100)
    assert torch.allclose(loss, ref.detach(), atol=2e-3, rtol=1e-3)
    gs = torch.full((rows,), 1.0 / rows, device="cuda")
    d = kx.ce_bwd(logits, target, lse, gs)
    (ref.sum() / rows).backward()
    assert torch.allclose(d.float(), lf.grad, atol=_tol(dtype) / 4, rtol=2e-2)


def test_mse_embedding_rope():
    from pfeife_b200.ops import kernels as kx
    a, b = _t(4, 4, 64, 64), _t(4, 4, 64, 64, seed=1)
    out = kx.mse_fwd(a, b)
    assert torch.allclose(out, F.mse_loss(a.float(), b.float()).view(1), rtol=1e-3)
    da = kx.mse_bwd(a, b, torch.ones(1, device="cuda"))
    assert torch.allclose(da.float(), 2 * (a.float() - b.float()) / a.numel(), atol=1e-6, rtol=2e-2)

    table = torch.randn(500, 96, device="cuda")
    ids = torch.randint(0, 500, (3, 17), device="cuda")
    e = kx.embed_fwd(table, ids, torch.bfloat16)
    assert torch.equal(e, table[ids].to(torch.bfloat16))
    dt_ = torch.zeros_like(table)
    dout = _t(3, 17, 96)
    kx.embed_bwd(dout, ids, dt_)
    ref = torch.zeros_like(table).index_add_(0, ids.view(-1), dout.float().view(-1, 96))
    assert torch.allclose(dt_, ref, atol=1e-3)

    B, S, H, D = 2, 33, 4, 64
    x = _t(B, S, H, D)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.outer(torch.arange(S, device="cuda").float(), inv)
    cos, sin = ang.cos(), ang.sin()
    y = kx.rope(x, cos, sin)
    xf = x.float()
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    assert torch.allclose(y.float(), ref, atol=2e-2, rtol=2e-2)
    back = kx.rope(y, cos, sin, inverse=True)
    assert torch.allclose(back.float(), xf, atol=4e-2, rtol=4e-2)

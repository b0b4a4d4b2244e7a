"""The differentiable ops against PyTorch autograd.  On CPU this checks the reference formulas
that the CPU pipeline tests rely on; the GPU variants check the native kernels end to end
(forward and backward through the custom-op autograd wiring)."""
import pytest
import torch
import torch.nn.functional as F

from pfeife_b200 import ops

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _cfg(device):
    if device == "cpu":
        return torch.float32, 1e-4
    return torch.bfloat16, 6e-2


def _rand(*shape, device, dtype, seed=0, grad=True, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    t = (torch.randn(*shape, generator=g) * scale).to(device=device, dtype=dtype)
    return t.requires_grad_(grad)


def _check(a, b, tol):
    assert a.shape == b.shape
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item() + 1e-6
    assert err <= tol * max(1.0, ref), f"err {err} vs ref magnitude {ref}"


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("act", [None, "gelu", "gelu_tanh", "silu"])
def test_linear(device, act):
    dtype, tol = _cfg(device)
    x = _rand(3, 40, 64, device=device, dtype=dtype, scale=0.5)
    w = _rand(48, 64, device=device, dtype=dtype, seed=1, scale=0.2)
    b = _rand(48, device=device, dtype=torch.float32, seed=2)
    r = _rand(3, 40, 48, device=device, dtype=dtype, seed=3)
    y = ops.linear(x, w, b, activation=act, residual=r)
    y.backward(torch.ones_like(y))
    xr, wr, br, rr = (t.detach().float().requires_grad_() for t in (x, w, b, r))
    z = F.linear(xr, wr, br)
    z = {None: z, "gelu": F.gelu(z), "gelu_tanh": F.gelu(z, approximate="tanh"),
         "silu": F.silu(z)}[act]
    yr = z + rr
    yr.backward(torch.ones_like(yr))
    _check(y, yr, tol)
    _check(x.grad, xr.grad, tol)
    _check(w.grad, wr.grad, tol * 4)
    _check(b.grad, br.grad, tol * 4)
    _check(r.grad, rr.grad, tol)


@pytest.mark.parametrize("device", DEVICES)
def test_linear_with_an_input_width_that_is_not_a_multiple_of_8(device):
    """ViT patch embedding: 3 * 14 * 14 = 588 input features (padded to 592 inside the GEMMs)."""
    dtype, tol = _cfg(device)
    x = _rand(2, 30, 588, device=device, dtype=dtype, scale=0.5)
    w = _rand(64, 588, device=device, dtype=dtype, seed=1, scale=0.1)
    b = _rand(64, device=device, dtype=torch.float32, seed=2)
    y = ops.linear(x, w, b)
    gy = _rand(2, 30, 64, device=device, dtype=dtype, seed=5, grad=False)
    y.backward(gy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.linear(xr, wr, br)
    yr.backward(gy.float())
    _check(y, yr, tol)
    _check(x.grad, xr.grad, tol * 2)
    _check(w.grad, wr.grad, tol * 4)
    _check(b.grad, br.grad, tol * 4)


@pytest.mark.parametrize("device", DEVICES)
def test_mlp(device):
    dtype, tol = _cfg(device)
    x = _rand(2, 50, 64, device=device, dtype=dtype, scale=0.5)
    w1 = _rand(128, 64, device=device, dtype=dtype, seed=1, scale=0.2)
    b1 = _rand(128, device=device, dtype=torch.float32, seed=2)
    w2 = _rand(64, 128, device=device, dtype=dtype, seed=3, scale=0.2)
    b2 = _rand(64, device=device, dtype=torch.float32, seed=4)
    y = ops.mlp(x, w1, b1, w2, b2, "gelu", residual=x)
    y.backward(torch.ones_like(y))
    ts = [t.detach().float().requires_grad_() for t in (x, w1, b1, w2, b2)]
    yr = F.linear(F.gelu(F.linear(ts[0], ts[1], ts[2])), ts[3], ts[4]) + ts[0]
    yr.backward(torch.ones_like(yr))
    _check(y, yr, tol)
    for a, b in zip((x, w1, b1, w2, b2), ts):
        _check(a.grad, b.grad, tol * 4)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("with_res", [False, True])
def test_norms(device, rms, with_res):
    dtype, tol = _cfg(device)
    x = _rand(4, 17, 64, device=device, dtype=dtype)
    r = _rand(4, 17, 64, device=device, dtype=dtype, seed=1) if with_res else None
    g = _rand(64, device=device, dtype=torch.float32, seed=2)
    b = None if rms else _rand(64, device=device, dtype=torch.float32, seed=3)
    out = ops.rms_norm(x, g, 1e-5, residual=r) if rms else ops.layer_norm(x, g, b, 1e-5, residual=r)
    if with_res:
        y, h = out
        (y.float().sum() + (h.float() * 0.5).sum()).backward()
    else:
        y = out
        y.float().sum().backward()
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    gr = g.detach().clone().requires_grad_()
    br = None if rms else b.detach().clone().requires_grad_()
    hr = xr + rr if with_res else xr
    if rms:
        yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        yr = F.layer_norm(hr, (64,), gr, br, 1e-5)
    (yr.sum() + ((hr * 0.5).sum() if with_res else 0)).backward()
    _check(y, yr, tol)
    _check(x.grad, xr.grad, tol * 2)
    _check(g.grad, gr.grad, tol * 8)
    if not rms:
        _check(b.grad, br.grad, tol * 8)
    if with_res:
        _check(r.grad, rr.grad, tol * 2)


@pytest.mark.parametrize("device", DEVICES)
def test_activations_and_glu(device):
    dtype, tol = _cfg(device)
    x = _rand(5, 33, 64, device=device, dtype=dtype)
    for fn, ref in ((ops.gelu, F.gelu), (ops.silu, F.silu)):
        x.grad = None
        y = fn(x)
        y.backward(torch.ones_like(y))
        xr = x.detach().float().requires_grad_()
        yr = ref(xr)
        yr.backward(torch.ones_like(yr))
        _check(y, yr, tol)
        _check(x.grad, xr.grad, tol)
    for fn, ref in ((ops.swiglu, F.silu), (ops.geglu, F.gelu)):
        x.grad = None
        y = fn(x)
        y.backward(torch.ones_like(y))
        xr = x.detach().float().requires_grad_()
        yr = ref(xr[..., :32]) * xr[..., 32:]
        yr.backward(torch.ones_like(yr))
        _check(y, yr, tol)
        _check(x.grad, xr.grad, tol * 2)


@pytest.mark.parametrize("device", DEVICES)
def test_losses_embedding_rope(device):
    dtype, tol = _cfg(device)
    logits = _rand(6, 11, 50, device=device, dtype=dtype, scale=2.0)
    target = torch.randint(0, 50, (6, 11), generator=torch.Generator().manual_seed(0)).to(device)
    target[0, 0] = -100
    loss = ops.cross_entropy(logits, target)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lr.view(-1, 50), target.view(-1), ignore_index=-100)
    ref.backward()
    _check(loss, ref, tol)
    _check(logits.grad, lr.grad, tol)

    a = _rand(4, 8, 16, device=device, dtype=dtype)
    b = _rand(4, 8, 16, device=device, dtype=dtype, seed=1, grad=False)
    m = ops.mse_loss(a, b)
    m.backward()
    ar = a.detach().float().requires_grad_()
    mr = F.mse_loss(ar, b.float())
    mr.backward()
    _check(m, mr, tol)
    _check(a.grad, ar.grad, tol)

    table = _rand(30, 16, device=device, dtype=torch.float32)
    ids = torch.randint(0, 30, (3, 7), generator=torch.Generator().manual_seed(1)).to(device)
    e = ops.embedding(ids, table, out_dtype=dtype)
    e.float().sum().backward()
    tr = table.detach().clone().requires_grad_()
    F.embedding(ids, tr).sum().backward()
    _check(e, F.embedding(ids, table.detach()), tol)
    _check(table.grad, tr.grad, tol)

    q = _rand(2, 9, 3, 16, device=device, dtype=dtype)
    cos, sin = ops.rope_tables(9, 16, device=device)
    y = ops.rope(q, cos, sin)
    y.backward(torch.ones_like(y))
    qr = q.detach().float().requires_grad_()
    x1, x2 = qr[..., :8], qr[..., 8:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    yr = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    yr.backward(torch.ones_like(yr))
    _check(y, yr, tol)
    _check(q.grad, qr.grad, tol)


@pytest.mark.parametrize("device", DEVICES)
def test_registered_param_accumulates_into_bucket(device):
    """A registered master weight: forward reads the 16-bit shadow, wgrad lands in the fp32
    bucket and autograd sees no gradient for the weight."""
    dtype, tol = _cfg(device)
    if device == "cpu":
        pytest.skip("bucket accumulation is a property of the native wgrad epilogue")
    master = torch.randn(48, 64, device=device) * 0.2
    master.requires_grad_()
    lp = master.detach().to(dtype)
    bucket = torch.zeros(48 * 64, device=device)
    ops.register_param(master, lp, bucket)
    try:
        x = _rand(10, 64, device=device, dtype=dtype)
        for _ in range(2):
            ops.linear(x, master).float().sum().backward()
        assert master.grad is None
        ref = 2 * torch.ones(10, 48, device=device).t() @ x.detach().float()
        _check(bucket.view(48, 64), ref, tol)
    finally:
        ops.unregister_params()

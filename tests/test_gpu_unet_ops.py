"""UNet kernels (implicit-GEMM and im2col convolution, GroupNorm+SiLU, upsample) and the Llama / UNet model
families on the GPU against fp32 CPU references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float().cpu() - b.float().cpu()).abs().max().item()
    mag = b.float().abs().max().item()
    assert err <= tol * max(1.0, mag), f"err {err} vs magnitude {mag}"


@pytest.mark.parametrize("cin,cout,k,stride", [(16, 32, 3, 1), (32, 32, 3, 2), (24, 40, 1, 1),
                                               (4, 32, 3, 1), (32, 4, 3, 1)])
def test_conv2d_nhwc(cin, cout, k, stride):
    from pfeife_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(2, 16, 16, cin)
    w = torch.randn(cout, cin, k, k) * 0.1
    b = torch.randn(cout)
    xr, wr, br = (t.clone().requires_grad_() for t in (x, w, b))
    yr = F.conv2d(xr.permute(0, 3, 1, 2), wr, br, stride=stride, padding=k // 2).permute(0, 2, 3, 1)
    yr.sum().backward()
    xg = x.cuda().to(torch.bfloat16).requires_grad_()
    wg = w.cuda().to(torch.bfloat16).requires_grad_()
    bg = b.cuda().requires_grad_()
    y = ops.conv2d(xg, wg, bg, stride, k // 2)
    y.float().sum().backward()
    _close(y, yr.detach(), 3e-2)
    _close(xg.grad, xr.grad, 3e-2)
    _close(wg.grad, wr.grad, 3e-2)
    _close(bg.grad, br.grad, 3e-2)


@pytest.mark.parametrize("cin,cout,hw,k,stride", [
    (64, 128, 16, 3, 1),      # implicit GEMM forward and dgrad, tiles of 8 output rows
    (128, 64, 32, 3, 1),      # tiles of 4 output rows; 2048 output pixels
    (64, 64, 32, 3, 2),       # stride 2: implicit forward (16 x 16 outputs), col2im dgrad
    (128, 192, 64, 3, 1),     # two output rows per tile, several k-blocks per tap
    (64, 72, 16, 3, 1),       # Cout not a multiple of 64: implicit forward, GEMM + col2im dgrad
])
def test_conv2d_implicit_gemm(cin, cout, hw, k, stride):
    """Shapes the implicit-GEMM path covers (C % 64 == 0, whole output rows per 128-pixel tile):
    values and all gradients against an fp32 reference, with a random upstream gradient so that
    a misplaced filter tap cannot cancel out."""
    from pfeife_b200 import ops
    from pfeife_b200.ops import kernels as kx
    torch.manual_seed(1)
    x = torch.randn(2, hw, hw, cin)
    w = torch.randn(cout, cin, k, k) * 0.05
    b = torch.randn(cout)
    assert kx.conv_gemm_supported(x, k, k, stride, k // 2)
    xr, wr, br = (t.clone().requires_grad_() for t in (x, w, b))
    yr = F.conv2d(xr.permute(0, 3, 1, 2), wr, br, stride=stride, padding=k // 2).permute(0, 2, 3, 1)
    gy = torch.randn(yr.shape)
    yr.backward(gy)
    xg = x.cuda().to(torch.bfloat16).requires_grad_()
    wg = w.cuda().to(torch.bfloat16).requires_grad_()
    bg = b.cuda().requires_grad_()
    y = ops.conv2d(xg, wg, bg, stride, k // 2)
    y.backward(gy.cuda().to(y.dtype))
    torch.cuda.synchronize()
    kx.check_status()
    _close(y, yr.detach(), 3e-2)
    _close(xg.grad, xr.grad, 3e-2)
    _close(wg.grad, wr.grad, 3e-2)
    _close(bg.grad, br.grad, 3e-2)


@pytest.mark.parametrize("silu", [False, True])
def test_group_norm_silu(silu):
    from pfeife_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(2, 16, 16, 64)
    g, b = torch.randn(64) * 0.5 + 1, torch.randn(64) * 0.1
    xr, gr, br = (t.clone().requires_grad_() for t in (x, g, b))
    yr = F.group_norm(xr.permute(0, 3, 1, 2), 8, gr, br, 1e-5)
    yr = (F.silu(yr) if silu else yr).permute(0, 2, 3, 1)
    dy = torch.randn(2, 16, 16, 64)
    yr.backward(dy)
    xg = x.cuda().to(torch.bfloat16).requires_grad_()
    gg, bg = g.cuda().requires_grad_(), b.cuda().requires_grad_()
    y = ops.group_norm(xg, gg, bg, 8, 1e-5, silu)
    y.backward(dy.cuda().to(torch.bfloat16))
    _close(y, yr.detach(), 3e-2)
    _close(xg.grad, xr.grad, 5e-2)
    _close(gg.grad, gr.grad, 5e-2)
    _close(bg.grad, br.grad, 5e-2)


def test_upsample():
    from pfeife_b200 import ops
    x = torch.randn(2, 8, 8, 32, device="cuda").to(torch.bfloat16).requires_grad_()
    y = ops.upsample_nearest2x(x)
    y.float().pow(2).sum().backward()
    xr = x.detach().float().requires_grad_()
    yr = xr.repeat_interleave(2, 1).repeat_interleave(2, 2)
    yr.pow(2).sum().backward()
    _close(y, yr.detach(), 1e-2)
    _close(x.grad, xr.grad, 3e-2)


def _model_grads(model, loss_of, device, dtype):
    import copy
    m = copy.deepcopy(model).to(device)
    if dtype is not None:
        with torch.autocast("cuda", dtype=dtype):
            loss = loss_of(m)
    else:
        loss = loss_of(m)
    loss.backward()
    return float(loss.detach()), {n: p.grad.detach().float().cpu() for n, p in m.named_parameters()}


def test_llama_model_gpu_matches_cpu():
    from pfeife_b200.models.llama import Llama, causal_lm_loss, llama_config
    torch.manual_seed(0)
    model = Llama(llama_config("llama_tiny", hidden_size=128, num_heads=4, intermediate_size=256))
    ids = torch.randint(0, 256, (2, 32))
    lc, gc = _model_grads(model, lambda m: causal_lm_loss(m(ids).float(), ids), "cpu", None)
    lg, gg = _model_grads(model, lambda m: causal_lm_loss(m(ids.cuda()), ids.cuda()), "cuda",
                          torch.bfloat16)
    assert lg == pytest.approx(lc, rel=2e-2)
    for n in gc:
        _close(gg[n], gc[n], 8e-2)


def test_unet_model_gpu_matches_cpu():
    from pfeife_b200 import ops
    from pfeife_b200.models.unet import UNet, unet_config
    torch.manual_seed(0)
    model = UNet(unet_config("unet_tiny"))
    B = 2
    args = (torch.randn(B, 4, 16, 16), torch.randint(0, 1000, (B,)), torch.randn(B, 7, 32),
            torch.randn(B, 16), torch.randn(B, 6))
    noise = torch.randn(B, 4, 16, 16)
    lc, gc = _model_grads(model, lambda m: F.mse_loss(m(*args).float(), noise), "cpu", None)
    cargs = tuple(a.cuda() for a in args)
    lg, gg = _model_grads(
        model, lambda m: F.mse_loss(m(cargs[0].to(torch.bfloat16), *cargs[1:]).float(),
                                    noise.cuda()), "cuda", torch.bfloat16)
    assert lg == pytest.approx(lc, rel=3e-2)
    worst = max((gg[n] - gc[n]).abs().max().item() / max(1e-3, gc[n].abs().max().item())
                for n in gc)
    assert worst < 0.25

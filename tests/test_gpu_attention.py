"""tcgen05 flash attention (forward and backward) against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_attn(q, k, v, causal, scale):
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = torch.ones(sq, sk, dtype=torch.bool, device=s.device).tril(sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    return (p @ vf).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


CASES = [  # B, H, Sq, Sk, D, causal
    (2, 3, 197, 197, 64, False),     # ViT-L
    (1, 2, 257, 257, 88, False),     # ViT-g/14 head dim
    (1, 2, 300, 300, 128, True),     # Llama-style causal
    (2, 2, 128, 77, 64, False),      # UNet cross attention
    (1, 1, 1024, 1024, 64, False),
    (1, 2, 64, 64, 32, True),
    # a few rows past a multiple of 128: leftover queries / keys run on CUDA cores
    (2, 2, 259, 259, 64, True),
    (1, 2, 130, 257, 96, False),
    (1, 2, 260, 384, 32, False),
    (1, 2, 256, 258, 64, False),
    (1, 2, 261, 261, 64, False),     # five leftover rows: a ragged tensor-core tile instead
    (1, 2, 258, 300, 64, True),      # causal with Sq != Sk: ragged key tiles in the backward
    (1, 4, 1024, 1024, 128, True),   # several query tiles per head, many key tiles each
    (3, 5, 384, 640, 64, False),     # more work items than one wave of a small grid
    (4, 3, 17, 17, 64, False),       # far fewer rows than one tile (reduced ViT of the tests)
    (2, 4, 16, 16, 32, True),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Sq,Sk,D,causal", CASES)
def test_attention_fwd_bwd(dtype, B, H, Sq, Sk, D, causal):
    from pfeife_b200.ops import kernels as kx
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda S: torch.randn(B, S, H, D, device="cuda", generator=g).to(dtype)
    q, k, v = mk(Sq), mk(Sk), mk(Sk)
    do = mk(Sq)
    scale = 1.0 / math.sqrt(D)
    o, lse = kx.attn_fwd(q, k, v, causal, scale)
    dq, dk, dv = kx.attn_bwd(do, q, k, v, o, lse, causal, scale)
    torch.cuda.synchronize()
    kx.check_status()
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref, lse_ref = ref_attn(qr, kr, vr, causal, scale)
    o_ref.backward(do.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert (o.float() - o_ref).abs().max() <= tol * 2
    assert (lse - lse_ref).abs().max() <= 2e-2
    for got, want, name in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
        err = (got.float() - want).abs().max().item()
        mag = want.abs().max().item()
        assert err <= tol * 4 * max(1.0, mag), f"{name}: err {err} (max |ref| {mag})"


@pytest.mark.parametrize("D", [64, 128])
def test_attention_forward_when_the_row_maximum_keeps_growing(D):
    """Later key tiles carry much larger scores than earlier ones, so the maximum that scales
    the probabilities has to be raised (and the accumulated output rescaled) several times
    within one row; keys of the last tile are tiny again (no rescale there)."""
    from pfeife_b200.ops import kernels as kx
    B, H, Sq, Sk = 1, 2, 256, 768
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(B, Sq, H, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, Sk, H, D, device="cuda", generator=g)
    ramp = torch.tensor([0.1, 1.0, 4.0, 12.0, 30.0, 0.05], device="cuda").repeat_interleave(128)
    k = (k * ramp[None, :, None, None]).to(torch.bfloat16)
    v = torch.randn(B, Sk, H, D, device="cuda", generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    o, lse = kx.attn_fwd(q, k, v, False, scale)
    torch.cuda.synchronize()
    kx.check_status()
    o_ref, lse_ref = ref_attn(q, k, v, False, scale)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref).abs().max() <= 4e-2
    assert ((lse - lse_ref).abs() / lse_ref.abs().clamp_min(1.0)).max() <= 1e-2


def test_attention_on_fused_qkv_views():
    """q, k, v as strided slices of one [B, S, 3, H, D] projection, through autograd."""
    from pfeife_b200 import ops
    B, S, H, D = 2, 257, 4, 88
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.5).to(torch.float16).requires_grad_()
    out = ops.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2])
    out.float().sum().backward()
    ref_in = qkv.detach().float().requires_grad_()
    o_ref, _ = ref_attn(ref_in[:, :, 0], ref_in[:, :, 1], ref_in[:, :, 2], False, 1 / math.sqrt(D))
    o_ref.sum().backward()
    assert (out.float() - o_ref).abs().max() <= 1e-2
    assert (qkv.grad.float() - ref_in.grad).abs().max() <= 5e-2


def test_packed_qkv_attention_writes_fused_gradient():
    from pfeife_b200 import ops
    B, S, H, D = 2, 300, 2, 64
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    out = ops.attention_qkv(qkv, causal=True)
    out.float().sum().backward()
    ref_in = qkv.detach().float().requires_grad_()
    o_ref, _ = ref_attn(ref_in[:, :, 0], ref_in[:, :, 1], ref_in[:, :, 2], True, 1 / math.sqrt(D))
    o_ref.sum().backward()
    assert (out.float() - o_ref).abs().max() <= 2e-2
    assert (qkv.grad.float() - ref_in.grad).abs().max() <= 1e-1

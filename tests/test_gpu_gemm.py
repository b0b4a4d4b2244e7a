"""tcgen05 GEMM against an fp32 PyTorch reference: every operand-major combination, ragged
tile edges, every epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _mk(M, N, K, a_mn, b_mn, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).to(dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).to(dtype)
    return a, b


def _close(out, ref, K, dtype):
    tol = (2e-2 if dtype == torch.bfloat16 else 4e-3) * (K ** 0.5)
    err = (out.float() - ref).abs().max().item()
    assert err <= tol, f"max abs err {err} > {tol}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136),
                                   (6168, 1408, 1408), (1000, 128, 72)])
def test_gemm_layouts(a_mn, b_mn, dtype, M, N, K):
    from pfeife_b200.ops import kernels as kx
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned pitch")
    a, b = _mk(M, N, K, a_mn, b_mn, dtype)
    out = kx.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    kx.check_status()
    _close(out, _ref(a, b, a_mn, b_mn), K, dtype)


@pytest.mark.parametrize("tile_n", [128, 256, 1024 + 256])   # bit 10: direct-store epilogue
def test_gemm_tile_variants_and_fp32_out(tile_n):
    from pfeife_b200.ops import kernels as kx
    a, b = _mk(520, 776, 320, False, False, torch.bfloat16)
    out = kx.gemm(a, b, out_dtype=torch.float32, tile_n=tile_n)
    torch.cuda.synchronize()
    _close(out, _ref(a, b, False, False), 320, torch.float32)


@pytest.mark.parametrize("tile_n", [0, 1024])
@pytest.mark.parametrize("M,N,K", [(400, 384, 192), (6168, 1408, 320)])
def test_gemm_epilogues(tile_n, M, N, K):
    """Every fused epilogue through the TMA-store path (tile_n 0) and the direct-store path."""
    from pfeife_b200.ops import kernels as kx
    dtype = torch.bfloat16
    a, b = _mk(M, N, K, False, False, dtype)
    a = a * 0.1
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").to(dtype)
    ref = _ref(a, b, False, False) + bias
    # bias + residual
    out = kx.gemm(a, b, bias=bias, residual=res, tile_n=tile_n)
    _close(out, ref + res.float(), K, dtype)
    # bias + GELU with saved pre-activation
    aux = torch.empty(M, N, device="cuda", dtype=dtype)
    out = kx.gemm(a, b, bias=bias, aux=aux, epilogue=kx.EPI_GELU, tile_n=tile_n)
    _close(aux, ref, K, dtype)
    _close(out, torch.nn.functional.gelu(ref), K, dtype)
    # dGELU: out = acc * gelu'(aux)
    z = torch.randn(M, N, device="cuda").to(dtype)
    out = kx.gemm(a, b, aux=z, epilogue=kx.EPI_DGELU, tile_n=tile_n)
    zf = z.float().requires_grad_()
    torch.nn.functional.gelu(zf).sum().backward()
    _close(out, _ref(a, b, False, False) * zf.grad, K, dtype)
    # fp32 accumulate (gradient bucket), both operands MN-major as in wgrad
    at, bt = a.t().contiguous(), b.t().contiguous()
    bucket = torch.ones(M, N, device="cuda")
    kx.gemm(at, bt, a_mn=True, b_mn=True, out=bucket, accumulate=True, tile_n=tile_n)
    kx.gemm(at, bt, a_mn=True, b_mn=True, out=bucket, accumulate=True, tile_n=tile_n)
    torch.cuda.synchronize()
    kx.check_status()
    _close(bucket, 1.0 + 2.0 * _ref(a, b, False, False), K, torch.float32)


def test_gemm_strided_views():
    """Operands that are column slices of a wider tensor (fused QKV) keep their pitch."""
    from pfeife_b200.ops import kernels as kx
    big = torch.randn(512, 3 * 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(128, 256, device="cuda").to(torch.bfloat16)
    q = big[:, 256:512]
    out = torch.empty(512, 2 * 128, device="cuda", dtype=torch.bfloat16)
    kx.gemm(q, w, out=out[:, 128:])
    torch.cuda.synchronize()
    _close(out[:, 128:], q.float() @ w.float().t(), 256, torch.bfloat16)

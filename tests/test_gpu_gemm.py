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
    # relative bound: all that separates the two is the rounding of the output to 16 bits (and
    # of 16-bit intermediates some epilogues save), far below one percent of the result's norm
    rel = ((out.float() - ref).norm() / ref.norm().clamp_min(1e-20)).item()
    rtol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    assert rel <= rtol, f"relative error {rel} > {rtol}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136),
                                   (6168, 1408, 1408), (1000, 128, 72)])
@pytest.mark.parametrize("form", [4096, 2048])   # single-CTA tiles / CTA-pair tiles
def test_gemm_layouts(a_mn, b_mn, dtype, M, N, K, form):
    from pfeife_b200.ops import kernels as kx
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned pitch")
    a, b = _mk(M, N, K, a_mn, b_mn, dtype)
    out = kx.gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=form)
    torch.cuda.synchronize()
    kx.check_status()
    _close(out, _ref(a, b, a_mn, b_mn), K, dtype)


# bit 10: direct-store epilogue, bit 11: CTA-pair form, bit 12: single-CTA form
@pytest.mark.parametrize("tile_n", [4096 + 128, 4096 + 256, 4096 + 1024 + 256, 2048, 2048 + 1024, 0])
def test_gemm_tile_variants_and_fp32_out(tile_n):
    from pfeife_b200.ops import kernels as kx
    a, b = _mk(520, 776, 320, False, False, torch.bfloat16)
    out = kx.gemm(a, b, out_dtype=torch.float32, tile_n=tile_n)
    torch.cuda.synchronize()
    _close(out, _ref(a, b, False, False), 320, torch.float32)


@pytest.mark.parametrize("tile_n", [4096, 4096 + 1024, 2048, 2048 + 1024])
@pytest.mark.parametrize("M,N,K", [(400, 384, 192), (6168, 1408, 320)])
def test_gemm_epilogues(tile_n, M, N, K):
    """Every fused epilogue through the TMA-store path and the direct-store path (bit 10), on
    single-CTA tiles (bit 12) and on CTA-pair tiles (bit 11)."""
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


@pytest.mark.parametrize("M,N,K", [(512, 512, 4096), (1408, 1408, 6168), (304, 704, 2048)])
@pytest.mark.parametrize("form", [0, 4096])
def test_gemm_accumulate_with_split_reduction(M, N, K, form):
    """Few output tiles and a long reduction: the gradient-accumulating GEMM divides each tile's
    k-blocks among several work items that all add into the fp32 output."""
    from pfeife_b200.ops import kernels as kx
    a, b = _mk(M, N, K, True, True, torch.bfloat16, seed=3)
    a, b = a * 0.1, b * 0.1
    out = torch.full((M, N), 0.5, device="cuda")
    kx.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, tile_n=form)
    kx.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, tile_n=form)
    torch.cuda.synchronize()
    kx.check_status()
    _close(out, 0.5 + 2.0 * _ref(a, b, True, True), K, torch.float32)


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


@pytest.mark.parametrize("world,rank,ends", [(2, 0, None), (2, 1, None), (4, 2, None),
                                             (3, 1, (500, 1100, 1536)), (2, 1, (1536, 1536))])
def test_gemm_allgather_one_device(world, rank, ends):
    """The all-gather GEMM with every "peer" copy on this GPU: one launch copies the rows the
    other ranks own into the local weight while it computes, and the product must match
    x @ W^T.  Each copy is current only in the rows its rank owns (the rest is poisoned)."""
    from pfeife_b200.ops import kernels as kx
    from pfeife_b200.parallel.dp_fused import _table
    M, N, K = 700, 1536, 320
    ends = ends or tuple((r + 1) * (N // world) for r in range(world))
    starts = (0,) + tuple(ends[:-1])
    torch.manual_seed(world * 10 + rank)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    copies = []
    for r in range(world):
        c = torch.full_like(w, float("nan"))
        c[starts[r]:ends[r]] = w[starts[r]:ends[r]]
        copies.append(c)
    w_full = copies[rank]
    ready = torch.zeros((N + 255) // 256 + 1, dtype=torch.int32, device="cuda")
    out = kx.gemm_allgather(x, w_full, _table([c.data_ptr() for c in copies]), world, rank, ends,
                            ready)
    torch.cuda.synchronize()
    kx.check_status()
    assert torch.equal(w_full, w)
    assert int(ready[-1]) == N - (ends[rank] - starts[rank])
    _close(out, x.float() @ w.float().t(), K, torch.bfloat16)


def test_gather_rows_one_device():
    """Stand-alone row gather: rows owned by the other ranks arrive from their copies."""
    from pfeife_b200.ops import kernels as kx
    from pfeife_b200.parallel.dp_fused import _table
    N, K, world, rank = 1000, 264, 4, 2
    ends = (100, 400, 650, 1000)
    starts = (0,) + ends[:-1]
    w = torch.randn(N, K, device="cuda").to(torch.float16)
    copies = []
    for r in range(world):
        c = torch.zeros_like(w)
        c[starts[r]:ends[r]] = w[starts[r]:ends[r]]
        copies.append(c)
    kx.gather_rows(copies[rank], _table([c.data_ptr() for c in copies]), world, rank, ends)
    torch.cuda.synchronize()
    assert torch.equal(copies[rank], w)

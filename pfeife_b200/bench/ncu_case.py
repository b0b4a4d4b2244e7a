"""Small single-kernel workloads for Nsight Compute captures (a few launches, inputs larger than
L2, a few hundred MB on the device at most).

    python -m pfeife_b200.bench.ncu_case {gemm,gemm_plain,gemm_plain_single,gemm_plain_pair,gemm_wgrad,attn,attn_unet,attn_llama,norm,adamw,ce,unet,llama}

Each case launches its kernel(s) a handful of times and checks the kernel status word, so the
same command can first be run plainly (must exit 0) and then under
``ncu --clock-control none -k regex:<kernel> -c <n>``.
"""
from __future__ import annotations

import math
import sys

import torch


def main(argv=None) -> int:
    which = (argv or sys.argv[1:] or ["gemm"])[0]
    from pfeife_b200.ops import kernels as kx
    dev = "cuda"
    torch.manual_seed(0)
    reps = 4
    if which == "gemm":       # ViT-g/14 fc1 forward with the bias + GELU (+aux) epilogue
        M, N, K = 6168, 6144, 1408
        a = torch.randn(M, K, device=dev).to(torch.float16)
        b = torch.randn(N, K, device=dev).to(torch.float16) * 0.02
        bias = torch.zeros(N, device=dev)
        out = torch.empty(M, N, device=dev, dtype=torch.float16)
        aux = torch.empty_like(out)
        for _ in range(reps):
            kx.gemm(a, b, out=out, bias=bias, aux=aux, epilogue=kx.EPI_GELU)
    elif which in ("gemm_plain", "gemm_plain_single", "gemm_plain_pair"):
        # same shape, no epilogue work; tile form chosen by the library, or forced
        M, N, K = 6168, 6144, 1408
        a = torch.randn(M, K, device=dev).to(torch.float16)
        b = torch.randn(N, K, device=dev).to(torch.float16) * 0.02
        out = torch.empty(M, N, device=dev, dtype=torch.float16)
        form = 4096 if which.endswith("single") else 2048 if which.endswith("pair") else 0
        for _ in range(reps):
            kx.gemm(a, b, out=out, tile_n=form)
    elif which == "gemm_wgrad":   # both operands MN-major, fp32 accumulate into the bucket
        M, N, K = 6144, 1408, 6168
        a = torch.randn(K, M, device=dev).to(torch.float16)
        b = torch.randn(K, N, device=dev).to(torch.float16)
        out = torch.zeros(M, N, device=dev)
        for _ in range(reps):
            kx.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    elif which == "attn":     # ViT-g/14 attention, forward and backward
        B, S, H, D = 24, 257, 16, 88
        qkv = (torch.randn(B, S, 3, H, D, device=dev) * 0.5).to(torch.float16)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        do = torch.randn(B, S, H, D, device=dev).to(torch.float16)
        for _ in range(reps):
            o, lse = kx.attn_fwd(q, k, v, False, 1 / math.sqrt(D))
            kx.attn_bwd(do, q, k, v, o, lse, False, 1 / math.sqrt(D), packed=True)
    elif which in ("attn_unet", "attn_llama"):   # long sequences: many key tiles per query tile
        B, S, H, D, causal = (2, 4096, 10, 64, False) if which == "attn_unet" else \
            (1, 2048, 32, 128, True)
        q, k, v, do = (torch.randn(B, S, H, D, device=dev).to(torch.bfloat16) for _ in range(4))
        for _ in range(reps):
            o, lse = kx.attn_fwd(q, k, v, causal, 1 / math.sqrt(D))
            kx.attn_bwd(do, q, k, v, o, lse, causal, 1 / math.sqrt(D))
    elif which == "norm":
        rows, N = 49344, 1408
        x = torch.randn(rows, N, device=dev).to(torch.float16)
        g, b = torch.ones(N, device=dev), torch.zeros(N, device=dev)
        for _ in range(reps):
            y, h, mean, rstd = kx.norm_fwd(x, g, b, 1e-12, False)
            kx.norm_bwd(x, x, g, mean, rstd, False)
    elif which == "adamw":
        n = 64 << 20
        p, g, m, v = (torch.zeros(n, device=dev) for _ in range(4))
        lp = torch.empty(n, device=dev, dtype=torch.float16)
        for step in range(1, reps + 1):
            kx.adamw(p, g, m, v, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                     step=step, lp=lp)
    elif which == "ce":
        rows, V = 4096, 32000
        logits = torch.randn(rows, V, device=dev).to(torch.bfloat16)
        tgt = torch.randint(0, V, (rows,), device=dev)
        for _ in range(reps):
            loss, lse = kx.ce_fwd(logits, tgt)
            kx.ce_bwd(logits, tgt, lse, torch.full((rows,), 1.0 / rows, device=dev))
    elif which == "unet":     # SDXL UNet block kernels: GroupNorm+SiLU fwd/bwd, im2col, col2im
        B, H, W, C = 4, 64, 64, 640
        x = torch.randn(B, H, W, C, device=dev).to(torch.bfloat16)
        g, b = torch.ones(C, device=dev), torch.zeros(C, device=dev)
        for _ in range(reps):
            y, mean, rstd = kx.groupnorm_fwd(x, g, b, 32, 1e-5, True)
            kx.groupnorm_bwd(y, x, mean, rstd, g, b, 32, True)
            cols = kx.im2col(x, 3, 3, 1, 1)
            kx.col2im(cols, (B, H, W, C), 3, 3, 1, 1)
    elif which == "llama":    # Llama-2-7B elementwise kernels: SwiGLU fwd/bwd, RoPE, embedding
        rows, Hd = 2048, 11008
        gu = torch.randn(rows, 2 * Hd, device=dev).to(torch.bfloat16)
        do = torch.randn(rows, Hd, device=dev).to(torch.bfloat16)
        q = torch.randn(1, 2048, 32, 128, device=dev).to(torch.bfloat16)
        ang = torch.rand(2048, 64, device=dev)
        table = torch.randn(32000, 4096, device=dev)
        ids = torch.randint(0, 32000, (8, 2048), device=dev)
        for _ in range(reps):
            kx.glu_fwd(gu, False)
            kx.glu_bwd(gu, do, False)
            kx.rope(q, ang.cos(), ang.sin())
            kx.embed_fwd(table, ids, torch.bfloat16)
    else:
        print(f"unknown case {which}", file=sys.stderr)
        return 2
    torch.cuda.synchronize()
    kx.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Kernel micro-benchmarks with roofline fractions.

    python -m pfeife_b200.bench.kernels [--which gemm,conv,norm,adamw,attn,groupnorm,rope]
                                        [--json out.jsonl]

Timing: CUDA events on the launching stream, 3 warm-up launches, L2 flushed between timed
launches by writing a 256 MiB buffer, median of `--iters`.  Fractions are against the measured
peaks in MEASURED_PEAKS.json at the repository root when present ("of measured"), else against
the fallback 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


class Timer:
    def __init__(self, iters=10):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)


def bench_gemm(timer, out):
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    shapes = [  # (name, M, N, K, a_mn, b_mn)
        ("vitg_qkv_fwd", 6168, 4224, 1408, False, False),
        ("vitg_fc1_fwd", 6168, 6144, 1408, False, False),
        ("vitg_fc2_fwd", 6168, 1408, 6144, False, False),
        ("vitg_proj_fwd", 6168, 1408, 1408, False, False),
        ("vitg_fc2_dgrad", 6168, 6144, 1408, False, True),
        ("vitg_fc1_dgrad", 6168, 1408, 6144, False, True),
        ("vitg_fc1_wgrad", 6144, 1408, 6168, True, True),
        ("llama_ffn_fwd", 2048, 11008, 4096, False, False),
        ("square_8192", 8192, 8192, 8192, False, False),
    ]
    for name, M, N, K, a_mn, b_mn in shapes:
        for dtype in (torch.bfloat16,):
            a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(dtype)
            b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(dtype)
            c = torch.empty(M, N, device="cuda", dtype=dtype)
            ms = timer(lambda: kx.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c))
            # the two tile forms on their own (bit 12: single-CTA tiles, bit 11: CTA pairs)
            ms_single = timer(lambda: kx.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c, tile_n=4096))
            ms_pair = timer(lambda: kx.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=c, tile_n=2048))
            A = a.t() if a_mn else a
            Bt = b if b_mn else b.t()
            ms_ref = timer(lambda: torch.matmul(A, Bt, out=c))
            tfl = 2.0 * M * N * K / ms / 1e9
            out({"kernel": "gemm_tcgen05", "case": name, "M": M, "N": N, "K": K, "ms": ms,
                 "tflops": tfl, "frac_peak": tfl / tf, "peak_ref": tag,
                 "ms_single_cta": ms_single, "ms_cta_pair": ms_pair,
                 "torch_matmul_ms": ms_ref, "vs_torch": ms_ref / ms})


def bench_conv(timer, out):
    """SDXL UNet 3x3 convolutions (NHWC, bf16): implicit GEMM vs im2col + GEMM vs cuDNN."""
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    shapes = [("sdxl_320_128", 4, 128, 320, 320), ("sdxl_640_64", 4, 64, 640, 640),
              ("sdxl_1280_32", 4, 32, 1280, 1280), ("sdxl_up_1920_640_64", 4, 64, 1920, 640)]
    for name, B, HW, Cin, Cout in shapes:
        x = torch.randn(B, HW, HW, Cin, device="cuda").to(torch.bfloat16)
        w = (torch.randn(Cout, Cin, 3, 3, device="cuda") * 0.02).to(torch.bfloat16)
        w2 = w.permute(0, 2, 3, 1).reshape(Cout, 9 * Cin).contiguous()
        ms = timer(lambda: kx.conv_gemm(x, w2, 3, 3, 1, 1))
        ms_cols = timer(lambda: kx.gemm(kx.im2col(x, 3, 3, 1, 1), w2))
        xn = x.permute(0, 3, 1, 2)     # channels-last view for cuDNN
        wn = w.contiguous(memory_format=torch.channels_last)
        ms_ref = timer(lambda: torch.nn.functional.conv2d(xn, wn, padding=1))
        flops = 2.0 * B * HW * HW * Cout * 9 * Cin
        out({"kernel": "conv_implicit_gemm", "case": name, "ms": ms, "tflops": flops / ms / 1e9,
             "frac_peak": flops / ms / 1e9 / tf, "peak_ref": tag, "ms_im2col_gemm": ms_cols,
             "torch_conv2d_ms": ms_ref, "vs_torch": ms_ref / ms})


def bench_norm(timer, out):
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    for rows, N in ((6168 * 8, 1408), (2048 * 16, 4096)):
        x = torch.randn(rows, N, device="cuda").to(torch.bfloat16)
        g = torch.ones(N, device="cuda")
        b = torch.zeros(N, device="cuda")
        ms = timer(lambda: kx.norm_fwd(x, g, b, 1e-5, False))
        gb = 2 * x.numel() * 2 / 1e9
        out({"kernel": "layernorm_fwd", "rows": rows, "N": N, "ms": ms, "gbs": gb / ms * 1e3,
             "frac_peak": gb / ms * 1e3 / hbm, "peak_ref": tag})
        y, h, mean, rstd = kx.norm_fwd(x, g, b, 1e-5, False)
        ms = timer(lambda: kx.norm_bwd(x, h, g, mean, rstd, False))
        gb = 3 * x.numel() * 2 / 1e9
        out({"kernel": "layernorm_bwd", "rows": rows, "N": N, "ms": ms, "gbs": gb / ms * 1e3,
             "frac_peak": gb / ms * 1e3 / hbm, "peak_ref": tag})


def bench_attn(timer, out):
    """Flash attention forward / backward against ``F.scaled_dot_product_attention`` on the
    shapes of the benchmark models: ViT-g/14 (d = 88), Llama-2-7B (causal, d = 128), the SDXL
    UNet's self-attention at 64x64 and 32x32 latents and its cross-attention (77 text tokens)."""
    import torch.nn.functional as F
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    shapes = [("vitg", 24, 16, 257, 257, 88, False), ("llama7b", 1, 32, 2048, 2048, 128, True),
              ("unet_64x64", 4, 10, 4096, 4096, 64, False), ("unet_32x32", 4, 20, 1024, 1024, 64, False),
              ("unet_cross_77", 4, 20, 1024, 77, 64, False)]
    for name, B, H, Sq, Sk, D, causal in shapes:
        dtype = torch.bfloat16
        q = torch.randn(B, Sq, H, D, device="cuda").to(dtype)
        k = torch.randn(B, Sk, H, D, device="cuda").to(dtype)
        v = torch.randn(B, Sk, H, D, device="cuda").to(dtype)
        do = torch.randn(B, Sq, H, D, device="cuda").to(dtype)
        scale = D ** -0.5
        ms_f = timer(lambda: kx.attn_fwd(q, k, v, causal, scale))
        o, lse = kx.attn_fwd(q, k, v, causal, scale)
        ms_b = timer(lambda: kx.attn_bwd(do, q, k, v, o, lse, causal, scale))
        # SDPA wants [B, H, S, D]; the transposed views cost it nothing (strided inputs)
        qt, kt, vt = (t.transpose(1, 2).detach().requires_grad_() for t in (q, k, v))
        ms_rf = timer(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal))
        ot = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal)
        dot = do.transpose(1, 2)
        ms_rb = timer(lambda: torch.autograd.grad(ot, (qt, kt, vt), dot, retain_graph=True))
        frac = 0.5 if causal else 1.0
        fl = 4.0 * B * H * Sq * Sk * D * frac
        out({"kernel": "flash_attention", "case": name, "B": B, "H": H, "Sq": Sq, "Sk": Sk, "D": D,
             "causal": causal, "fwd_ms": ms_f, "bwd_ms": ms_b, "fwd_tflops": fl / ms_f / 1e9,
             "bwd_tflops": 2.5 * fl / ms_b / 1e9, "sdpa_fwd_ms": ms_rf, "sdpa_bwd_ms": ms_rb,
             "fwd_vs_sdpa": ms_rf / ms_f, "bwd_vs_sdpa": ms_rb / ms_b, "peak_ref": tag})


def bench_groupnorm(timer, out):
    """GroupNorm(32) + SiLU on NHWC activations of the SDXL UNet, forward and backward, against
    ``F.group_norm`` + ``F.silu`` on channels-last tensors."""
    import torch.nn.functional as F
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    for name, B, HW, C in (("sdxl_320_128", 4, 128, 320), ("sdxl_640_64", 4, 64, 640),
                           ("sdxl_1280_32", 4, 32, 1280), ("sdxl_1920_64", 4, 64, 1920)):
        x = torch.randn(B, HW, HW, C, device="cuda").to(torch.bfloat16)
        g = torch.ones(C, device="cuda")
        b = torch.zeros(C, device="cuda")
        dy = torch.randn_like(x)
        ms_f = timer(lambda: kx.groupnorm_fwd(x, g, b, 32, 1e-5, True))
        y, mean, rstd = kx.groupnorm_fwd(x, g, b, 32, 1e-5, True)
        ms_b = timer(lambda: kx.groupnorm_bwd(dy, x, mean, rstd, g, b, 32, True))
        xn = x.permute(0, 3, 1, 2).detach().requires_grad_()
        gh, bh = g.to(x.dtype), b.to(x.dtype)       # ATen wants the affine terms in x's dtype
        ms_rf = timer(lambda: F.silu(F.group_norm(xn, 32, gh, bh, 1e-5)))
        yr = F.silu(F.group_norm(xn, 32, gh, bh, 1e-5))
        dyn = dy.permute(0, 3, 1, 2)
        ms_rb = timer(lambda: torch.autograd.grad(yr, xn, dyn, retain_graph=True))
        nb = x.numel() * 2
        out({"kernel": "groupnorm_silu", "case": name, "fwd_ms": ms_f, "bwd_ms": ms_b,
             "fwd_gbs": 2 * nb / ms_f / 1e6, "bwd_gbs": 3 * nb / ms_b / 1e6,
             "fwd_frac_peak": 2 * nb / ms_f / 1e6 / hbm, "bwd_frac_peak": 3 * nb / ms_b / 1e6 / hbm,
             "torch_fwd_ms": ms_rf, "torch_bwd_ms": ms_rb, "fwd_vs_torch": ms_rf / ms_f,
             "bwd_vs_torch": ms_rb / ms_b, "peak_ref": tag})


def bench_rope(timer, out):
    from pfeife_b200.ops import functional as Fn
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    B, S, H, D = 16, 2048, 32, 128
    x = torch.randn(B, S, H, D, device="cuda").to(torch.bfloat16)
    cos, sin = Fn.rope_tables(S, D, device="cuda")
    ms = timer(lambda: kx.rope(x, cos, sin))
    gb = 2 * x.numel() * 2 / 1e9
    out({"kernel": "rope", "shape": [B, S, H, D], "ms": ms, "gbs": gb / ms * 1e3,
         "frac_peak": gb / ms * 1e3 / hbm, "peak_ref": tag})


def bench_adamw(timer, out):
    from pfeife_b200.ops import kernels as kx
    hbm, tf, tag = peaks()
    n = 256 << 20
    p, g, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = timer(lambda: kx.adamw(p, g, m, v, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8,
                                weight_decay=0.01, step=1, lp=lp))
    gb = n * (4 * 4 + 4 * 4 + 2) / 1e9
    out({"kernel": "adamw_fused", "n": n, "ms": ms, "gbs": gb / ms * 1e3,
         "frac_peak": gb / ms * 1e3 / hbm, "peak_ref": tag})


def bench_dp_local(timer, out):
    """The fused data-parallel step with a world of one rank: its local part (read the
    gradient, AdamW, write moments, master, 16-bit weights, clear the gradient) without any
    peer traffic, against the stand-alone optimizer kernel's rate."""
    from pfeife_b200.parallel.dp_fused import _table, launch_fused_step
    hbm, tf, tag = peaks()
    n = 256 << 20
    g, w, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    local_sync = torch.zeros(4, dtype=torch.int32, device="cuda")
    found = torch.zeros(1, device="cuda")
    applied = torch.zeros(1, dtype=torch.int32, device="cuda")
    state = {"epoch": 1, "arrivals": 0}

    def run():
        nbar, grid = launch_fused_step(
            0, 1, _table([g.data_ptr()]), _table([w.data_ptr()]), _table([lp.data_ptr()]),
            _table([flags.data_ptr()]), m, v, local_sync, (0, n), n, [(0, n, 0, 0)],
            [(1e-3, 0.9, 0.999, 1e-8, 0.01, True)], applied, 1, 1.0, lp.dtype, check_inf=False,
            found_given=False, loss_scale=None, found_inf=found, epoch=state["epoch"],
            arrivals=state["arrivals"], device=torch.device("cuda", 0))
        state["epoch"] += nbar
        state["arrivals"] += nbar * grid

    ms = timer(run)
    gb = n * (4 * 4 + 4 * 4 + 2) / 1e9
    out({"kernel": "dp_fused_world1", "n": n, "ms": ms, "gbs": gb / ms * 1e3,
         "frac_peak": gb / ms * 1e3 / hbm, "peak_ref": tag})


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", default="gemm,norm,adamw")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    sink = open(a.json, "w") if a.json else None

    def out(rec):
        line = json.dumps(rec)
        print(line, flush=True)
        if sink:
            sink.write(line + "\n")

    timer = Timer(a.iters)
    table = {"gemm": bench_gemm, "conv": bench_conv, "norm": bench_norm, "adamw": bench_adamw,
             "attn": bench_attn, "groupnorm": bench_groupnorm, "rope": bench_rope,
             "dp_local": bench_dp_local}
    for k in a.which.split(","):
        table[k](timer, out)
    from pfeife_b200.ops import kernels as kx
    kx.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Fused all-gather + GEMM over peer memory, one process per GPU (run under ``mp_launch.py
--all_main``): every rank owns a row shard of W, the kernel gathers the rest while computing,
and the result must equal x @ W^T with the full W.  Also times the fused kernel against
"NCCL all-gather, then the same GEMM" and reports the fraction of the roofline
max(FLOPs / measured GEMM peak, remote bytes / 770 GB/s)."""
import argparse
import ctypes
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from pfeife_b200 import initialize_pfeife  # noqa
from pfeife_b200.ops import kernels as kx  # noqa
from pfeife_b200.parallel.dp_fused import PeerMemory, _table  # noqa


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--M", type=int, default=6168)
    ap.add_argument("--N", type=int, default=6144)
    ap.add_argument("--K", type=int, default=1408)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    st = initialize_pfeife(dp_mesh=f"-{int(os.environ['WORLD_SIZE'])},1")
    dev, W, r = st.device, st.world_size, st.rank
    M, N, K = a.M, a.N, a.K
    rows = N // W
    g = torch.Generator(device="cpu").manual_seed(0)
    w_all = (torch.randn(N, K, generator=g) * 0.05).to(torch.float16)
    x = torch.randn(M, K, generator=g).to(torch.float16).to(dev)
    shard = w_all[r * rows:(r + 1) * rows].contiguous().to(dev)
    # every rank's copy of W is full size and current only in the rows the rank owns
    w_full = torch.zeros(N, K, dtype=torch.float16, device=dev)
    w_full[r * rows:(r + 1) * rows] = shard
    ends = [(i + 1) * rows for i in range(W)]
    ends[-1] = N
    ready = torch.zeros((N + 255) // 256 + 1, dtype=torch.int32, device=dev)
    peers = PeerMemory(st.ctrl_dp, W, r)
    table = _table(peers.share(w_full))
    torch.cuda.synchronize()
    dist.barrier()
    out = kx.gemm_allgather(x, w_full, table, W, r, ends, ready)
    torch.cuda.synchronize()
    kx.check_status()
    ref = x.float() @ w_all.to(dev).float().t()
    err = float((out.float() - ref).abs().max())
    gathered_ok = bool(torch.equal(w_full.cpu(), w_all))
    dist.barrier()    # nobody clears its copy below while a peer may still be reading it

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def fused():
        w_full[:r * rows].zero_()
        w_full[(r + 1) * rows:].zero_()
        kx.gemm_allgather(x, w_full, table, W, r, ends, ready, out=out)

    gathered = torch.empty(N, K, dtype=torch.float16, device=dev)

    def baseline():
        dist.all_gather_into_tensor(gathered, shard, group=st.dp_group)
        kx.gemm(x, gathered, out=out)

    def clear_only():
        w_full[:r * rows].zero_()
        w_full[(r + 1) * rows:].zero_()

    ms_fused = timed(fused) - timed(clear_only)
    ms_base = timed(baseline)
    flops = 2.0 * M * N * K
    remote = (W - 1) * rows * K * 2
    roof_ms = max(flops / 1418.6e12, remote / 770e9) * 1e3
    res = {"err": err, "gathered_ok": gathered_ok, "ms_fused": ms_fused, "ms_nccl_then_gemm": ms_base,
           "roofline_ms": roof_ms, "frac_of_roofline": roof_ms / ms_fused, "world": W,
           "shape": [M, N, K]}
    if st.is_main_process:
        with open(a.out, "w") as f:
            json.dump(res, f)
        print(json.dumps(res))
    dist.barrier()


if __name__ == "__main__":
    main()

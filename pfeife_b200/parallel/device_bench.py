"""Link model: measured point-to-point transfer time between every pair of ranks, fitted to

    t(ms) = c                      if MiB <= x_break
            m * (MiB - x_break) + c otherwise

and cached as ``pickle.dump({(rank_i, rank_j): (c, m, x_break)})`` with i < j (the file format of
pfeife/device_bench.py:153-185, lookup symmetric as in :47-53).  Message sizes follow the
reference grid: fp32 tensors ``b x w x h``, b in {1,2,4}, w,h in {100,400,800,3200}
(40 KB ... 164 MB), 10 timed transfers each after warm-up.

Flavours: ``DeviceBench`` (one process, device-to-device copies between local GPUs),
``NCCLDeviceBench`` (one process per rank; send/recv over the data-plane group, works with gloo
on CPU too; rank 0 writes the file, the others load it).  On one NVSwitch box every pair sees
the same link, so ``uniform=True`` measures pair (0, 1) only and replicates the triple.
"""
from __future__ import annotations

import os
import pickle
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..utils import get_logger

MB = 1024 ** 2
BENCH_CNT = 10
WARM_CNT = 3
DEFAULT_OFFSET = 0.0
Triple = Tuple[float, float, float]

_B = (1, 2, 4)
_WH = (100, 400, 800, 3200)


def bench_sizes() -> List[Tuple[int, int, int]]:
    return [(b, w, h) for b in _B for w in _WH for h in _WH]


def biased_relu(x, c, m, x_break):
    return np.where(x <= x_break, c, m * (x - x_break) + c)


def fit_link(sizes_mb: Sequence[float], times_ms: Sequence[float]) -> Triple:
    """Least-squares fit of the piecewise model; falls back to a robust closed form when scipy
    is unavailable or the fit does not converge."""
    x = np.asarray(sizes_mb, dtype=np.float64)
    y = np.asarray(times_ms, dtype=np.float64)
    c0 = float(np.min(y))
    big = x >= np.percentile(x, 60)
    m0 = float(np.polyfit(x[big], y[big], 1)[0]) if big.sum() >= 2 else float(y.max() / x.max())
    m0 = max(m0, 1e-9)
    try:
        from scipy.optimize import curve_fit
        (c, m, xb), _ = curve_fit(biased_relu, x, y, p0=(c0, m0, float(x.min())),
                                  bounds=((0.0, 0.0, 0.0), (np.inf, np.inf, float(x.max()))))
        return float(c), float(m), float(xb)
    except Exception:
        return c0, m0, max(0.0, c0 / m0 * 0.0)


class DeviceBench:
    """Link model + single-process measurement (device-to-device copies)."""

    def __init__(self, devices: Sequence = (), option=None):
        self.devices = [torch.device(d) for d in devices]
        self.option = option
        self.params: Dict[Tuple[int, int], Triple] = {}

    # ---------------------------------------------------------------- model
    def set_uniform(self, n: int, triple: Triple) -> None:
        self.params = {(i, j): triple for i in range(n) for j in range(i + 1, n)}

    def send_time(self, key: Tuple[int, int], nbytes: float) -> float:
        c, m, xb = self.params[key]
        mb = nbytes / MB
        return c if mb <= xb else m * (mb - xb) + c

    def send_time_rank(self, r1: int, r2: int, nbytes: float) -> float:
        if r1 == r2:
            return 0.0
        key = (r1, r2) if r1 < r2 else (r2, r1)
        if key not in self.params:
            if not self.params:
                return DEFAULT_OFFSET
            key = next(iter(self.params))
        return self.send_time(key, nbytes)

    # ---------------------------------------------------------------- file
    def load(self, path: str) -> bool:
        if path and os.path.exists(path):
            with open(path, "rb") as f:
                self.params = pickle.load(f)
            return True
        return False

    def save(self, path: str) -> None:
        if path:
            d = os.path.dirname(os.path.abspath(path))
            os.makedirs(d, exist_ok=True)
            with open(path, "wb") as f:
                pickle.dump(self.params, f)

    # ---------------------------------------------------------------- measurement
    def _time_pair(self, i: int, j: int) -> Triple:
        src, dst = self.devices[i], self.devices[j]
        xs, ys = [], []
        for b, w, h in bench_sizes():
            a = torch.empty(b, w, h, device=src)
            o = torch.empty(b, w, h, device=dst)
            cuda = src.type == "cuda"
            for _ in range(WARM_CNT):
                o.copy_(a, non_blocking=True)
            if cuda:
                torch.cuda.synchronize(src)
                torch.cuda.synchronize(dst)
            t0 = time.perf_counter()
            for _ in range(BENCH_CNT):
                o.copy_(a, non_blocking=True)
            if cuda:
                torch.cuda.synchronize(src)
                torch.cuda.synchronize(dst)
            ys.append((time.perf_counter() - t0) * 1e3 / BENCH_CNT)
            xs.append(a.numel() * 4 / MB)
        return fit_link(xs, ys)

    def run_bench(self, file_path: Optional[str] = None, uniform: bool = False) -> None:
        if self.load(file_path):
            return
        n = len(self.devices)
        if n < 2:
            self.params = {}
        elif uniform:
            self.set_uniform(n, self._time_pair(0, 1))
        else:
            self.params = {(i, j): self._time_pair(i, j) for i in range(n)
                           for j in range(i + 1, n)}
        self.save(file_path)


class NCCLDeviceBench(DeviceBench):
    """One process per rank.  Every rank calls ``run_bench``; pairs are measured one at a time
    over ``group`` (NCCL on GPUs, gloo on CPU) with device-side timing on the sender."""

    def __init__(self, rank: int, ranks: Sequence[int], device: torch.device, group=None,
                 option=None):
        super().__init__([], option)
        self.rank, self.ranks, self.device, self.group = rank, list(ranks), device, group

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _pair_times(self, a: int, b: int) -> Optional[Triple]:
        me = self.rank
        xs, ys = [], []
        for bb, w, h in bench_sizes():
            if me not in (a, b):
                continue
            t = torch.empty(bb, w, h, device=self.device)
            xs.append(t.numel() * 4 / MB)
            for phase, cnt in (("warm", WARM_CNT), ("time", BENCH_CNT)):
                self._sync()
                t0 = time.perf_counter()
                for _ in range(cnt):
                    if me == a:
                        dist.send(t, b, group=self.group)
                    else:
                        dist.recv(t, a, group=self.group)
                self._sync()
                if phase == "time":
                    ys.append((time.perf_counter() - t0) * 1e3 / cnt)
        if me == b:
            return fit_link(xs, ys)
        return None

    def run_bench(self, file_path: Optional[str] = None, uniform: bool = True) -> None:
        log = get_logger()
        if file_path and os.path.exists(file_path):
            self.load(file_path)
            return
        n = len(self.ranks)
        pairs = [(0, 1)] if (uniform and n >= 2) else [(i, j) for i in range(n)
                                                       for j in range(i + 1, n)]
        local: Dict[Tuple[int, int], Triple] = {}
        for i, j in pairs:
            r = self._pair_times(self.ranks[i], self.ranks[j])
            if r is not None:
                local[(i, j)] = r
        gathered: List[Optional[dict]] = [None] * n
        dist.all_gather_object(gathered, local, group=self.group) if n > 1 else None
        merged: Dict[Tuple[int, int], Triple] = {}
        for d in gathered:
            if d:
                merged.update(d)
        if uniform and n >= 2 and merged:
            self.set_uniform(n, merged[(0, 1)])
        else:
            self.params = merged
        if self.rank == self.ranks[0]:
            self.save(file_path)
            if self.params:
                k = next(iter(self.params))
                c, m, xb = self.params[k]
                log.info("link model %s: c=%.4f ms, m=%.5f ms/MiB (%.1f GB/s), break %.3f MiB",
                         k, c, m, (MB / 1e9) / (m / 1e3) if m > 0 else float("inf"), xb)


def nvswitch_default(n: int, gbs: float = 700.0, latency_ms: float = 0.02) -> DeviceBench:
    """Analytic stand-in for one NVSwitch box when no measurement is wanted."""
    b = DeviceBench()
    b.set_uniform(max(n, 2), (latency_ms, (MB / 1e9) / gbs * 1e3, 0.0))
    return b


def main(argv=None) -> int:
    """``python -m pfeife_b200.parallel.device_bench --out FILE [--nccl]``: measure and print."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--nccl", action="store_true", help="one process per rank (torchrun)")
    ap.add_argument("--all_pairs", action="store_true")
    a = ap.parse_args(argv)
    if a.nccl:
        from ..topology import initialize_pfeife
        st = initialize_pfeife()
        b = NCCLDeviceBench(st.rank, list(range(st.world_size)), st.device)
        b.run_bench(a.out, uniform=not a.all_pairs)
        if st.rank == 0:
            print(b.params)
    else:
        n = torch.cuda.device_count()
        b = DeviceBench([f"cuda:{i}" for i in range(n)])
        b.run_bench(a.out, uniform=not a.all_pairs)
        print(b.params)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

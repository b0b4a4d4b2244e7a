"""Fused data-parallel path: the gradient reduce-scatter, unscale, non-finite agreement,
partitioned AdamW and the all-gather of the updated weights run as one hand-written kernel per
rank that reads and writes the other ranks' buffers directly over NVLink (csrc/dp_fused.cu).

Host side: the flat gradient / master / shadow buffers of ``RankParams`` are ordinary device
allocations whose CUDA IPC handles are exchanged once over the control group; every rank maps
its peers' buffers and keeps a table of peer pointers.  Optimizer moments exist only for the
rank's own shard (ZeRO-1), and so do current fp32 masters of the weights that are only ever read
through their 16-bit shadow (``gather_master`` completes them for checkpoints).  The kernel's cross-GPU barriers are epoch counters in a small
peer-visible flag buffer.

Optimizers other than Adam / AdamW fall back to the NCCL path.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import kernels as kx
from ..ops._lib import c_f, c_ll, check, dt, ptr, sm_count, stream
from .dp import NcclDP

DP_MAX = 8
DP_MAX_GROUPS = 8
ALIGN = 128


class PeerMemory:
    """Maps the peers' copies of local device tensors.  All ranks call ``share`` with tensors
    in the same order."""

    def __init__(self, ctrl_group, size: int, rank: int):
        self.ctrl_group, self.size, self.rank = ctrl_group, size, rank
        self._opened: Dict[Tuple[int, bytes], int] = {}

    def share(self, t: torch.Tensor) -> List[int]:
        """-> per-rank device pointers of `t` (own pointer at index ``rank``)."""
        L = _lib.lib()
        _lib.bind_thread()
        handle = ctypes.create_string_buffer(64)
        code = L.pf_ipc_get_handle(ctypes.c_void_p(t.data_ptr()), handle)
        if code:
            raise _lib.KernelError(f"cudaIpcGetMemHandle failed: {code}")
        base = ctypes.c_void_p()
        size = ctypes.c_longlong()
        code = L.pf_get_base(ctypes.c_void_p(t.data_ptr()), ctypes.byref(base), ctypes.byref(size))
        if code:
            raise _lib.KernelError(f"cuMemGetAddressRange failed: {code}")
        mine = (handle.raw, t.data_ptr() - (base.value or 0))
        everyone: List[Optional[Tuple[bytes, int]]] = [None] * self.size
        dist.all_gather_object(everyone, mine, group=self.ctrl_group)
        ptrs: List[int] = []
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            key = (r, h)
            if key not in self._opened:
                out = ctypes.c_void_p()
                code = L.pf_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(out))
                if code:
                    raise _lib.KernelError(f"cudaIpcOpenMemHandle(rank {r}) failed: {code}")
                self._opened[key] = out.value
            ptrs.append(self._opened[key] + off)
        self._verify(t, ptrs)
        return ptrs

    def _verify(self, t: torch.Tensor, ptrs: List[int]) -> None:
        """Checks every peer mapping end to end before any kernel trusts it: each rank
        publishes the first and last 32-bit word of its buffer, and every rank reads the same
        two words through its mapping of that peer (a copy-engine read, which reports an
        unmapped address as an error code)."""
        L = _lib.lib()
        nbytes = t.numel() * t.element_size()
        if nbytes < 8:
            return
        torch.cuda.synchronize(t.device)

        def peek(addr: int) -> int:
            out = ctypes.c_uint(0)
            code = L.pf_peek_u32(ctypes.c_void_p(addr), ctypes.byref(out))
            if code:
                raise _lib.KernelError(f"peer mapping unreadable at {addr:#x}: CUDA error {code}")
            return int(out.value)

        last = (nbytes - 4) // 4 * 4
        # stamp a rank-specific signature on both ends for the duration of the check (the
        # buffers may be all zeros, which would match any readable memory)
        raw = t.view(-1).view(torch.uint8)
        saved = (raw[:4].clone(), raw[last:last + 4].clone())
        sig = torch.tensor([0xA5, 0x5A, self.rank + 1, 0xC3], dtype=torch.uint8, device=t.device)
        raw[:4].copy_(sig)
        raw[last:last + 4].copy_(sig.flip(0))
        torch.cuda.synchronize(t.device)
        mine = (peek(t.data_ptr()), peek(t.data_ptr() + last), nbytes)
        everyone: List[Optional[Tuple[int, int, int]]] = [None] * self.size
        dist.all_gather_object(everyone, mine, group=self.ctrl_group)
        for r, (first_w, last_w, nb) in enumerate(everyone):
            if r == self.rank:
                continue
            if nb != nbytes:
                raise _lib.KernelError(f"rank {r} shares {nb} bytes, this rank {nbytes}")
            got = (peek(ptrs[r]), peek(ptrs[r] + last))
            if got != (first_w, last_w):
                raise _lib.KernelError(
                    f"peer mapping of rank {r} does not show that rank's data "
                    f"(read {got}, expected {(first_w, last_w)})")
        dist.barrier(group=self.ctrl_group)      # everyone has read before anyone restores
        raw[:4].copy_(saved[0])
        raw[last:last + 4].copy_(saved[1])
        torch.cuda.synchronize(t.device)


def _table(ptrs: List[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def shard_bounds(numel: int, world: int, matrices=()) -> List[int]:
    """Ownership boundaries [b_0 = 0, ..., b_world = numel] of the flat parameter buffer: an even
    split in units of ALIGN elements, except that a boundary falling inside one of `matrices`
    ((offset, cols, rows) of a weight whose 16-bit copy is gathered row by row) moves to the
    nearest boundary between two of its rows, so that every row has one owner."""
    per = (numel + world - 1) // world
    per = (per + ALIGN - 1) // ALIGN * ALIGN
    bounds = [min(numel, r * per) for r in range(world + 1)]
    bounds[world] = numel
    for i in range(1, world):
        b = bounds[i]
        for off, cols, rows in matrices:
            if off < b < off + rows * cols:
                b = off + int(round((b - off) / cols)) * cols
                break
        bounds[i] = max(bounds[i - 1], b)
    return bounds


def row_ends(offset: int, cols: int, rows: int, bounds: Sequence[int]) -> List[int]:
    """For a [rows, cols] matrix at `offset` of the flat buffer: row_end[r] such that rank r owns
    rows [row_end[r-1], row_end[r]) under the ownership `bounds`."""
    ends = []
    for r in range(len(bounds) - 1):
        hi = min(max(bounds[r + 1] - offset, 0), rows * cols)
        ends.append(hi // cols)
    ends[-1] = rows
    return ends


def launch_fused_step(rank: int, world: int, t_grad, t_master, t_lp, t_flags, m: torch.Tensor,
                      v: torch.Tensor, local_sync: torch.Tensor, shard: Tuple[int, int],
                      total: int, groups: Sequence[Tuple[int, int, int, int]],
                      hyper: Sequence[Tuple[float, float, float, float, float, bool]],
                      applied_steps: Optional[torch.Tensor], host_step: int, grad_scale: float,
                      lp_dtype: Optional[torch.dtype], check_inf: bool, found_given: bool,
                      loss_scale: Optional[torch.Tensor], found_inf: torch.Tensor, epoch: int,
                      arrivals: int, device, trace: Optional[torch.Tensor] = None
                      ) -> Tuple[int, int]:
    """One launch of the fused kernel on the current stream.  `t_*` are pointer tables
    (``_table``) with one entry per rank; `groups` holds (lo, hi, local_below, master_from) and
    `hyper` (lr, beta1, beta2, eps, weight_decay, adamw) per optimizer group.  Returns
    (barriers used, grid size): the caller adds them to its running epoch / arrival counts,
    which must be the same on every rank."""
    L = _lib.lib()
    flat_g = [int(x) for g in groups for x in g]
    flat_h = [float(x) for h in hyper for x in h]
    c_groups = (ctypes.c_longlong * len(flat_g))(*flat_g)
    c_hyper = (ctypes.c_float * len(flat_h))(*flat_h)
    nbar, grid = ctypes.c_int(0), ctypes.c_int(0)
    code = L.pf_dp_fused_step(
        int(rank), int(world), t_grad, t_master, t_lp, t_flags, ptr(m), ptr(v), ptr(local_sync),
        c_ll(shard[0]), c_ll(shard[1]), c_ll(total), len(groups), c_groups, c_hyper,
        ptr(applied_steps), int(host_step), c_f(grad_scale),
        dt(lp_dtype) if lp_dtype is not None else 0, int(check_inf), int(found_given),
        ptr(loss_scale), ptr(found_inf), int(epoch) & 0x7FFFFFFF, int(arrivals) & 0x7FFFFFFF,
        ctypes.byref(nbar), ctypes.byref(grid), ptr(kx.status_word(device)), ptr(trace),
        sm_count(device), stream())
    check(code, "pf_dp_fused_step")
    return nbar.value, grid.value


class FusedDP(NcclDP):
    fused = True

    def __init__(self, state, option):
        super().__init__(state, option)
        if self.size > DP_MAX:
            raise ValueError(f"fused data parallelism supports up to {DP_MAX} ranks")
        self.rank = state.dp_rank
        self.device = state.device
        self.peers = PeerMemory(state.ctrl_dp, self.size, self.rank)
        self.calls = 0
        self.params = None

    def attach(self, params) -> None:
        super().attach(params)          # replicas start from dp rank 0's values
        self.params = params
        if params.optimizer_type not in ("adam", "adamw") or not params.numel or \
                not params.native or len(params.group_ranges) > DP_MAX_GROUPS:
            self.fused = False
            return
        n = params.numel
        deferred = [s for s in params.slots.values() if getattr(s, "deferred", False)]
        bounds = shard_bounds(n, self.size, [(s.offset, s.entry.tensor.shape[1],
                                              s.entry.tensor.shape[0]) for s in deferred])
        self.bounds = bounds
        self.shard = (bounds[self.rank], bounds[self.rank + 1])
        ln = max(self.shard[1] - self.shard[0], 4)
        self.m = torch.zeros(ln, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(ln, dtype=torch.float32, device=self.device)
        params.dp_state = self      # checkpoints read / restore the sharded state through us
        self.flags = torch.zeros(2 * DP_MAX, dtype=torch.int32, device=self.device)
        self.local_sync = torch.zeros(4, dtype=torch.int32, device=self.device)
        # barrier bookkeeping, identical on every rank: epoch of the next call's first barrier
        # and the arrivals counted so far (both wrap; the kernel compares modulo 2^32)
        self.epoch, self.arrivals = 1, 0
        self.trace = torch.zeros(8, dtype=torch.int64, device=self.device)
        # fp32 masters are pushed to the peers only where some op reads them in fp32; without a
        # 16-bit shadow everything is read in fp32
        self.master_from = dict(params.master_from) if params.lp is not None else {}
        torch.cuda.synchronize(self.device)
        self.t_grad = _table(self.peers.share(params.grad))
        self.t_master = _table(self.peers.share(params.master))
        self.t_lp = _table(self.peers.share(params.lp)) if params.lp is not None else None
        self.t_flags = _table(self.peers.share(self.flags))
        self.deferred_below = dict(getattr(params, "deferred_below", {})) \
            if (deferred and self.t_lp is not None) else {}
        if deferred and self.t_lp is not None:
            from ..ops import functional as Fn
            es = params.lp.element_size()
            for s in deferred:
                rows, cols = s.entry.tensor.shape
                ends = tuple(row_ends(s.offset, cols, rows, bounds))
                copies = _table([int(base) + s.offset * es for base in self.t_lp])
                ready = torch.zeros((rows + 255) // 256 + 1, dtype=torch.int32,
                                    device=self.device)
                Fn.set_gather(s.master, Fn.GatherInfo(copies, ends, self.size, self.rank, ready))
        dist.barrier(group=self.state.ctrl_dp)

    def reduce_and_step(self, params, scaler, fp16: bool, found_agreed: bool = False) -> None:
        """One launch for the whole bucket (every optimizer group).  With ``found_agreed`` the
        non-finite decision in ``params.found_inf`` was already agreed over the whole job and
        the kernel only reads it; otherwise, under fp16, the replicas agree inside the kernel
        (enough for a job that is one pipeline stage wide)."""
        params.step_count += 1
        adamw = params.optimizer_type == "adamw"
        groups, hyper = [], []
        for g, lo, hi in params.group_ranges:
            h = params.hyper[min(g, len(params.hyper) - 1)]
            b1, b2 = h.get("betas", (0.9, 0.999))
            groups.append((lo, hi, self.deferred_below.get(g, lo), self.master_from.get(g, lo)))
            hyper.append((h.get("lr", 1e-3), b1, b2, h.get("eps", 1e-8),
                          h.get("weight_decay", 0.01 if adamw else 0.0), adamw))
        nbar, grid = launch_fused_step(
            self.rank, self.size, self.t_grad, self.t_master, self.t_lp, self.t_flags, self.m,
            self.v, self.local_sync, self.shard, params.numel, groups, hyper,
            params.applied_steps, params.step_count, 1.0 / self.size,
            params.lp.dtype if params.lp is not None else None,
            check_inf=bool(fp16 and not found_agreed), found_given=bool(fp16 and found_agreed),
            loss_scale=scaler.scale_tensor, found_inf=params.found_inf, epoch=self.epoch,
            arrivals=self.arrivals, device=self.device, trace=self.trace)
        self.epoch += nbar
        self.arrivals += nbar * grid
        self.calls += 1
        kx.step_advance(params.applied_steps, params.found_inf if fp16 else None)
        if fp16:
            scaler.update(params.found_inf)

    def phase_ms(self) -> Dict[str, float]:
        """Durations of the last fused step's phases on this rank (device timer): waiting at the
        entry barrier for the slowest replica, the reduce-scatter, the skip agreement, the
        update with its pushes, the closing barrier, clearing the bucket."""
        t = [int(v) for v in self.trace.cpu().tolist()]
        names = ("entry_wait", "reduce_scatter", "agree", "update_and_push", "exit_wait", "clear")
        return {n: round((t[i + 1] - t[i]) / 1e6, 3) for i, n in enumerate(names)
                if t[i + 1] and t[i]}

    def gather_master(self) -> None:
        """Makes every replica's fp32 master buffer complete (for checkpoints): between steps a
        rank holds current masters only for its own shard, plus the small fp32-read tail of each
        group that the step pushes everywhere."""
        p = self.params
        if p is None or not self.fused or not p.numel:
            return
        for r in range(self.size):
            lo, hi = self.bounds[r], self.bounds[r + 1]
            if hi > lo:
                dist.broadcast(p.master[lo:hi], self.state.dp_group_ranks[r], group=self.group)

    def gather_optimizer_state(self) -> Dict[str, torch.Tensor]:
        """Full-length moments assembled from every rank's shard (for checkpoints)."""
        n = self.params.numel
        out = {}
        for name, local in (("exp_avg", self.m), ("exp_avg_sq", self.v)):
            full = torch.zeros(n, dtype=torch.float32, device=self.device)
            lo, hi = self.shard
            full[lo:hi] = local[:hi - lo]
            dist.all_reduce(full, group=self.group)
            out[name] = full
        return out

    def load_optimizer_state(self, flats: Dict[str, torch.Tensor]) -> None:
        """Inverse of ``gather_optimizer_state``: keeps this rank's shard of full-length moments
        (resume from a checkpoint)."""
        lo, hi = self.shard
        for name, local in (("exp_avg", self.m), ("exp_avg_sq", self.v)):
            full = flats.get(name)
            if full is not None and hi > lo:
                local[:hi - lo].copy_(full[lo:hi].to(local.device))

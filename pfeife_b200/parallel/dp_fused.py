"""Fused data-parallel path: the gradient reduce-scatter, unscale, non-finite agreement,
partitioned AdamW and the all-gather of the updated weights run as one hand-written kernel per
rank that reads and writes the other ranks' buffers directly over NVLink (csrc/dp_fused.cu).

Host side: the flat gradient / master / shadow buffers of ``RankParams`` are ordinary device
allocations whose CUDA IPC handles are exchanged once over the control group; every rank maps
its peers' buffers and keeps a table of peer pointers.  Optimizer moments exist only for the
rank's own shard (ZeRO-1).  The kernel's cross-GPU barriers are epoch counters in a small
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
        if params.optimizer_type not in ("adam", "adamw") or not params.numel:
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
        params.dp_state = self      # checkpoints read / restore the sharded moments through us
        self.flags = torch.zeros(2 * DP_MAX, dtype=torch.int32, device=self.device)
        self.local_sync = torch.zeros(2, dtype=torch.int32, device=self.device)
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

    def reduce_and_step(self, params, scaler, fp16: bool) -> None:
        L = _lib.lib()
        params.step_count += 1
        lo_s, hi_s = self.shard
        for g, lo, hi in params.group_ranges:
            h = params.hyper[min(g, len(params.hyper) - 1)]
            a, b = max(lo, lo_s), min(hi, hi_s)
            if b < a:
                a = b = lo       # nothing of this group is owned here: only clear its gradients
            b1, b2 = h.get("betas", (0.9, 0.999))
            adamw = params.optimizer_type == "adamw"
            off = max(a - lo_s, 0)
            m = self.m[off:] if off < self.m.numel() else self.m
            v = self.v[off:] if off < self.v.numel() else self.v
            code = L.pf_dp_fused_step(
                self.rank, self.size, self.t_grad, self.t_master, self.t_lp, self.t_flags,
                ptr(m), ptr(v), ptr(self.local_sync), c_ll(a), c_ll(b),
                c_ll(self.deferred_below.get(g, 0)), c_ll(lo), c_ll(hi), c_f(h.get("lr", 1e-3)),
                c_f(b1), c_f(b2), c_f(h.get("eps", 1e-8)),
                c_f(h.get("weight_decay", 0.01 if adamw else 0.0)), int(params.step_count),
                c_f(1.0 / self.size), int(adamw),
                dt(params.lp.dtype) if params.lp is not None else 0, int(fp16),
                ptr(scaler.scale_tensor), ptr(params.found_inf), 3 * self.calls + 1, self.calls,
                ptr(kx.status_word(self.device)), sm_count(self.device), stream())
            check(code, "pf_dp_fused_step")
            self.calls += 1
        if fp16:
            scaler.update(params.found_inf)

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

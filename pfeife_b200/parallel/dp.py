"""Data parallelism over the flat gradient bucket of a pipeline rank.

Two implementations behind one interface (``make_dp``):
  * ``NcclDP``  - the measured baseline: one NCCL all-reduce of the fp32 bucket after the last
    micro-batch's backward, then the local fused optimizer kernel on the whole bucket (what
    DDP + GradScaler + torch.optim amount to in the reference, pfeife/mp/worker.py:1464-1494).
  * ``FusedDP`` - the product path (dp_fused.py): gradient reduce-scatter, unscale, partitioned
    AdamW and the all-gather of the updated weights in hand-written kernels that read and
    write peer memory over NVLink; optimizer moments exist only for the owned shard.
Parameters are broadcast from DP rank 0 when the reducer is attached, so replicas start equal
even if the user's script seeded them differently.
"""
from __future__ import annotations


import torch
import torch.distributed as dist


class NcclDP:
    fused = False

    def __init__(self, state, option):
        self.state = state
        self.group = state.dp_group
        self.size = state.dp_size
        self.src = state.dp_group_ranks[0]

    def attach(self, params) -> None:
        if params.numel:
            dist.broadcast(params.master, self.src, group=self.group)
            if params.lp is not None:
                params.lp.copy_(params.master)
        for s in params.slots.values():
            if s.offset < 0 and torch.is_tensor(s.view) and s.view.numel():
                dist.broadcast(s.view, self.src, group=self.group)

    def all_reduce(self, params) -> None:
        if params.numel:
            dist.all_reduce(params.grad, op=dist.ReduceOp.SUM, group=self.group)


def make_dp(state, option):
    if option.fused_dp and state.device.type == "cuda":
        try:
            from .dp_fused import FusedDP
        except ImportError:
            return NcclDP(state, option)
        return FusedDP(state, option)
    return NcclDP(state, option)

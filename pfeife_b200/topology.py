"""Process topology: signed PPxDP mesh arithmetic, the per-process state singleton and
``initialize_pfeife``.

Mesh semantics (pfeife/mp/net_states.py:11-107): ``dp_mesh = (a, b)`` is an ``|a| x |b|``
row-major matrix of global ranks and the NEGATIVE entry marks the data-parallel axis.
``"-2,4"``: rows are pipelines of 4 contiguous ranks, columns are DP groups; ``"2,-4"``: columns
are pipelines (stride-4 ranks), rows are DP groups.  A single entry (or None) means pure
pipeline parallelism over all ranks.  The main rank of a pipeline is its last PP rank.

Unlike the reference the backend is selectable: ``nccl`` + ``cuda:LOCAL_RANK`` when CUDA is
present, ``gloo`` + ``cpu`` otherwise (or when ``PFEIFE_CPU=1`` / ``cpu=True``), which is what
lets the whole runtime be tested without a GPU.  A second, gloo-backed group carries the control
plane (pickled objects, flags) so that nothing small ever goes through NCCL.
"""
from __future__ import annotations

import atexit
import datetime
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

MeshSpec = Optional[Union[str, Sequence[int]]]


# ------------------------------------------------------------------------- pure mesh arithmetic
def parse_dp_mesh(spec: MeshSpec) -> Optional[Tuple[int, ...]]:
    """"-2,4" -> (-2, 4); "8" -> (8,); None / "" -> None."""
    if spec is None:
        return None
    if isinstance(spec, str):
        spec = spec.strip()
        if not spec or spec.lower() == "none":
            return None
        vals = tuple(int(t) for t in spec.split(","))
    else:
        vals = tuple(int(t) for t in spec)
    if len(vals) == 0:
        return None
    if len(vals) > 2:
        raise ValueError(f"dp_mesh takes one or two integers, got {vals}")
    if len(vals) == 2 and (vals[0] < 0) == (vals[1] < 0):
        raise ValueError(f"exactly one entry of dp_mesh must be negative (the DP axis): {vals}")
    return vals


@dataclass(frozen=True)
class MeshLayout:
    """Resolved geometry of a mesh over ``world_size`` ranks."""
    world_size: int
    rows: int
    cols: int
    dp_axis: Optional[int]  # 0: rows index DP replicas, 1: cols do, None: no DP

    @staticmethod
    def build(world_size: int, spec: MeshSpec) -> "MeshLayout":
        mesh = parse_dp_mesh(spec)
        if mesh is None or len(mesh) == 1:
            n = world_size if mesh is None else abs(mesh[0])
            if n != world_size:
                raise ValueError(f"dp_mesh {mesh} does not cover world_size {world_size}")
            return MeshLayout(world_size, 1, world_size, None)
        a, b = mesh
        if abs(a) * abs(b) != world_size:
            raise ValueError(f"dp_mesh {mesh} does not cover world_size {world_size}")
        return MeshLayout(world_size, abs(a), abs(b), 0 if a < 0 else 1)

    @property
    def pp_size(self) -> int:
        if self.dp_axis is None:
            return self.world_size
        return self.cols if self.dp_axis == 0 else self.rows

    @property
    def dp_size(self) -> int:
        if self.dp_axis is None:
            return 1
        return self.rows if self.dp_axis == 0 else self.cols

    def coords(self, rank: int) -> Tuple[int, int]:
        return divmod(rank, self.cols)

    def pp_rank(self, rank: int) -> int:
        r, c = self.coords(rank)
        return rank if self.dp_axis is None else (c if self.dp_axis == 0 else r)

    def dp_rank(self, rank: int) -> int:
        r, c = self.coords(rank)
        return 0 if self.dp_axis is None else (r if self.dp_axis == 0 else c)

    def global_rank(self, pp_rank: int, dp_rank: int = 0) -> int:
        if self.dp_axis is None:
            return pp_rank
        if self.dp_axis == 0:
            return dp_rank * self.cols + pp_rank
        return pp_rank * self.cols + dp_rank

    def pp_group_ranks(self, rank: int) -> List[int]:
        d = self.dp_rank(rank)
        return [self.global_rank(p, d) for p in range(self.pp_size)]

    def dp_group_ranks(self, rank: int) -> List[int]:
        p = self.pp_rank(rank)
        return [self.global_rank(p, d) for d in range(self.dp_size)]

    def is_main_rank(self, rank: int) -> bool:
        return self.pp_rank(rank) == self.pp_size - 1

    def main_rank_of(self, rank: int) -> int:
        return self.pp_group_ranks(rank)[-1]

    def all_pp_groups(self) -> List[List[int]]:
        return [self.pp_group_ranks(self.global_rank(0, d)) for d in range(self.dp_size)]

    def all_dp_groups(self) -> List[List[int]]:
        return [self.dp_group_ranks(self.global_rank(p, 0)) for p in range(self.pp_size)]


# Free-function spellings of the reference API (pfeife/mp/net_states.py:18-107)
def check_main_rank(rank: int, world_size: int, dp_mesh: MeshSpec) -> bool:
    return MeshLayout.build(world_size, dp_mesh).is_main_rank(rank)


def target_main_rank(rank: int, world_size: int, dp_mesh: MeshSpec) -> int:
    return MeshLayout.build(world_size, dp_mesh).main_rank_of(rank)


def get_global_rank(pp_rank: int, dp_rank: int, world_size: int, dp_mesh: MeshSpec) -> int:
    return MeshLayout.build(world_size, dp_mesh).global_rank(pp_rank, dp_rank)


def get_pp_rank(rank: int, world_size: int, dp_mesh: MeshSpec) -> int:
    return MeshLayout.build(world_size, dp_mesh).pp_rank(rank)


def get_pp_group_ranks(rank: int, world_size: int, dp_mesh: MeshSpec) -> List[int]:
    return MeshLayout.build(world_size, dp_mesh).pp_group_ranks(rank)


def get_dp_group_ranks(rank: int, world_size: int, dp_mesh: MeshSpec) -> List[int]:
    return MeshLayout.build(world_size, dp_mesh).dp_group_ranks(rank)


# ------------------------------------------------------------------------- process state
class PfeifeState:
    """Per-process topology (fields of pfeife/mp/net_states.py:110-153)."""

    def __init__(self, dp_mesh: MeshSpec = None, cpu: Optional[bool] = None,
                 timeout_s: float = 1800.0):
        env = os.environ
        self.world_size = int(env.get("WORLD_SIZE", "1"))
        self.rank = int(env.get("RANK", "0"))
        self.local_rank = int(env.get("LOCAL_RANK", str(self.rank)))
        self.nnodes = int(env.get("NNODES", "1"))
        self.node_rank = int(env.get("NODE_RANK", "0"))
        if dp_mesh is None:
            dp_mesh = env.get("DP_MESH")
        self.dp_mesh = parse_dp_mesh(dp_mesh)
        self.layout = MeshLayout.build(self.world_size, self.dp_mesh)

        if cpu is None:
            cpu = env.get("PFEIFE_CPU", "0") == "1" or not torch.cuda.is_available()
        self.cpu = bool(cpu)
        if self.cpu:
            self.backend = "gloo"
            self.device = torch.device("cpu")
        else:
            self.backend = "nccl"
            self.device = torch.device("cuda", self.local_rank % max(1, torch.cuda.device_count()))
            torch.cuda.set_device(self.device)

        lay = self.layout
        self.is_main_rank = lay.is_main_rank(self.rank)
        self.is_main_process = self.rank == self.world_size - 1
        self.pp_rank = lay.pp_rank(self.rank)
        self.dp_rank = lay.dp_rank(self.rank)
        self.pp_size, self.dp_size = lay.pp_size, lay.dp_size
        self.pp_group_ranks = lay.pp_group_ranks(self.rank)
        self.dp_group_ranks = lay.dp_group_ranks(self.rank)
        self.pp_main_rank = self.pp_group_ranks[-1]

        self._owns_pg = False
        timeout = datetime.timedelta(seconds=timeout_s)
        if not dist.is_initialized():
            env.setdefault("MASTER_ADDR", "127.0.0.1")
            env.setdefault("MASTER_PORT", "24446")
            kwargs = {}
            if not self.cpu:
                kwargs["device_id"] = self.device
            dist.init_process_group(self.backend, rank=self.rank, world_size=self.world_size,
                                    timeout=timeout, **kwargs)
            self._owns_pg = True
            if self.cpu:
                # gloo's worker threads must be gone before the interpreter tears its modules
                # down, or a rank can abort in its last moments, after all its work was done
                atexit.register(self.destroy)

        # Data-plane groups.  Every rank must create every group, in the same order.
        self.pp_group = None
        self.dp_group = None
        for ranks in lay.all_pp_groups():
            g = dist.new_group(ranks, timeout=timeout) if len(ranks) < self.world_size or \
                lay.dp_size > 1 else dist.group.WORLD
            if self.rank in ranks:
                self.pp_group = g
        for ranks in lay.all_dp_groups():
            if lay.dp_size == 1:
                continue
            g = dist.new_group(ranks, timeout=timeout)
            if self.rank in ranks:
                self.dp_group = g
        # Control-plane groups (always gloo): objects, flags, small scalars.
        if self.cpu:
            self.ctrl_world, self.ctrl_pp, self.ctrl_dp = dist.group.WORLD, self.pp_group, self.dp_group
        else:
            self.ctrl_world = dist.new_group(list(range(self.world_size)), backend="gloo",
                                             timeout=timeout)
            self.ctrl_pp = self.ctrl_dp = None
            for ranks in lay.all_pp_groups():
                g = dist.new_group(ranks, backend="gloo", timeout=timeout)
                if self.rank in ranks:
                    self.ctrl_pp = g
            for ranks in lay.all_dp_groups():
                if lay.dp_size == 1:
                    continue
                g = dist.new_group(ranks, backend="gloo", timeout=timeout)
                if self.rank in ranks:
                    self.ctrl_dp = g
        self.device_mesh = None  # a torch DeviceMesh is not needed by this runtime

    def destroy(self) -> None:
        if self._owns_pg and dist.is_initialized():
            dist.destroy_process_group()
            self._owns_pg = False

    def __repr__(self) -> str:
        return (f"PfeifeState(rank={self.rank}/{self.world_size}, pp={self.pp_rank}/{self.pp_size}, "
                f"dp={self.dp_rank}/{self.dp_size}, main={self.is_main_rank}, "
                f"device={self.device}, backend={self.backend})")


_state: Optional[PfeifeState] = None


def initialize_pfeife(dp_mesh: MeshSpec = None, cpu: Optional[bool] = None,
                      timeout_s: float = 1800.0) -> PfeifeState:
    """Creates (once) the process-wide topology state from the launcher's environment
    (pfeife/mp/net_states.py:169-181)."""
    global _state
    if _state is None:
        _state = PfeifeState(dp_mesh, cpu, timeout_s)
    return _state


def get_state() -> PfeifeState:
    if _state is None:
        raise RuntimeError("call initialize_pfeife() first")
    return _state


def get_device() -> torch.device:
    return get_state().device


def reset_state() -> None:
    """Drops the singleton (tests and re-meshing after the planner picked a PPxDP shape)."""
    global _state
    if _state is not None:
        _state.destroy()
    _state = None

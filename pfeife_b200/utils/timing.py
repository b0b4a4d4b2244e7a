"""Per-stage forward/backward event recorders (pfeife/timing.py:7-56)."""
from __future__ import annotations

import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch


class CPUEvent:
    def __init__(self):
        self.t = time.perf_counter()

    def elapsed_time(self, end: "CPUEvent") -> float:
        return (end.t - self.t) * 1e3


class TimeRecorder:
    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.fw: Dict[int, List[Tuple[object, object]]] = defaultdict(list)
        self.bw: Dict[int, List[Tuple[object, object]]] = defaultdict(list)

    def append_fw(self, stage: int, start, end) -> None:
        self.fw[stage].append((start, end))

    def append_bw(self, stage: int, start, end) -> None:
        self.bw[stage].append((start, end))

    def get_event_logs(self):
        """-> ({stage: [ms...]} forward, {stage: [ms...]} backward); synchronises first."""
        self.sync()
        conv = lambda d: {k: [s.elapsed_time(e) for s, e in v] for k, v in d.items()}
        return conv(self.fw), conv(self.bw)

    def sync(self) -> None:
        pass

    def record_event(self, device, stream=None):
        raise NotImplementedError


class CPUTimeRecorder(TimeRecorder):
    def record_event(self, device=None, stream=None):
        return CPUEvent()


class CUDATimeRecorder(TimeRecorder):
    def record_event(self, device=None, stream=None):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream if stream is not None else torch.cuda.current_stream(device))
        return ev

    def sync(self) -> None:
        torch.cuda.synchronize()

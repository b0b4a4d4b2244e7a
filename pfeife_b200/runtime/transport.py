"""Point-to-point transports for stage-boundary tensors.

A *channel* is a DIRECTED rank pair.  Messages on a channel are FIFO in the order the sender
issues them; that order is static (it follows the sender's step program), so the receiver can
post its receives in the same order without any negotiation, and ahead of time.

``DistTransport`` uses ``torch.distributed`` point-to-point ops (NCCL on GPUs, gloo on CPU) with
one two-rank process group PER DIRECTED PAIR.  Each such group owns its communicator and its
stream, so a transfer queued in one direction can never block a transfer of the other
direction or of another pair; together with FIFO channels this makes the runtime deadlock-free
for any valid schedule without replaying a simulated global order.  Communicators are created
lazily by the backend on first use, so ``warm_up`` touches the channels of a plan in one global
order on every rank (the reference forces communicator creation with a ping-pong,
pfeife/mp/worker.py:222-240).

``LocalTransport`` serves the single-process runtime (one thread per device): the sender hands
over a tensor through a queue and the receiver copies it into its buffer on a side stream
(``Tensor.copy_`` across devices is a peer copy over NVLink), as pfeife/local/worker.py:566-646.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class Handle:
    """Completion handle; ``wait()`` makes the consumer (stream or host) wait for the data."""

    def wait(self) -> None:
        raise NotImplementedError


class _DoneHandle(Handle):
    def wait(self) -> None:
        return


class _WorkHandle(Handle):
    def __init__(self, work, keep=None):
        self.work = work
        self.keep = keep

    def wait(self) -> None:
        if self.work is not None:
            self.work.wait()
            self.work = None
            self.keep = None


class Transport:
    def isend(self, tensor: torch.Tensor, dst: int) -> Handle:
        raise NotImplementedError

    def irecv(self, buf: torch.Tensor, src: int) -> Handle:
        raise NotImplementedError

    def warm_up(self, channels: Sequence[Tuple[int, int]]) -> None:
        pass


class DistTransport(Transport):
    """`rank` and peers are GLOBAL ranks; `pipeline_ranks` lists the global ranks of every
    pipeline of the job (all replicas), because process groups must be created by all ranks of
    the job in the same order."""

    def __init__(self, rank: int, all_pipelines: Sequence[Sequence[int]], device: torch.device,
                 timeout=None):
        self.rank = rank
        self.device = device
        self.groups: Dict[Tuple[int, int], object] = {}
        for ranks in all_pipelines:
            for a in ranks:
                for b in ranks:
                    if a == b:
                        continue
                    kw = {"timeout": timeout} if timeout is not None else {}
                    g = dist.new_group([a, b], **kw)
                    if rank in (a, b):
                        self.groups[(a, b)] = g

    def isend(self, tensor: torch.Tensor, dst: int) -> Handle:
        work = dist.isend(tensor, dst, group=self.groups[(self.rank, dst)])
        return _WorkHandle(work, tensor)

    def irecv(self, buf: torch.Tensor, src: int) -> Handle:
        work = dist.irecv(buf, src, group=self.groups[(src, self.rank)])
        return _WorkHandle(work, buf)

    def warm_up(self, channels: Sequence[Tuple[int, int]]) -> None:
        """One tiny transfer per channel, channels visited in sorted order by every rank."""
        t = torch.zeros(1, device=self.device)
        for a, b in sorted(set(channels)):
            if self.rank == a:
                dist.send(t, b, group=self.groups[(a, b)])
            elif self.rank == b:
                dist.recv(t, a, group=self.groups[(a, b)])
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)


class _LocalHub:
    """Shared by the LocalTransports of one process: one queue per directed channel."""

    def __init__(self):
        self.queues: Dict[Tuple[int, int], "queue.Queue"] = {}
        self.lock = threading.Lock()
        # set when a device thread failed: receivers stop waiting for data that will never come
        self.aborted: Optional[BaseException] = None

    def get(self, src: int, dst: int, timeout: float):
        q = self.q(src, dst)
        deadline = time.monotonic() + timeout
        while True:
            if self.aborted is not None:
                raise RuntimeError(f"pipeline aborted: another stage failed ({self.aborted!r})")
            try:
                return q.get(timeout=min(0.2, max(0.0, deadline - time.monotonic())))
            except queue.Empty:
                if time.monotonic() >= deadline:
                    raise

    def q(self, src: int, dst: int) -> "queue.Queue":
        with self.lock:
            if (src, dst) not in self.queues:
                self.queues[(src, dst)] = queue.Queue()
            return self.queues[(src, dst)]


class _LocalRecv(Handle):
    def __init__(self, transport: "LocalTransport", buf: torch.Tensor, src: int):
        self.t, self.buf, self.src = transport, buf, src
        self.done = False

    def wait(self) -> None:
        if self.done:
            # completed while another handle of the channel was being waited for: the copy is
            # queued on the side stream, and the consumer's stream still has to wait for it
            self._join_stream()
            return
        t = self.t
        # receives on a channel complete in posting order
        pend = t.pending[self.src]
        while not self.done:
            head = pend[0]
            tensor, event = t.hub.get(head.src, t.rank, t.timeout)
            if head.buf.is_cuda:
                stream = t.copy_stream(head.src)
                if event is not None:
                    stream.wait_event(event)
                with torch.cuda.stream(stream):
                    head.buf.copy_(tensor, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(stream)
                head.event = ev
            else:
                head.buf.copy_(tensor)
                head.event = None
            head.done = True
            pend.pop(0)
        self._join_stream()

    def _join_stream(self) -> None:
        ev = getattr(self, "event", None)
        if ev is not None:
            torch.cuda.current_stream(self.buf.device).wait_event(ev)


class LocalTransport(Transport):
    def __init__(self, rank: int, hub: _LocalHub, device: torch.device, timeout: float = 600.0):
        self.rank, self.hub, self.device, self.timeout = rank, hub, device, timeout
        self.pending: Dict[int, List[_LocalRecv]] = {}
        self._streams: Dict[int, torch.cuda.Stream] = {}

    def copy_stream(self, src: int):
        if src not in self._streams:
            self._streams[src] = torch.cuda.Stream(self.device)
        return self._streams[src]

    def isend(self, tensor: torch.Tensor, dst: int) -> Handle:
        event = None
        if tensor.is_cuda:
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(tensor.device))
        self.hub.q(self.rank, dst).put((tensor, event))
        return _DoneHandle()

    def irecv(self, buf: torch.Tensor, src: int) -> Handle:
        h = _LocalRecv(self, buf, src)
        self.pending.setdefault(src, []).append(h)
        return h

"""Single-process runtime: one thread per device, activations and gradients moved with
device-to-device copies on side streams ("memcpy" mode; single node only).

Role of pfeife/local/manager.py, local/runner.py and local/worker.py.  The stage executor, the
planner, the partitioner and the front-end threads are the same objects as in the
process-per-GPU runtime; only the transport (``LocalTransport``: queue hand-off + peer copy),
the control plane (direct method calls) and the shared-parameter reducer (a thread barrier
instead of a process group / reducer sub-process) differ.  ``option.cpu_test`` runs every
"device" on the CPU with synchronous copies, which is the mode the unit tests use.
"""
from __future__ import annotations

import queue
import threading
from typing import Any, Dict, List, Tuple

import torch

from ..parallel.device_bench import DeviceBench
from .partial import SCALER_KEY, PartialRunner
from .transport import LocalTransport, _LocalHub
from .worker import LoopFlag, StageWorker


class _LocalState:
    """The fields of the process topology the front-end reads, for one in-process pipeline."""

    def __init__(self, devices: List[torch.device]):
        self.pp_size = len(devices)
        self.pp_rank = self.pp_size - 1
        self.dp_size, self.dp_rank = 1, 0
        self.world_size, self.rank = 1, 0
        self.device = devices[-1]
        self.cpu = self.device.type == "cpu"
        self.is_main_rank = self.is_main_process = True
        self.pp_group_ranks = list(range(self.pp_size))


class LocalReducer:
    """Sum of one tensor per participating thread (tied-parameter gradients)."""

    def __init__(self, n: int):
        self.n = n
        self.barrier = threading.Barrier(n)
        self.slots: Dict[int, torch.Tensor] = {}
        self.lock = threading.Lock()

    def all_reduce_sum(self, t: torch.Tensor) -> None:
        me = threading.get_ident()
        with self.lock:
            self.slots[me] = t
        self.barrier.wait()
        others = [v for k, v in self.slots.items() if k != me]
        total = t.clone()
        for o in others:
            total += o.to(t.device)
        self.barrier.wait()          # everyone has read the originals
        t.copy_(total)
        self.barrier.wait()
        with self.lock:
            self.slots.pop(me, None)


class PipelineStopped(RuntimeError):
    """Raised by a runner whose pipeline was torn down by an earlier failure."""


class _LocalControl:
    """Control plane of the in-process pipeline: plain calls into the worker threads."""

    def __init__(self, runner: "LocalRunner"):
        self.runner = runner

    def bcast(self, obj: Any = None) -> Any:
        if isinstance(obj, dict) and "flag" in obj:
            self.runner._dispatch(obj)
        return obj

    def scatter(self, objs: List[Any]) -> Any:
        if objs and isinstance(objs[0], dict) and objs[0].get("abort"):
            for q in self.runner._jobs:      # the first step failed: end the device threads
                q.put(None)
            return objs[-1]
        for w, payload in zip(self.runner.workers[:-1], objs[:-1]):
            self.runner._install(w, payload)
        return objs[-1]

    def gather(self, obj: Any) -> List[Any]:
        out = []
        for w in self.runner.workers[:-1]:
            out.append(({k: v.cpu() for k, v in w.params.named_tensors().items()},
                        {k: {kk: vv.cpu() for kk, vv in st.items()}
                         for k, st in w.params.optimizer_state().items()}))
        return out + [obj]

    def barrier(self) -> None:
        return

    def share_with_replicas(self, obj: Any = None) -> Any:
        return obj       # one pipeline, no replicas


class LocalRunner(PartialRunner):
    """``PartialRunner`` over devices of this process (``option.device_map``, or CPU threads
    with ``option.cpu_test``)."""

    def _setup_runtime(self) -> None:
        opt = self.option
        if opt.cpu_test or not torch.cuda.is_available():
            devices = [torch.device("cpu")] * opt.device_cnt
        else:
            devices = [torch.device(d) for d in opt.device_map[:opt.device_cnt]]
        self.devices = devices
        self.state = _LocalState(devices)
        self.hub = _LocalHub()
        self.workers: List[StageWorker] = []
        for r, dev in enumerate(devices):
            tr = LocalTransport(r, self.hub, dev, timeout=opt.ctrl_timeout) \
                if len(devices) > 1 else None
            self.workers.append(StageWorker(r, len(devices), dev, opt, tr,
                                            runner=self if r == len(devices) - 1 else None))
        self.worker = self.workers[-1]
        self.ctrl = _LocalControl(self)
        self.device_bench = DeviceBench(devices, opt)
        if len(devices) > 1:
            if self.state.cpu:
                self.device_bench.set_uniform(len(devices), (0.05, 1.0, 0.0))
            else:
                self.device_bench.run_bench(opt.device_bench, uniform=True)
        self._jobs = [queue.Queue() for _ in self.workers[:-1]]
        self._done = [queue.Queue() for _ in self.workers[:-1]]
        self._busy = [False] * len(self._jobs)
        self._wthreads = []
        for i, w in enumerate(self.workers[:-1]):
            t = threading.Thread(target=self._worker_loop, args=(i, w), daemon=True)
            t.start()
            self._wthreads.append(t)

    # plan installation: tied-parameter reducers are thread barriers
    def _install(self, worker: StageWorker, payload: Dict[str, Any]) -> None:
        worker.batch_cnt = payload["batch_cnt"]
        worker.set_partition_graph(payload["part"], payload["entries"], payload["optimizer_type"],
                                   payload["hyper"])
        worker.set_scheduler_steps(payload["steps"], payload["eval_steps"])
        if not hasattr(self, "_reducers"):
            self._reducers = {tuple(r): LocalReducer(len(r))
                              for r in payload["part"].shared_states.values()}
        worker.shared_groups = {k: v for k, v in self._reducers.items() if worker.pp_rank in k}

    def install_plan(self, payload: Dict[str, Any]) -> None:
        self._install(self.worker, payload)

    # per-step dispatch to the device threads
    def _wait_idle(self) -> None:
        for i in range(len(self._jobs)):
            if self._busy[i]:
                res = self._done[i].get(timeout=self.option.ctrl_timeout)
                self._busy[i] = False
                if isinstance(res, BaseException):
                    raise res

    def time_report(self, reset: bool = True) -> List[Dict[str, Any]]:
        self._wait_idle()
        reps = []
        for w in self.workers:
            rep = w.time_report(reset)
            rep["memory"] = w.memory_usage()
            reps.append(rep)
        return reps

    def _dispatch(self, msg: Dict[str, Any]) -> None:
        flag = msg["flag"]
        if flag == LoopFlag.STOP_LOOP:
            try:
                self._wait_idle()
            except BaseException:       # a failed step was reported when it happened
                pass
            for q in self._jobs:
                q.put(None)
            return
        if self.hub.aborted is not None:
            raise PipelineStopped("this pipeline stopped after a failed step; build a new "
                                  "runner") from self.hub.aborted
        self._wait_idle()
        if flag in (LoopFlag.CONTINUE_LOOP, LoopFlag.EVAL_LOOP):
            for i, q in enumerate(self._jobs):
                q.put(msg)
                self._busy[i] = True
        elif flag == LoopFlag.LOAD_PARAMS:
            for w in self.workers[:-1]:
                w.params.load_named(msg["named"])
                if msg.get("opt"):
                    w.params.load_optimizer_state(msg["opt"])
                    w.scaler.load_state_dict(msg["opt"].get(SCALER_KEY))
        elif flag == LoopFlag.LOG_MEMORY_USAGE:
            for w in self.workers[:-1]:
                w.log_memory_usage()

    def _worker_loop(self, idx: int, worker: StageWorker) -> None:
        if worker.device.type == "cuda":
            torch.cuda.set_device(worker.device)
        while True:
            msg = self._jobs[idx].get()
            if msg is None:
                return
            try:
                worker.reset_cache()
                worker.params.set_hyper(msg.get("hyper"))
                worker.run(training=(msg["flag"] == LoopFlag.CONTINUE_LOOP))
                self._done[idx].put(True)
            except BaseException as e:
                if self.hub.aborted is None:
                    self.hub.aborted = e       # stages waiting for this one's tensors give up
                self._done[idx].put(e)

    def _run(self, a_split, k_split, training: bool):
        try:
            out = super()._run(a_split, k_split, training)
            self._wait_idle()
        except PipelineStopped:
            raise
        except BaseException as e:
            # one stage failed: the others are waiting for tensors that will never arrive
            if self.hub.aborted is None:
                self.hub.aborted = e
            for i in range(len(self._jobs)):
                if self._busy[i]:
                    try:
                        self._done[i].get(timeout=self.option.ctrl_timeout)
                    except queue.Empty:
                        pass
                    self._busy[i] = False
            if self.hub.aborted is not e:
                raise self.hub.aborted      # the failure that started it, not its echo
            raise
        return out

    def record_times(self) -> Dict[int, Tuple[float, float]]:
        """stage -> (mean forward ms, mean backward ms) over the recorded steps."""
        stats: Dict[int, Tuple[float, float]] = {}
        for w in self.workers:
            fw, bw = w.recorder.get_event_logs()
            for s in fw:
                f = sum(fw[s]) / max(1, len(fw[s]))
                b = sum(bw.get(s, [0.0])) / max(1, len(bw.get(s, [0.0])))
                stats[s] = (f, b)
            w.recorder.reset()
        return stats

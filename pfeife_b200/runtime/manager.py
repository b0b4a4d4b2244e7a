"""Manager-style front-ends in which the framework owns the loss
(pfeife/mp/manager.py:21-203 and pfeife/local/manager.py:22-272):

    manager = PipeManager(model, loss_fn, option)        # or LocalPipeManager(...)
    losses = manager.run(target, *model_inputs)

``loss_fn(output, target, model)`` follows the ``LossWrapper`` call shape.  Each micro-batch
runs ``model`` and ``loss_fn`` and calls ``backward`` in its own front-end thread; the optimizer
is created from ``option.optimizer_type`` / ``optimizer_kwargs`` when none is given.
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional

import torch

from ..option import PipeOption
from .partial import PartialRunner, partial_compiler


def _leaves(v):
    if isinstance(v, dict):
        v = list(v.values())
    if isinstance(v, (list, tuple)):
        for e in v:
            yield from _leaves(e)
    elif hasattr(v, "values") and callable(v.values) and not torch.is_tensor(v):
        try:
            yield from _leaves(list(v.values()))      # HuggingFace output objects
        except Exception:
            return
    else:
        yield v


def _to_device(v, dev):
    if torch.is_tensor(v):
        return v if v.device == dev else v.to(dev, non_blocking=True)
    if isinstance(v, (list, tuple)):
        return type(v)(_to_device(e, dev) for e in v)
    if isinstance(v, dict):
        return {k: _to_device(e, dev) for k, e in v.items()}
    return v


class PipeManager:
    runner_cls = PartialRunner

    def __init__(self, model: torch.nn.Module, loss_fn: Callable, option: Optional[PipeOption] = None,
                 optimizer=None):
        self.option = option or PipeOption()
        self.module = model
        self.loss_fn = loss_fn
        self.optimizer = optimizer or self.option.make_optimizer(model.parameters())
        self.runner = self.runner_cls(self.option, self.optimizer)
        self.model = torch.compile(model, backend=partial_compiler)
        self.runner.set_exec_fn(self._exec)

    def _exec(self, target, *args, **kwargs):
        out = self.model(*args, **kwargs)
        # the first (profiling) call runs the whole model where its inputs are; the pipelined
        # calls deliver the output on the last stage's device, where the target already is
        dev = next((t.device for t in _leaves(out) if torch.is_tensor(t)), None)
        if dev is not None:
            target = _to_device(target, dev)
        loss = self.loss_fn(out, target, self.module)
        self.runner.scaler.scale(loss).backward()
        return loss.detach()

    def run(self, target, *args, **kwargs) -> List[Any]:
        """One optimizer step over ``batch_cnt`` micro-batches; returns the per-micro-batch
        losses."""
        return self.runner.step(target, *args, **kwargs)

    def eval(self, *args, **kwargs) -> List[Any]:
        self.runner.set_exec_fn(lambda *a, **k: self.model(*a, **k))
        try:
            return self.runner.eval_step(*args, **kwargs)
        finally:
            self.runner.set_exec_fn(self._exec)

    def gather_params(self, with_optimizer: bool = False):
        return self.runner.gather_params(with_optimizer)

    def clear_record(self) -> None:
        for w in getattr(self.runner, "workers", [self.runner.worker]):
            w.recorder.reset()

    def print_record(self) -> None:
        from ..utils import Recorder, get_logger
        log = get_logger()
        for w in getattr(self.runner, "workers", [self.runner.worker]):
            fw, bw = w.recorder.get_event_logs()
            for s in sorted(fw):
                rf, rb = Recorder(), Recorder()
                rf.update(fw[s])
                rb.update(bw.get(s, []))
                log.info("stage %d: forward %.3f ms (std %.3f), backward %.3f ms (std %.3f)", s,
                         rf.mean(), rf.stddev(), rb.mean(), rb.stddev())

    def close(self) -> None:
        self.runner.close()


class LocalPipeManager(PipeManager):
    """Single-process (thread-per-device) flavour."""

    @property
    def runner_cls(self):
        from .local import LocalRunner
        return LocalRunner

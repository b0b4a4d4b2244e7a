"""Logging, pytree helpers, running statistics and seeding (pfeife/utils.py:14-216)."""
from __future__ import annotations

import logging
import math
import random
import sys
from typing import Any, Callable, Iterable, List

import torch
from torch.utils._pytree import tree_flatten, tree_map, tree_unflatten

_LOGGER_NAME = "pfeife"


def get_logger() -> logging.Logger:
    """The framework logger, formatted ``(HH:MM:SS.mmm) message`` (pfeife/utils.py:14-22)."""
    logger = logging.getLogger(_LOGGER_NAME)
    if not logger.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter("(%(asctime)s.%(msecs)03d) %(message)s", "%H:%M:%S"))
        logger.addHandler(h)
        logger.setLevel(logging.INFO)
        logger.propagate = False
    return logger


def set_logger_level(level: int) -> None:
    get_logger().setLevel(level)


def fmem(nbytes: float) -> str:
    """Bytes -> 'x.xxMB' (1 MB = 1024^2 bytes)."""
    return f"{nbytes / (1024 ** 2):.2f}MB"


def to_device(value: Any, device) -> Any:
    """Moves every tensor of a pytree to `device`; other leaves pass through."""
    return tree_map(lambda v: v.to(device) if torch.is_tensor(v) else v, value)


def tree_trav(fn: Callable[[Any], None], pytree: Any) -> None:
    for leaf in tree_flatten(pytree)[0]:
        fn(leaf)


def tree_filter(fn: Callable[[Any], bool], pytree: Any) -> List[Any]:
    return [leaf for leaf in tree_flatten(pytree)[0] if fn(leaf)]


def tree_filter_tensor(pytree: Any) -> List[torch.Tensor]:
    return tree_filter(torch.is_tensor, pytree)


def fetch_attr(module: torch.nn.Module, target: str) -> Any:
    """``a.b.c`` attribute walk used for FX ``get_attr`` / ``call_module`` targets."""
    obj = module
    for i, atom in enumerate(target.split(".")):
        if not hasattr(obj, atom):
            raise AttributeError(f"no attribute {'.'.join(target.split('.')[: i + 1])!r}")
        obj = getattr(obj, atom)
    return obj


def module_set_attr(module: torch.nn.Module, target: str, attr: Any) -> None:
    *path, last = target.split(".")
    obj = module
    for atom in path:
        obj = getattr(obj, atom)
    setattr(obj, last, attr)


def list_params(attr: Any) -> List[torch.nn.Parameter]:
    if isinstance(attr, torch.nn.Module):
        return list(attr.parameters())
    if isinstance(attr, torch.nn.Parameter):
        return [attr]
    return []


def get_submodules(gm: torch.fx.GraphModule):
    return {n.target: fetch_attr(gm, n.target) for n in gm.graph.nodes if n.op == "call_module"}


def to_device_graphmodule(gm: torch.fx.GraphModule, device) -> torch.fx.GraphModule:
    """Moves a GraphModule and rewrites ``device=`` literals baked into its nodes."""
    gm.to(device)
    dev = torch.device(device)
    changed = False
    for node in gm.graph.nodes:
        if "device" in node.kwargs and isinstance(node.kwargs["device"], (torch.device, str)):
            kw = dict(node.kwargs)
            kw["device"] = dev
            node.kwargs = kw
            changed = True
        new_args = tuple(dev if isinstance(a, torch.device) else a for a in node.args)
        if new_args != node.args:
            node.args = new_args
            changed = True
    if changed:
        gm.recompile()
    return gm


class Recorder:
    """Streaming mean / standard deviation (Welford)."""

    def __init__(self):
        self.n = 0
        self._mean = 0.0
        self._m2 = 0.0

    def append(self, x: float) -> None:
        self.n += 1
        d = x - self._mean
        self._mean += d / self.n
        self._m2 += d * (x - self._mean)

    def update(self, xs: Iterable[float]) -> None:
        for x in xs:
            self.append(x)

    def mean(self) -> float:
        return self._mean

    def stddev(self) -> float:
        return math.sqrt(self._m2 / self.n) if self.n > 0 else 0.0


class MinMaxRecorder:
    def __init__(self):
        self.min = math.inf
        self.max = -math.inf

    def append(self, x: float) -> None:
        self.min = min(self.min, x)
        self.max = max(self.max, x)

    def update(self, xs: Iterable[float]) -> None:
        for x in xs:
            self.append(x)


def set_seed(seed: int = 42) -> None:
    """Seeds python, numpy and torch (all devices) and asks cuDNN for determinism."""
    random.seed(seed)
    try:
        import numpy as np
        np.random.seed(seed)
    except Exception:  # numpy is optional here
        pass
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False

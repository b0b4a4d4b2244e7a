"""Run options: one declarative table drives the keyword constructor, the argparse binding and
``from_args``.

Same flag names, option fields and defaults as the reference (pfeife/option.py:52-103 for the
fields, :105-165 for ``from_args``, :170-279 for the flags), plus the additions of this
framework (``dp_mesh``, ``fused_dp``, ``native_ops``, ``loss_scale`` ...).
"""
from __future__ import annotations

import argparse
import logging
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.optim as optim

default_optimizer = dict(type="adam", lr=1e-5)

_OPTIMIZERS = {
    "adam": optim.Adam, "adamw": optim.AdamW, "adagrad": optim.Adagrad, "adamax": optim.Adamax,
    "asgd": optim.ASGD, "rmsprop": optim.RMSprop, "rprop": optim.Rprop, "sgd": optim.SGD,
}


def get_optimizer_cls(optimizer_type: str):
    """Optimizer name -> class; unknown names fall back to SGD (pfeife/option.py:9-29)."""
    cls = _OPTIMIZERS.get(optimizer_type.lower())
    if cls is None:
        logging.getLogger("pfeife").warning("unknown optimizer %r, using SGD", optimizer_type)
        cls = optim.SGD
    return cls


_VERBOSITY = {"error": logging.ERROR, "warning": logging.WARNING, "info": logging.INFO,
              "debug": logging.DEBUG}
_PRECISION = {None: None, "no": None, "fp32": None, "fp16": torch.float16, "bf16": torch.bfloat16,
              torch.float16: torch.float16, torch.bfloat16: torch.bfloat16}


def _parse_device_map(text: Optional[str]) -> Optional[List[str]]:
    if not text:
        return None
    text = text.strip()
    if ":" in text:
        lo, hi = text.split(":")
        return [f"cuda:{i}" for i in range(int(lo), int(hi))]
    return [f"cuda:{int(t)}" for t in text.split(",")]


def _parse_int_list(text: Optional[str]) -> Optional[List[int]]:
    if not text:
        return None
    return [int(t.strip()) for t in text.strip().split(",") if t.strip()]


@dataclass(frozen=True)
class _Flag:
    field: str                      # PipeOption attribute
    default: Any
    flag: Optional[str] = None      # command-line flag (None: constructor-only)
    kw: Optional[Dict[str, Any]] = None   # argparse kwargs
    arg_default: Any = None         # default of the command-line flag when it differs
    convert: Optional[Callable[[Any], Any]] = None  # argparse value -> option value
    help: str = ""


_FLAGS: List[_Flag] = [
    _Flag("compiler", None, "--backend", dict(type=str), help="dynamo backend applied per stage"),
    _Flag("reducer_backend", "nccl", "--reducer_backend", dict(type=str, choices=["nccl", "gloo"]),
          arg_default="nccl", help="backend of the local runtime's tied-gradient reducers"),
    _Flag("device_cnt", 2, "--device_cnt", dict(type=int), arg_default=2,
          help="pipeline-parallel size"),
    _Flag("batch_size", 4, "--batch_size", dict(type=int), arg_default=2,
          help="micro-batch size"),
    _Flag("batch_cnt", None, "--batch_cnt", dict(type=int), arg_default=4,
          help="micro-batches per optimizer step (default: device_cnt)"),
    _Flag("loop_cnt", None, "--loop_cnt", dict(type=int), help="stages per rank (None: search)"),
    _Flag("loop_batch", None, "--loop_batch", dict(type=int),
          help="micro-batches per loop of a looped pipeline (None: search)"),
    _Flag("prefetch_fwd", None, "--prefetch_fwd", dict(type=int),
          help="extra warm-up forwards before 1F1B alternation (None: search)"),
    _Flag("split_points", None, "--split_points", dict(type=str), convert=_parse_int_list,
          help='manual split points "10,20"; disables the search'),
    _Flag("bench_seed", 0, "--bench_seed", dict(type=int), arg_default=0),
    _Flag("print_graph", False, "--print_graph", dict(action="store_true")),
    _Flag("device_map", None, "--device_map", dict(type=str), convert=_parse_device_map,
          help='"0:3" or "1,2,5"'),
    _Flag("device_bench", None, "--device_bench", dict(type=str),
          help="path of the link-model cache"),
    _Flag("graph_bench", None, "--graph_bench", dict(type=str),
          help="path of the per-segment latency/memory profile cache"),
    _Flag("scheduler", "single_comm", "--scheduler",
          dict(type=str, choices=["single_comm", "beam", "dfs", "bfs", "pipeless"]),
          arg_default="single_comm"),
    _Flag("partitioner", "beam_single", "--partitioner",
          dict(type=str, choices=["beam_single", "beam_2", "random_walk", "same_mem", "same_time"]),
          arg_default="beam_single"),
    _Flag("linearizer", "none", "--linearizer",
          dict(type=str, choices=["save_mem", "short_first", "long_first", "none"]),
          arg_default="none"),
    _Flag("use_fsdp", False, "--use_fsdp", dict(action="store_true")),
    _Flag("mixed_precision", None, "--mixed_precision", dict(type=str, choices=["fp16", "bf16"])),
    _Flag("cpu_test", False, "--cpu", dict(action="store_true"),
          help="run on CPU (gloo), for tests"),
    _Flag("no_side_effect", False, "--no_side_effect", dict(action="store_true"),
          help="manager front-ends: the framework owns the loss and hands back only losses; "
               "that is how PipeManager / LocalPipeManager always run here, so the flag "
               "selects nothing further"),
    _Flag("no_io_cache", False, "--no_io_cache", dict(action="store_true"),
          help="allocate stage-boundary receive buffers per step instead of keeping them"),
    _Flag("single_comm_thread", False, "--single_comm_thread", dict(action="store_true"),
          help="accepted for compatibility: this runtime posts transfers from the stage "
               "thread itself and has no sender threads to merge"),
    _Flag("no_bench_optimizer", False, "--no_bench_optimizer", dict(action="store_true")),
    _Flag("schedule_picture", None, "--schedule_picture", dict(type=str),
          help="write the planned schedule as an SVG chart (one lane per pipeline rank) to FILE"),
    # ---- additions of this framework
    _Flag("dp_mesh", None, "--dp_mesh_opt", dict(type=str),
          help='signed PPxDP mesh "-2,4", or "auto" to let the planner choose'),
    _Flag("fused_dp", True, "--no_fused_dp", dict(action="store_false"),
          help="use the NCCL-only data-parallel baseline instead of the fused P2P kernel"),
    _Flag("native_ops", True, "--no_native_ops", dict(action="store_false"),
          help="do not rewrite stage graphs onto the sm_100a kernels"),
    _Flag("init_loss_scale", 65536.0, "--init_loss_scale", dict(type=float), arg_default=65536.0),
    _Flag("ctrl_timeout", 1800.0, "--ctrl_timeout", dict(type=float), arg_default=1800.0,
          help="seconds before a control-plane wait gives up"),
    _Flag("cuda_graphs", False, "--cuda_graphs", dict(action="store_true"),
          help="capture per-(stage, micro-batch) forward/backward in CUDA graphs"),
]


class PipeOption:
    """Keyword-constructed option bag (pfeife/option.py:32-103).

    ``mixed_precision`` is stored as a torch dtype (or None), ``verbosity`` as a logging level,
    ``device_map`` defaults to ``cuda:0..device_cnt-1`` and ``batch_cnt`` to ``device_cnt``.
    """

    def __init__(self, **kwargs):
        known = {f.field for f in _FLAGS} | {"optimizer", "verbosity"}
        unknown = set(kwargs) - known
        if unknown:
            raise TypeError(f"unknown PipeOption field(s): {sorted(unknown)}")
        for f in _FLAGS:
            setattr(self, f.field, kwargs.get(f.field, f.default))
        if self.batch_cnt is None:
            self.batch_cnt = self.device_cnt
        if self.device_map is None:
            self.device_map = [f"cuda:{i}" for i in range(self.device_cnt)]
        if self.mixed_precision not in _PRECISION:
            raise ValueError(f"mixed_precision must be fp16 or bf16, got {self.mixed_precision!r}")
        self.mixed_precision = _PRECISION[self.mixed_precision]
        verbosity = kwargs.get("verbosity", "info")
        self.verbosity = _VERBOSITY.get(verbosity, logging.WARNING) \
            if isinstance(verbosity, str) else int(verbosity)
        opt = dict(kwargs.get("optimizer", default_optimizer))
        self.optimizer_type = opt.pop("type")
        self.optimizer_kwargs = opt

    # ------------------------------------------------------------------ argparse binding
    @staticmethod
    def add_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        for f in _FLAGS:
            if f.flag is None:
                continue
            kw = dict(f.kw or {})
            if kw.get("action") == "store_false":
                kw["dest"] = f.field
            elif kw.get("action") != "store_true":
                kw.setdefault("default", f.arg_default)
            if f.help:
                kw["help"] = f.help
            if f.field == "cpu_test":
                kw["dest"] = "cpu"
            if f.field == "compiler":
                kw["dest"] = "backend"
            if f.field == "dp_mesh":
                kw["dest"] = "dp_mesh_opt"
            parser.add_argument(f.flag, **kw)
        parser.add_argument("--optimizer_type", type=str, default="adam")
        parser.add_argument("--verbose", action="store_true")
        parser.add_argument("--old_ver", action="store_true",
                            help="no_side_effect + no_io_cache + single_comm_thread")
        return parser

    @staticmethod
    def from_args(args: argparse.Namespace) -> "PipeOption":
        """Namespace -> option.  Like the reference this pins the optimizer lr to 1e-3
        (pfeife/option.py:115) and applies the ``--old_ver`` / ``--cpu`` implications."""
        if getattr(args, "old_ver", False):
            args.no_side_effect = args.no_io_cache = args.single_comm_thread = True
        if getattr(args, "cpu", False):
            args.single_comm_thread = True
        kw: Dict[str, Any] = {}
        for f in _FLAGS:
            name = {"cpu_test": "cpu", "compiler": "backend", "dp_mesh": "dp_mesh_opt"}.get(
                f.field, f.field)
            if not hasattr(args, name):
                continue
            val = getattr(args, name)
            if f.convert is not None:
                val = f.convert(val)
            if val is None and f.field in ("device_map", "batch_cnt"):
                continue
            kw[f.field] = val
        kw["optimizer"] = {"type": getattr(args, "optimizer_type", "adam"), "lr": 1e-3}
        kw["verbosity"] = "debug" if getattr(args, "verbose", False) else "info"
        kw["bench_seed"] = 0
        option = PipeOption(**kw)
        option.set_logger()
        return option

    def set_logger(self) -> None:
        from .utils import set_logger_level
        set_logger_level(self.verbosity)

    # ------------------------------------------------------------------ helpers
    def make_optimizer(self, params):
        return get_optimizer_cls(self.optimizer_type)(params, **self.optimizer_kwargs)

    def to_dict(self) -> Dict[str, Any]:
        d = {f.field: getattr(self, f.field) for f in _FLAGS}
        d.update(verbosity=self.verbosity, optimizer_type=self.optimizer_type,
                 optimizer_kwargs=dict(self.optimizer_kwargs))
        return d

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in sorted(self.to_dict().items()))
        return f"PipeOption({inner})"

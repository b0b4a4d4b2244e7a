"""ctypes loader for the in-tree sm_100a kernel library.

The library is built by ``python -m pfeife_b200.csrc.build`` into the package directory.  On a
machine with a CUDA device a missing library is an error (there is no silent eager fallback on
GPU); on a CPU-only machine ``lib()`` returns ``None`` and the ops use their PyTorch reference
implementations, which is what the CPU/gloo tests run.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path
from typing import Optional

import torch

_PKG = Path(__file__).resolve().parent.parent
_KERNEL_LIB = _PKG / "libpfeife_b200_kernels.so"
_HOST_LIB = _PKG / "libpfeife_b200_host.so"

_lib: Optional[ctypes.CDLL] = None
_host: Optional[ctypes.CDLL] = None
_tried = False
_launches = 0  # kernels launched through this module (reported by bench.py)

PF_F32, PF_F16, PF_BF16 = 0, 1, 2
_tls = threading.local()
_DT = {torch.float32: PF_F32, torch.float16: PF_F16, torch.bfloat16: PF_BF16}


class KernelError(RuntimeError):
    pass


def dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}") from None


def lib() -> Optional[ctypes.CDLL]:
    """The kernel library, or None on a machine without CUDA."""
    global _lib, _tried
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        return None
    if _tried:
        raise KernelError(f"{_KERNEL_LIB} failed to load earlier")
    _tried = True
    if not _KERNEL_LIB.exists():
        raise KernelError(
            f"{_KERNEL_LIB.name} is missing on a CUDA machine; run "
            "`python -m pfeife_b200.csrc.build` (GPU paths never fall back to eager PyTorch)")
    # make sure libcudart from torch is already mapped so the library binds to the same runtime
    torch.cuda.init()
    _lib = ctypes.CDLL(str(_KERNEL_LIB), mode=ctypes.RTLD_GLOBAL)
    return _lib


def host_lib() -> Optional[ctypes.CDLL]:
    """Host-side C++ helpers (planner evaluator).  None when not built."""
    global _host
    if _host is None and _HOST_LIB.exists():
        _host = ctypes.CDLL(str(_HOST_LIB))
    return _host


def available() -> bool:
    return torch.cuda.is_available() and lib() is not None


def use_kernels(t: torch.Tensor) -> bool:
    """True when `t` lives on a CUDA device (then the native kernels must be used)."""
    return t.is_cuda


def ptr(t: Optional[torch.Tensor]):
    """Device pointer of `t` (NULL for None).  Also remembers, per thread, the device of the
    last tensor seen, which is the device ``stream()`` launches on: a thread's *current* torch
    device is not reliable (new Python threads start on device 0)."""
    if t is None:
        return ctypes.c_void_p(0)
    if t.is_cuda:
        _tls.op_device = t.device.index
    return ctypes.c_void_p(t.data_ptr())


def bind_thread(device_index: Optional[int] = None) -> None:
    """Makes sure the calling thread has the device's context bound inside the library's own
    CUDA runtime (threads created by PyTorch, such as autograd workers, arrive without one)."""
    idx = torch.cuda.current_device() if device_index is None else device_index
    if getattr(_tls, "dev", None) != idx:
        code = lib().pf_bind_device(int(idx))
        if code != 0:
            raise KernelError(f"pf_bind_device({idx}): CUDA error {code}")
        _tls.dev = idx


def stream(device: Optional[int] = None) -> ctypes.c_void_p:
    """Handle of the torch stream that is current for the device of the operands (the device
    of the last tensor passed through ``ptr`` in this thread); binds the calling thread of the
    library's own CUDA runtime to that device."""
    if device is None:
        device = getattr(_tls, "op_device", None)
    if device is None:
        device = torch.cuda.current_device()
    bind_thread(device)
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_sm_count_cache = {}


def sm_count(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx not in _sm_count_cache:
        _sm_count_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count_cache[idx]


def check(code: int, what: str) -> None:
    global _launches
    if code != 0:
        if code > 0:
            raise KernelError(f"{what}: CUDA error {code}")
        reasons = {-1: "unsupported dtype", -2: "misaligned pointer or pitch",
                   -3: "size beyond kernel limit", -100: "tensor-map encoder unavailable",
                   -101: "tensor-map encoding failed"}
        if code <= -1000:
            raise KernelError(f"{what}: tensor-map encoding failed (CUresult {-code - 1000})")
        raise KernelError(f"{what}: {reasons.get(code, code)}")
    _launches += 1


def launch_count() -> int:
    return _launches


def add_launches(n: int) -> None:
    """Accounts for kernels launched by replaying a captured CUDA graph."""
    global _launches
    _launches += n


def c_ll(v) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(v))


def c_f(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))

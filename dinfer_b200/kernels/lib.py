"""Loads the kernel libraries (ctypes) and turns their return codes into exceptions.

There is no fallback: if a library cannot be built or loaded the call raises.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch

from ..csrc import build as _build


class KernelError(RuntimeError):
    """A kernel library refused its arguments or CUDA reported an error."""


_LIBS: Dict[str, ctypes.CDLL] = {}

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dt]
    except KeyError:
        raise KernelError(f"dtype {dt} is not one the kernels take (float32, bfloat16)") from None


def library(name: str) -> ctypes.CDLL:
    lib = _LIBS.get(name)
    if lib is None:
        path = _build.ensure_built([name])[name]
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load kernel library {path}: {e}") from e
        lib.dinfer_last_error.restype = ctypes.c_char_p
        _LIBS[name] = lib
    return lib


def preload(names) -> None:
    """Build (in parallel) and load several libraries at once."""
    names = [n for n in names if n not in _LIBS]
    if names:
        _build.ensure_built(names)
        for n in names:
            library(n)


_SMS: Dict[int, int] = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of the device (the current one by default), asked once per device; the split
    heuristics size their grids by it.  148 (a whole B200) where no device can be asked."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or torch.cuda.current_device())
    n = _SMS.get(idx)
    if n is None:
        n = _SMS[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


_launches = 0


def launch_count() -> int:
    """Kernel launches so far: calls into the kernel libraries, library matrix products, and for a
    replayed CUDA graph the launches it captured."""
    return _launches


def add_launches(n: int = 1) -> None:
    global _launches
    _launches += n


def check(lib: ctypes.CDLL, code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        msg = lib.dinfer_last_error()
        raise KernelError(f"{what} failed (code {code}): {msg.decode('utf-8', 'replace') if msg else ''}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_handle() -> ctypes.c_void_p:
    """The current stream of the current device (the capture stream while a graph is being captured).
    Asked for at every launch, so through torch's raw accessor where this torch has it."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only (there is no CPU path)")

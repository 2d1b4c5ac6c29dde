"""Glue between torch tensors and the C entry points of the compiled kernel libraries."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_int, c_float, c_ll, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.dtype) -> int:
    try:
        return _CODES[t]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {t}") from None


def ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def stream() -> c_void_p:
    """The current CUDA stream of the current device as a raw handle.  Asked of torch on every launch (a capture
    or a ``torch.cuda.stream`` block changes it), through the cheapest call torch offers: a step of a small batch
    is bound by what the host spends per launch."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this op runs on the GPU only (tensor is on "
                              f"{t.device}); the engine has no CPU path")


def need_contiguous(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous (shape {tuple(t.shape)}, strides {t.stride()})")


def need_int32(name: str, t: torch.Tensor) -> None:
    if t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


_launches = 0


def launch_count() -> int:
    """How many kernel entry points of this package have been called (each launches one kernel)."""
    return _launches


class Library:
    """A lazily compiled and loaded kernel library; ``call`` raises on a non-zero return."""

    def __init__(self, name: str):
        self.name = name
        self._lib: Optional[ctypes.CDLL] = None
        self._fns = {}

    @property
    def lib(self) -> ctypes.CDLL:
        if self._lib is None:
            self._lib = build.load_library(self.name)
        return self._lib

    def call(self, fn_name: str, *args) -> None:
        global _launches
        _launches += 1
        fn = self._fns.get(fn_name)
        if fn is None:
            fn = self._fns[fn_name] = getattr(self.lib, fn_name)
        rc = fn(*args)
        if rc != 0:
            raise KernelError(f"{fn_name}: {build.last_error(self.name)}")

"""Tensor and context handles for driving the backend from Python.

Plays the role of diopi_test/python/conformance/diopi_runtime.py (Tensor, Context, Sizes,
Dtype) for the reference's conformance suite, but wraps memory that already exists: a
torch tensor (CUDA for real runs, CPU only for argument-validation tests that never reach
a kernel) is handed to the C ABI by pointer, shape and stride, without a copy.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int64

import torch

from . import _lib


class DiopiError(RuntimeError):
    """A non-zero return code of an op, with the backend's last error string."""

    def __init__(self, op: str, code: int, message: str):
        super().__init__(f"{op} returned {code}: {message}")
        self.op, self.code, self.message = op, code, message


class FunctionNotImplementedError(DiopiError):
    """Return code 13 (diopiNoImplement)."""


class Dtype:
    """Numeric values of diopiDtype_t (diopirt.h:60-79)."""

    int8, uint8, int16, uint16, int32, uint32, int64, uint64 = range(8)
    float16, float32, float64, bool, bfloat16 = 8, 9, 10, 11, 12


_TORCH_TO_DIOPI = {
    torch.int8: Dtype.int8, torch.uint8: Dtype.uint8, torch.int16: Dtype.int16, torch.int32: Dtype.int32,
    torch.int64: Dtype.int64, torch.float16: Dtype.float16, torch.float32: Dtype.float32,
    torch.float64: Dtype.float64, torch.bool: Dtype.bool, torch.bfloat16: Dtype.bfloat16,
}

SUCCESS, ERROR_OCCURRED, NO_IMPLEMENT, DTYPE_NOT_SUPPORTED = 0, 1, 13, 1000


def Sizes(values) -> _lib.diopiSize_t:
    """A by-value diopiSize_t; the backing array is kept alive on the returned object."""
    arr = (c_int64 * len(values))(*[int(v) for v in values])
    s = _lib.diopiSize_t(ctypes.cast(arr, ctypes.POINTER(c_int64)), len(values))
    s._keepalive = arr
    return s


class Tensor:
    """A diopiTensorHandle_t that borrows the memory of a torch tensor."""

    def __init__(self, t: torch.Tensor, *, as_device: bool | None = None):
        libs = _lib.load()
        if t.dtype not in _TORCH_TO_DIOPI:
            raise TypeError(f"dtype {t.dtype} has no DIOPI counterpart")
        self.torch = t  # keeps the memory alive
        nd = t.dim()
        shape = (c_int64 * max(nd, 1))(*t.shape)
        stride = (c_int64 * max(nd, 1))(*t.stride())
        device = 1 if (t.is_cuda if as_device is None else as_device) else 0
        self._rt = libs.rt
        self.handle = libs.rt.b200rt_tensor_create(
            ctypes.c_void_p(t.data_ptr()), nd, shape, stride, _TORCH_TO_DIOPI[t.dtype], device
        )

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            self._rt.b200rt_tensor_destroy(h)


class Context:
    """A diopiContextHandle_t bound to a CUDA stream (default: torch's current stream)."""

    def __init__(self, stream: torch.cuda.Stream | int | None = "current", lazy: bool = False):
        libs = _lib.load()
        self._rt = libs.rt
        if stream == "current":
            ptr = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0
        elif stream is None:
            ptr = 0
        elif isinstance(stream, int):
            ptr = stream
        else:
            ptr = stream.cuda_stream
        self.handle = libs.rt.b200rt_context_create(ctypes.c_void_p(ptr), 1 if lazy else 0)

    def set_stream(self, stream: torch.cuda.Stream) -> None:
        self._rt.b200rt_context_set_stream(self.handle, ctypes.c_void_p(stream.cuda_stream))

    def release(self) -> None:
        """Lets the context reuse the scratch it handed out; call between steps."""
        self._rt.b200rt_context_release(self.handle)

    def synchronize(self) -> None:
        rc = self._rt.b200rt_context_synchronize(self.handle)
        if rc != 0:
            raise RuntimeError(f"cudaStreamSynchronize failed with {rc}")

    def stats(self) -> dict:
        out = (c_int64 * 4)()
        self._rt.b200rt_context_stats(self.handle, out)
        return {"require_calls": out[0], "device_allocs": out[1], "blocks": out[2], "bytes": out[3]}

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h:
            try:   # the backend may hold a recorded call for this handle (opt-in pair fusion): let it go first
                _lib.load().impl.diopiB200ContextRelease(h)
            except Exception:  # noqa: BLE001
                pass
            self._rt.b200rt_context_destroy(h)


_default_ctx: dict[int, Context] = {}


def default_context() -> Context:
    """One context per CUDA device, on torch's current stream at the time of each call."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    ctx = _default_ctx.get(dev)
    if ctx is None:
        ctx = _default_ctx[dev] = Context()
    elif torch.cuda.is_available():
        ctx.set_stream(torch.cuda.current_stream())
    return ctx


def as_handle(x) -> ctypes.c_void_p | None:
    if x is None:
        return None
    if isinstance(x, Tensor):
        return x.handle
    raise TypeError(f"expected a diopi_b200 Tensor, got {type(x)}")


def check_returncode(op: str, rc: int) -> None:
    """Raises on a non-zero return code, as diopi_functions.check_returncode does."""
    if rc == SUCCESS:
        return
    msg = _lib.load().impl.diopiGetLastErrorString().decode(errors="replace")
    if rc == NO_IMPLEMENT:
        raise FunctionNotImplementedError(op, rc, msg)
    raise DiopiError(op, rc, msg)

"""Loads the two shared libraries and declares their C signatures for ctypes.

The consumer-side run time (libdiopi_rt.so) is loaded first with RTLD_GLOBAL so that
the backend (libdiopi_impl.so) resolves diopiGetTensorData, diopiGetStream, ... from
it, exactly as a DIOPI backend resolves them from the framework that loads it.
There is no fallback: a missing library is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_bool, c_char_p, c_double, c_int, c_int64, c_void_p
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"


class diopiSize_t(ctypes.Structure):
    """Mirror of the by-value {const int64_t* data; int64_t len} struct (diopirt.h:27-30)."""

    _fields_ = [("data", POINTER(c_int64)), ("len", c_int64)]


class _Libs:
    rt: ctypes.CDLL | None = None
    impl: ctypes.CDLL | None = None


_libs = _Libs()

OPS = {
    # name: argtypes after the context handle
    "diopiDestIndexCopyKV": [c_void_p, c_void_p, c_void_p],
    "diopiTokenAttentionInference": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "diopiTokenSoftmaxReduceVInference": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int],
    "diopiTokenDecodeAttentionInference": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "diopiTokenDecodeAttentionInferenceNoAlloc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "diopiContextAttentionInference": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "diopiApplyPenalty": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int],
    "diopiPagedAttention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, diopiSize_t, c_int64, c_int64, c_int64, c_void_p, c_int64],
    "diopiPromptFlashAttention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, diopiSize_t, c_int64, c_int64, c_int64, c_int64],
    "diopiRotaryEmbeddingV2": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64],
    "diopiApplyPenaltyV2": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "diopiRotaryEmbedding": [c_void_p, c_void_p, c_void_p, c_void_p, c_bool, c_bool],
    "diopiRMSNorm": [c_void_p, c_void_p, c_void_p, diopiSize_t, c_void_p, c_void_p, c_double],
    "diopiRotaryEmbeddingCopyKV": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_bool],
    "diopiMatmulAllReduce": [c_void_p, c_void_p, c_void_p, c_void_p, c_char_p, c_char_p, c_int64, c_int64],
    "diopiB200ContextRelease": [],
    "diopiRMSNormBackward": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, diopiSize_t, c_double],
}
INFO = ["diopiGetVendorName", "diopiGetImplVersion", "diopiGetLastErrorString"]
# set-up calls that take no context handle
GROUP = {
    "diopiB200GroupCreate": [c_char_p, c_int, c_int, c_int64, c_void_p],
    "diopiB200GroupConnect": [c_char_p, c_void_p],
    "diopiB200GroupDestroy": [c_char_p],
    "diopiB200GroupSetOption": [c_char_p, c_char_p, c_int64],
    "diopiB200SetOption": [c_char_p, c_int64],
}


def load() -> _Libs:
    """Loads both libraries once. Raises RuntimeError when they have not been built."""
    if _libs.impl is not None:
        return _libs
    rt_path = LIB_DIR / "libdiopi_rt.so"
    impl_path = LIB_DIR / "libdiopi_impl.so"
    for p in (rt_path, impl_path):
        if not p.exists():
            raise RuntimeError(
                f"{p} is missing: the CUDA libraries of diopi_b200 are not built "
                "(run `python -m diopi_b200.build`); there is no CPU fallback"
            )
    rt = ctypes.CDLL(str(rt_path), mode=ctypes.RTLD_GLOBAL)
    impl = ctypes.CDLL(str(impl_path), mode=os.RTLD_NOW)

    rt.b200rt_tensor_create.restype = c_void_p
    rt.b200rt_tensor_create.argtypes = [c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), c_int, c_int]
    rt.b200rt_tensor_destroy.restype = None
    rt.b200rt_tensor_destroy.argtypes = [c_void_p]
    rt.b200rt_context_create.restype = c_void_p
    rt.b200rt_context_create.argtypes = [c_void_p, c_int]
    rt.b200rt_context_set_stream.restype = None
    rt.b200rt_context_set_stream.argtypes = [c_void_p, c_void_p]
    rt.b200rt_context_release.restype = None
    rt.b200rt_context_release.argtypes = [c_void_p]
    rt.b200rt_context_synchronize.restype = c_int
    rt.b200rt_context_synchronize.argtypes = [c_void_p]
    rt.b200rt_context_destroy.restype = None
    rt.b200rt_context_destroy.argtypes = [c_void_p]
    rt.b200rt_context_stats.restype = None
    rt.b200rt_context_stats.argtypes = [c_void_p, POINTER(c_int64)]

    for name, args in OPS.items():
        fn = getattr(impl, name)
        fn.restype = c_int
        fn.argtypes = [c_void_p] + args
    for name, args in GROUP.items():
        fn = getattr(impl, name)
        fn.restype = c_int
        fn.argtypes = args
    for name in INFO:
        fn = getattr(impl, name)
        fn.restype = c_char_p
        fn.argtypes = []
    _libs.rt, _libs.impl = rt, impl
    return _libs

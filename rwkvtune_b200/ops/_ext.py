"""ctypes binding of ``librwkvtune_b200.so``.

The library exports plain C functions taking device pointers and a stream handle;
this module loads it once, checks return codes and offers small helpers for passing
``torch.Tensor`` storage.  Nothing here falls back to another implementation: if the
library is absent a CUDA call raises ``NativeLibraryMissing``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
DEBUG_BUILD = os.environ.get("RWKVTUNE_DEBUG_LIB", "0") == "1"      # load the bounds-recording build of the library
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc",
                         "librwkvtune_b200_debug.so" if DEBUG_BUILD else "librwkvtune_b200.so")


class NativeLibraryMissing(RuntimeError):
    pass


class NativeCallError(RuntimeError):
    pass


_STATUS = {1: "bad shape", 2: "bad alignment", 3: "size beyond the supported maximum", 4: "not initialised",
           5: "device-side wait timed out"}


def lib_path() -> str:
    return _LIB_PATH


_AVAILABLE = None


def available() -> bool:
    """True when the native library has been built (checked once: this sits on the dispatch path of every GEMM)."""
    global _AVAILABLE
    if _AVAILABLE is None or not _AVAILABLE:
        _AVAILABLE = os.path.exists(_LIB_PATH)
    return _AVAILABLE


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(_LIB_PATH):
            raise NativeLibraryMissing(
                f"{_LIB_PATH} not found: build it with `python -m rwkvtune_b200.csrc.build` "
                "(CUDA tensors never fall back to a PyTorch implementation)")
        _LIB = ctypes.CDLL(_LIB_PATH)
    return _LIB


def check(status: int, what: str) -> None:
    if status == 0:
        return
    if status >= 1000:
        code = status - 1000
        try:
            msg = torch.cuda.cudart().cudaGetErrorString(code)  # type: ignore[attr-defined]
        except Exception:
            msg = f"cudaError {code}"
        raise NativeCallError(f"{what}: CUDA error {code} ({msg})")
    raise NativeCallError(f"{what}: {_STATUS.get(status, f'status {status}')}")


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    """Raw handle of the current CUDA stream (the C accessor: the Stream-object route costs ~20 us per call)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is None:
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return ctypes.c_void_p(raw(torch.cuda.current_device()))


LAUNCH_COUNT = 0   # native entry-point calls since import (each issues at least one kernel)


_FUNCS = {}


def call(name: str, *args) -> None:
    global LAUNCH_COUNT
    fn = _FUNCS.get(name)
    if fn is None:
        fn = getattr(lib(), name)
        fn.restype = ctypes.c_int
        _FUNCS[name] = fn
    LAUNCH_COUNT += 1
    status = fn(*args)
    if status:
        check(status, name)


def launch_count() -> int:
    return LAUNCH_COUNT


import contextlib as _contextlib
import os as _os


# ------------------------------------------------------------------------------- graph capture hygiene
@_contextlib.contextmanager
def capture_safe_gc():
    """Wrap a CUDA-graph capture.  Collects cyclic garbage first and keeps the collector off while capturing: an old
    ``CUDAGraph`` (or anything else whose finaliser frees device memory) that the cycle collector happens to reclaim in
    the middle of a capture makes a CUDA call that is illegal there and invalidates the capture - at a point that
    depends on allocation counts, i.e. not reproducibly."""
    import gc

    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()


# ------------------------------------------------------------------------------- chained launches

_CHAINING = False
CHAINING_ALLOWED = _os.environ.get("RWKVTUNE_CHAINED_LAUNCH", "1") == "1"


def chaining() -> bool:
    return _CHAINING


@_contextlib.contextmanager
def launch_chaining():
    """Inside this context the kernels of the decode path are launched as a programmatic dependent chain: each may be
    scheduled while its predecessor still runs and waits on the device for it before touching activations (see
    ``csrc/common.cuh``).  The decode GEMM additionally streams its first weight tiles before that wait, so the
    context must not enclose anything that writes model weights.  ``RWKVTUNE_CHAINED_LAUNCH=0`` turns it off."""
    global _CHAINING
    if not (CHAINING_ALLOWED and available() and hasattr(lib(), "rwkv_set_launch_chaining")) or _CHAINING:
        yield
        return
    lib().rwkv_set_launch_chaining(ctypes.c_int(1))
    _CHAINING = True
    try:
        yield
    finally:
        lib().rwkv_set_launch_chaining(ctypes.c_int(0))
        _CHAINING = False


def i32(v: int) -> ctypes.c_int:
    return ctypes.c_int(int(v))


def i64(v: int) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(v))


def f32(v: float) -> ctypes.c_float:
    return ctypes.c_float(float(v))


DEBUG_EVENT_SOURCES = ("gather", "loss_rows")


def debug_events(reset: bool = False):
    """Bounds violations recorded by the debug build since the last reset: ``{source file: (count, kernel tag, index,
    limit)}`` for every source that saw one.  Empty in the release build."""
    out = {}
    if not DEBUG_BUILD:
        return out
    torch.cuda.synchronize()
    for tag in DEBUG_EVENT_SOURCES:
        fn = getattr(lib(), f"rwkv_debug_read_{tag}", None)
        if fn is None:
            continue
        buf = (ctypes.c_longlong * 4)()
        fn.restype = ctypes.c_int
        check(fn(buf, ctypes.c_int(1 if reset else 0)), f"rwkv_debug_read_{tag}")
        if buf[0]:
            out[tag] = tuple(int(v) for v in buf)
    return out

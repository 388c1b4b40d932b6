"""ctypes binding to the in-tree native library ``lib/libb200dist.so``.

All native entry points are plain ``extern "C"`` functions that take raw device pointers and a
CUDA stream handle and return 0 or an error code (message via ``b200_last_error``). This keeps the
native build free of the torch headers (seconds instead of minutes per file) and lets callers that
are not Python use the same symbols.

Role in the reference: the pybind modules ``libtriton_distributed`` (``csrc/lib/op_pybind.cc:34-45``)
and ``triton._C.libtriton.distributed`` (``python/src/triton_distributed.cc``).
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_DEBUG = os.environ.get("B200DIST_DEBUG_LIB", "0") == "1"   # the checking build (python -m ...build --debug)
LIB_PATH = _PKG / "lib" / ("libb200dist_debug.so" if _DEBUG else "libb200dist.so")

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class NativeError(RuntimeError):
    """A native entry point returned a non-zero code."""

    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} failed (code {code}): {msg}")
        self.code = code


def lib_available() -> bool:
    return LIB_PATH.exists()


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load (building first when the shared object is absent) and return the native library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            if not build_if_missing or os.environ.get("B200DIST_NO_BUILD") == "1":
                raise RuntimeError(
                    f"native library {LIB_PATH} is missing; run `python -m triton_distributed_b200.build`")
            from . import build as _build
            _build.build(debug=_DEBUG)
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.b200_last_error.restype = ctypes.c_char_p
        for name in ("b200_heap_base", "b200_heap_mc_base", "b200_heap_bytes", "b200_heap_live_bytes"):
            getattr(lib, name).restype = ctypes.c_uint64
        _lib = lib
        return lib


def check(fn_name: str, code: int) -> None:
    if code != 0:
        msg = load().b200_last_error()
        raise NativeError(fn_name, code, msg.decode() if msg else "")


_NVTX = os.environ.get("B200DIST_NVTX", "0") == "1"


def call(fn_name: str, *args) -> None:
    """Call a native function that returns an int status and raise on failure. With ``B200DIST_NVTX=1`` every
    launcher call is wrapped in an NVTX range named after the entry point, so the fused kernels show up by name in a
    timeline next to the library kernels around them."""
    fn = getattr(load(), fn_name)
    if _NVTX:
        torch.cuda.nvtx.range_push(fn_name)
        try:
            check(fn_name, fn(*args))
        finally:
            torch.cuda.nvtx.range_pop()
        return
    check(fn_name, fn(*args))


# ---- argument helpers ------------------------------------------------------------------------
_DTYPE_CODE = {
    torch.bfloat16: 0,
    torch.float16: 1,
    torch.float32: 2,
    torch.float8_e4m3fn: 3,
    torch.uint8: 4,
    torch.int32: 5,
}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"dtype {dt} is not supported by the native kernels") from None


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(stream: torch.cuda.Stream | None = None) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def require_cuda() -> None:
    """Ops call this first: on a GPU machine the native path is the only path."""
    if not torch.cuda.is_available():
        raise RuntimeError("this op needs a CUDA device (sm_100a); use triton_distributed_b200.ref on CPU")


c_int = ctypes.c_int
c_u64 = ctypes.c_uint64
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p

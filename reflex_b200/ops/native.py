"""The native kernel library, loaded once through its C ABI.

There is no fallback: if the library cannot be built or loaded, or a kernel
returns a non-zero status, a `CudaError` is raised.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional

from ..errors import CudaError

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_longlong = ctypes.c_longlong

_SIGNATURES = {
    "rfx_embed": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p],
    "rfx_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                    c_void_p, c_int, c_int, c_void_p],
    "rfx_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "rfx_gather_dot": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "rfx_gemm_bf16_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_int, c_int, c_float, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_residual": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemm_bf16_tc_qkv": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                             c_float, c_float, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "rfx_gemv_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "rfx_qkv_post": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int,
                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "rfx_attention_plain": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "rfx_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong,
                             c_void_p, c_void_p],
    "rfx_attention_decode_cluster": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong,
                                     c_void_p, c_void_p],
    "rfx_attention_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_void_p],
    "rfx_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_float, c_void_p, c_void_p],
    "rfx_wait_probe": [c_longlong, c_void_p, c_void_p],
    "rfx_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "rfx_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p],
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc import build

        try:
            path = build.ensure_built()
            handle = ctypes.CDLL(path)
        except (RuntimeError, OSError) as e:
            raise CudaError(f"the native kernel library is not available: {e}") from e
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise CudaError(f"native library {path} lacks symbol {name}") from e
            fn.argtypes = argtypes
            fn.restype = c_int
        handle.rfx_gemm_bf16_tc_max_parts.argtypes = [c_int]
        handle.rfx_gemm_bf16_tc_max_parts.restype = c_int
        handle.rfx_sm_count.argtypes = []
        handle.rfx_sm_count.restype = c_int
        handle.rfx_sample_work_bytes.argtypes = [c_int, c_int]
        handle.rfx_sample_work_bytes.restype = c_longlong
        handle.rfx_error_string.argtypes = [c_int]
        handle.rfx_error_string.restype = ctypes.c_char_p
        _lib = handle
        return _lib


def register_signature(name: str, argtypes) -> None:
    """Declare one more exported function (used by kernels added later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


LAUNCHES = 0  # kernels of this library launched (or captured into a graph) so far


ERR_UNSUPPORTED = -2  # a kernel's answer for sizes it does not take


def check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status != 0:
        msg = lib().rfx_error_string(status).decode("utf-8", "replace")
        raise CudaError(f"{what} failed: {msg} (status {status})")

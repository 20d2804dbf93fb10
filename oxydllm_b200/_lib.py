"""ctypes binding of ``liboxq.so`` (the C ABI declared in ``include/oxq.h``).

The library is mandatory: there is no CPU or PyTorch fallback. If it is
missing it is built in-tree with nvcc; if that fails, importing raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

OXQ_F32, OXQ_F16, OXQ_BF16 = 0, 1, 2

_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

#: name -> argtypes; every entry returns an int status unless listed in _RESTYPE.
SIGNATURES = {
    "oxq_status_string": [_i],
    "oxq_last_error": [],
    "oxq_version": [],
    "oxq_awq_dequant": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "oxq_awq_gemv": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "oxq_decode_max_m": [],
    "oxq_decode_workspace_bytes": [_i, _i, _i],
    "oxq_awq_decode_matmul": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_awq_ffn_gate_up": [_vp, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _vp, ctypes.c_size_t, _vp],
    "oxq_gptq_gemv": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "oxq_w8a16_gemv": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "oxq_w8a16_dequant": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "oxq_w8a16_gemm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_gptq_dequant": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "oxq_gguf_dequant": [_i, _vp, _vp, _i, _i, _i, _vp],
    "oxq_gguf_gemv": [_i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "oxq_fp8_dequant": [_vp, _vp, _i, _i, _vp, _i, _i, _i, _vp],
    "oxq_fp8_gemv": [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "oxq_mxfp4_dequant": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "oxq_mxfp4_gemv": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp],
    "oxq_gemm_workspace_bytes": [_i, _i],
    "oxq_gemm_check": [_vp, _vp],
    "oxq_selftest_wait_expiry": [_vp, ctypes.c_int, _vp],
    "oxq_selftest_gemm_wait_expiry": [_vp, ctypes.c_size_t, ctypes.c_int, _vp],
    "oxq_selftest_moe_wait_expiry": [_vp, ctypes.c_size_t, _vp],
    "oxq_awq_gemv_check": [_vp],
    "oxq_gemm_workspace_init": [_vp, _vp],
    "oxq_awq_gemm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_awq_gemm_tp": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_gptq_gemm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_gguf_gemm": [_i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_fp8_gemm": [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_mxfp4_gemm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _sz, _vp],
    "oxq_gptoss_moe_workspace_bytes": [_i, _i, _i, _i, _i],
    "oxq_gptoss_moe_forward": [_vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, ctypes.c_float,
                               _i, _i, _vp, _i, _vp, _sz, _vp],
    "oxq_gptoss_experts_forward": [_vp, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, ctypes.c_float, _i, _i,
                                   _vp, _i, _vp, _sz, _vp],
    "oxq_moe_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i, _vp],
    "oxq_moe_dispatch_plan": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "oxq_moe_gather_rows": [_vp, _vp, _i, _i, _i, _vp, _vp],
    "oxq_moe_expand_ids": [_vp, _i, _i, _i, _vp, _vp],
    "oxq_moe_route": [_vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "oxq_awq_gemm_noalloc_max_k": [],
    "oxq_awq_gemm_noalloc": [_vp, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "oxq_awq_gemm_noalloc_check": [_vp],
}
_RESTYPE = {"oxq_status_string": ctypes.c_char_p, "oxq_last_error": ctypes.c_char_p,
            "oxq_gemm_workspace_bytes": ctypes.c_size_t, "oxq_decode_workspace_bytes": ctypes.c_size_t, "oxq_gptoss_moe_workspace_bytes": ctypes.c_size_t, "oxq_awq_gemm_noalloc_max_k": ctypes.c_size_t}

_lib = None


class OxqError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, message: str):
        super().__init__(f"{fn}: {message} (status {status})")
        self.status = status
        self.message = message


def lib_path() -> str:
    return _build.LIB


def load() -> ctypes.CDLL:
    """Load (building if needed) the shared library and declare its prototypes."""
    global _lib
    if _lib is None:
        path = _build.build()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing and could not be built; the CUDA library is required")
        lib = ctypes.CDLL(path)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPE.get(name, _i)
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Call an entry point; raise :class:`OxqError` with the library's message on failure."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.oxq_last_error().decode() or lib.oxq_status_string(rc).decode()
        raise OxqError(name, rc, msg)

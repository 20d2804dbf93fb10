"""Prefill-sized (m > 32) matmuls of the quantized linears.

Until a format has a tensor-core GEMM entry point, batches are cut into
decode-sized row chunks and run on the GEMV kernels, the same strategy as the
reference's ``chunked_batch_gemv`` (linear.rs:458-480).
"""
from __future__ import annotations

from .linear import GEMV_MAX_M


def _chunks(m: int):
    for r in range(0, m, GEMV_MAX_M):
        yield r, min(GEMV_MAX_M, m - r)


def awq_matmul(lin, x2, y):
    for r, rows in _chunks(x2.shape[0]):
        lin._gemv(x2[r:r + rows], y[r:r + rows], rows)


def _via_forward(lin, x2, y):
    for r, rows in _chunks(x2.shape[0]):
        y[r:r + rows] = lin.forward(x2[r:r + rows])


def fp8_matmul(lin, s, s_out, s_in, x2, y):
    _via_forward(lin, x2, y)


def gguf_matmul(lin, x2, y):
    _via_forward(lin, x2, y)


def mxfp4_matmul(lin, x2, y):
    _via_forward(lin, x2, y)

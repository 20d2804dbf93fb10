"""Prefill-sized (m > 32) matmuls of the quantized linears on the tensor cores.

Thin callers of the ``oxq_*_gemm`` entry points. The dequantization slab
workspace is caller-owned device memory: one cached ``torch`` buffer per
device and size, shared by stream-ordered calls.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_workspaces: dict = {}


def workspace_bytes(n: int, k: int) -> int:
    return int(_lib.load().oxq_gemm_workspace_bytes(n, k))


def workspace(n: int, k: int, device) -> torch.Tensor:
    """A device buffer large enough for ``oxq_*_gemm`` on an ``[n, k]`` weight (grown on demand, reused)."""
    need = workspace_bytes(n, k)
    key = _dev_index(device)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(need, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


_decode_ws: dict = {}


def _dev_index(device) -> int:
    idx = torch.device(device).index
    return torch.cuda.current_device() if idx is None else idx


def decode_workspace(m: int, k: int, n: int, device) -> torch.Tensor:
    """Workspace of ``oxq_awq_decode_matmul`` for this device (grown on demand, zero-filled, reused)."""
    need = int(_lib.load().oxq_decode_workspace_bytes(m, k, n))
    key = _dev_index(device)
    buf = _decode_ws.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(need, dtype=torch.uint8, device=torch.device("cuda", key))
        _decode_ws[key] = buf
    return buf


def awq_decode_matmul(lin, x2, y):
    """``y = x2 . deq(W)`` for decode-sized batches on the tensor cores (``oxq_awq_decode_matmul``)."""
    from .linear import _dt
    ws = decode_workspace(x2.shape[0], lin.in_features, lin.out_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_awq_decode_matmul", _p(x2), _dt(x2.dtype), _p(lin.qweight), _p(lin.qzeros), _p(lin.scales),
              _dt(lin.scales.dtype), bp, bd, _p(y), _dt(y.dtype), x2.shape[0], lin.in_features, lin.out_features,
              lin.group_size, _p(ws), ws.numel(), _st())


def check(ws: torch.Tensor) -> None:
    """Synchronise and raise if a tensor-core kernel recorded a timed-out wait in ``ws``."""
    _lib.call("oxq_gemm_check", ctypes.c_void_p(ws.data_ptr()),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bias(b):
    from .linear import _dt
    return _p(b), (_dt(b.dtype) if b is not None else 0)


def awq_matmul(lin, x2, y):
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_awq_gemm", _p(x2), _dt(x2.dtype), _p(lin.qweight), _p(lin.qzeros), _p(lin.scales),
              _dt(lin.scales.dtype), bp, bd, _p(y), _dt(y.dtype), x2.shape[0], lin.in_features, lin.out_features,
              lin.group_size, _p(ws), ws.numel(), _st())


def w8a16_matmul(lin, x2, y):
    """``y = x2 . deq(W)^T (+ bias)`` for the 8-bit AWQ layout (``oxq_w8a16_gemm``)."""
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_w8a16_gemm", _p(x2), _dt(x2.dtype), _p(lin.qweight), _p(lin.qzeros), _p(lin.scales),
              _dt(lin.scales.dtype), bp, bd, _p(y), _dt(y.dtype), x2.shape[0], lin.in_features, lin.out_features,
              lin.group_size, _p(ws), ws.numel(), _st())


def gptq_matmul(raw, x2, y, bias=None):
    """``y = x2 . deq(W)^T (+ bias)`` for a GPTQ-packed ``QuantWeight`` or ``PackedQuantLinear`` (4 or 8 bit,
    ``oxq_gptq_gemm``)."""
    from .linear import _as_u32_words, _dt
    feat = lambda v: v() if callable(v) else v
    k, n, g = feat(raw.in_features), feat(raw.out_features), feat(raw.group_size)
    ws = workspace(n, k, x2.device)
    qw, sc = _as_u32_words(raw.qweight), raw.scales.contiguous()
    qz = None if raw.qzeros is None else _as_u32_words(raw.qzeros)
    sym = raw.qzeros is None or raw.zero_point == "symmetric"
    bp, bd = _bias(bias)
    _lib.call("oxq_gptq_gemm", _p(x2), _dt(x2.dtype), _p(qw), _p(qz), _p(sc), _dt(sc.dtype), bp, bd, _p(y), _dt(y.dtype),
              x2.shape[0], k, n, g, raw.bits, int(sym), _p(ws), ws.numel(), _st())


def awq_ffn_gate_up(lin, x2, y, activation: int):
    """``y[m, inter] = act(x . W_gate^T) * (x . W_up^T)`` on the fused ``[gate | up]`` AWQ linear ``lin``."""
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    _lib.call("oxq_awq_ffn_gate_up", _p(x2), _dt(x2.dtype), _p(lin.qweight), _p(lin.qzeros), _p(lin.scales),
              _dt(lin.scales.dtype), activation, _p(y), x2.shape[0], lin.in_features, lin.out_features // 2,
              lin.group_size, _p(ws), ws.numel(), _st())


def fp8_matmul(lin, s, s_out, s_in, x2, y):
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_fp8_gemm", _p(x2), _dt(x2.dtype), _p(lin.weight), _p(s), s_out, s_in, bp, bd, _p(y), _dt(y.dtype),
              x2.shape[0], lin.in_features, lin.out_features, _p(ws), ws.numel(), _st())


def gguf_matmul(lin, x2, y):
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_gguf_gemm", lin.ggml_type, _p(x2), _dt(x2.dtype), _p(lin.blocks), bp, bd, _p(y), _dt(y.dtype),
              x2.shape[0], lin.in_features, lin.out_features, _p(ws), ws.numel(), _st())


def mxfp4_matmul(lin, x2, y):
    from .linear import _dt
    ws = workspace(lin.out_features, lin.in_features, x2.device)
    bp, bd = _bias(lin.bias)
    _lib.call("oxq_mxfp4_gemm", _p(x2), _dt(x2.dtype), _p(lin.blocks), _p(lin.scales), bp, bd, _p(y), _dt(y.dtype),
              x2.shape[0], lin.in_features, lin.out_features, _p(ws), ws.numel(), _st())

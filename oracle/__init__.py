"""numpy front end of the CPU oracle (``oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of ``bench.py``; never by the shipped package. Each function
forwards to the C restatement of the reference algorithm named in its
docstring; array plumbing (dtype widening, contiguity) is the only work done
here. Parity status of the oracle itself is described at the top of
``oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_SRC = os.path.join(_HERE, "oracle.c")

GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 2, 8, 12, 14
GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q5_K = 3, 6, 7, 13
GGML_Q2_K, GGML_Q3_K = 10, 11
GGML_BLOCK = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210),
              GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24), GGML_Q5_K: (256, 176), GGML_Q2_K: (256, 84), GGML_Q3_K: (256, 110)}


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` with gcc (idempotent)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        cmd = ["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", "-fvisibility=hidden", _SRC, "-o", _SO, "-lm"]
        subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> int:
    """Use ``n`` OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1); returns the count in effect."""
    lib().orc_set_num_threads(ctypes.c_int(int(n)))
    return num_threads()


# ------------------------------------------------------------------ rounding
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """f32 values rounded through bf16 and widened back."""
    return bf16_bits_to_f32(to_bf16_bits(x))


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = _c(b, np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().orc_f16_to_f32(_p(b), _p(out), ctypes.c_int64(b.size))
    return out


def _scales_f32(scales: np.ndarray) -> np.ndarray:
    """Widen stored scales to f32 with no pre-rounding (awq.rs:362-367)."""
    return _c(scales, np.float32)


# ----------------------------------------------------------------------- AWQ
def awq_dequant(qweight, qzeros, scales, group_size: int | None = None) -> np.ndarray:
    """``dequantize_awq`` (awq.rs:325-440) -> dense ``[out, in]`` f32."""
    qweight = _c(np.asarray(qweight).astype(np.int64) & 0xFFFFFFFF, np.uint32)
    qzeros = _c(np.asarray(qzeros).astype(np.int64) & 0xFFFFFFFF, np.uint32)
    scales = _scales_f32(scales)
    k, packed_out = qweight.shape
    groups, n = scales.shape
    if n % 8 or packed_out * 8 != n or groups == 0 or k % groups:
        raise ValueError("AWQ shape mismatch")
    g = k // groups
    if group_size is not None and g != group_size:
        raise ValueError("AWQ group_size mismatch")
    if qzeros.shape != (groups, packed_out):
        raise ValueError(f"AWQ qzeros shape {qzeros.shape} != [{groups}, {packed_out}]")
    out = np.empty((n, k), np.float32)
    rc = lib().orc_awq_dequant_f32(_p(qweight), _p(qzeros), _p(scales), ctypes.c_int64(k), ctypes.c_int64(n),
                                   ctypes.c_int64(g), _p(out))
    if rc:
        raise ValueError(f"orc_awq_dequant_f32 rc={rc}")
    return out


def gptq_dequant(qweight, qzeros, scales, bits: int, sym: bool = False) -> np.ndarray:
    """``dequantize_gptq`` (awq.rs:442-590) -> dense ``[out, in]`` f32."""
    qweight = _c(np.asarray(qweight).astype(np.int64) & 0xFFFFFFFF, np.uint32)
    scales = _scales_f32(scales)
    pf = 32 // bits
    packed_in, n = qweight.shape
    k = packed_in * pf
    groups = scales.shape[0]
    if scales.shape[1] != n or groups == 0 or k % groups or n % pf:
        raise ValueError("GPTQ shape mismatch")
    zp = None
    if qzeros is not None:
        qzeros = _c(np.asarray(qzeros).astype(np.int64) & 0xFFFFFFFF, np.uint32)
        if qzeros.shape != (groups, n // pf):
            raise ValueError("GPTQ qzeros shape mismatch")
        zp = _p(qzeros)
    out = np.empty((n, k), np.float32)
    rc = lib().orc_gptq_dequant_f32(_p(qweight), zp, _p(scales), ctypes.c_int64(k), ctypes.c_int64(n),
                                    ctypes.c_int64(k // groups), ctypes.c_int(bits), ctypes.c_int(int(sym)), _p(out))
    if rc:
        raise ValueError(f"orc_gptq_dequant_f32 rc={rc}")
    return out


def w8a16_dequant(qweight, qzeros, scales) -> np.ndarray:
    """8-bit AWQ layout ``[in, out / 4]`` (quant_kernels.metal:1-16,40-48) -> dense ``[out, in]`` f32."""
    qweight = _c(np.asarray(qweight).astype(np.int64) & 0xFFFFFFFF, np.uint32)
    qzeros = _c(np.asarray(qzeros).astype(np.int64) & 0xFFFFFFFF, np.uint32)
    scales = _scales_f32(scales)
    k, packed_out = qweight.shape
    n = packed_out * 4
    groups = scales.shape[0]
    if scales.shape[1] != n or groups == 0 or k % groups or qzeros.shape != (groups, packed_out):
        raise ValueError("W8A16 shape mismatch")
    out = np.empty((n, k), np.float32)
    rc = lib().orc_w8a16_dequant_f32(_p(qweight), _p(qzeros), _p(scales), ctypes.c_int64(k), ctypes.c_int64(n),
                                     ctypes.c_int64(k // groups), _p(out))
    if rc:
        raise ValueError(f"orc_w8a16_dequant_f32 rc={rc}")
    return out


# ----------------------------------------------------------------------- FP8
def e4m3_decode(b: np.ndarray) -> np.ndarray:
    """Spec decode of E4M3fn bytes (metal_ops.rs:2944-2956)."""
    b = _c(b, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_e4m3_decode(_p(b), _p(out), ctypes.c_int64(b.size))
    return out


def fp8_dequant(w_bytes: np.ndarray, scale_inv) -> np.ndarray:
    """``Fp8Linear`` dequant (linear.rs:96-141 + weights.rs:207-234) -> f32 ``[out, in]``.

    ``scale_inv`` may be None, rank 0, rank 1 (``[out]`` or ``[1]``) or a 2-D
    grid that tiles the weight evenly, as the reference accepts.
    """
    w_bytes = _c(w_bytes, np.uint8)
    n, k = w_bytes.shape
    if scale_inv is None:
        return e4m3_decode(w_bytes)
    s = _c(scale_inv, np.float32)
    if s.ndim == 0:
        s = s.reshape(1, 1)
    elif s.ndim == 1:
        if s.shape[0] == n:
            s = s.reshape(n, 1)
        elif s.shape[0] == 1:
            s = s.reshape(1, 1)
        else:
            raise ValueError(f"invalid FP8 scale_inv shape {list(s.shape)}")
    elif s.ndim != 2:
        raise ValueError(f"invalid FP8 scale_inv rank {s.ndim}")
    out = np.empty((n, k), np.float32)
    rc = lib().orc_fp8_block_dequant_f32(_p(w_bytes), _p(s), ctypes.c_int64(n), ctypes.c_int64(k),
                                         ctypes.c_int64(s.shape[0]), ctypes.c_int64(s.shape[1]), _p(out))
    if rc:
        raise ValueError("block-wise FP8 weight_scale_inv does not tile weight evenly")
    return out


# --------------------------------------------------------------------- MXFP4
def mxfp4_dequant(blocks, scales, rows: int, cols: int) -> np.ndarray:
    """``dequantize_mxfp4_f32`` (mxfp4.rs:35-64)."""
    blocks = _c(blocks, np.uint8).reshape(-1)
    scales = _c(scales, np.uint8).reshape(-1)
    if cols % 32 or blocks.size != rows * (cols // 32) * 16 or scales.size != rows * (cols // 32):
        raise ValueError("MXFP4 buffer sizes do not match shape")
    out = np.empty((rows, cols), np.float32)
    lib().orc_mxfp4_dequant_f32(_p(blocks), _p(scales), ctypes.c_int64(rows), ctypes.c_int64(cols), _p(out))
    return out


# ---------------------------------------------------------------------- GGUF
def gguf_dequant(ggml_type: int, data, rows: int, cols: int) -> np.ndarray:
    """Per-element GGUF block dequant (quant_kernels.metal strips) -> f32 ``[rows, cols]``."""
    bel, bby = GGML_BLOCK[ggml_type]
    data = _c(data, np.uint8).reshape(-1)
    if cols % bel or data.size != rows * (cols // bel) * bby:
        raise ValueError("GGUF byte count does not match shape")
    out = np.empty((rows, cols), np.float32)
    rc = lib().orc_gguf_dequant_f32(ctypes.c_int(ggml_type), _p(data), ctypes.c_int64(rows), ctypes.c_int64(cols),
                                    _p(out))
    if rc:
        raise ValueError(f"orc_gguf_dequant_f32 rc={rc}")
    return out


# -------------------------------------------------------------------- linear
def linear(x, w, bias=None) -> np.ndarray:
    """``x @ w.T + bias`` in f32 (linear.rs:40-68); ``w`` is ``[out, in]``."""
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    b = None if bias is None else _c(bias, np.float32)
    y = np.empty((m, n), np.float32)
    lib().orc_linear_f32(_p(x), _p(w), None if b is None else _p(b), _p(y), ctypes.c_int64(m), ctypes.c_int64(k),
                         ctypes.c_int64(n))
    return y


def gated_ffn(x, w_gate_up, activation: str = "silu") -> np.ndarray:
    """``act(gate) * up`` of the fused gate+up projection (ffn.rs:385-470, the non-Metal branch):
    ``out = x @ w_gate_up.T`` in f32, ``gate = out[:, :I]``, ``up = out[:, I:]``, ``act`` = SiLU
    ``g / (1 + exp(-g))`` or tanh-GeLU ``0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))``, all in f32
    (the reference rounds ``out`` to the activation dtype first; parity is checked with a tolerance)."""
    out = linear(x, w_gate_up).astype(np.float64)
    inter = out.shape[1] // 2
    g, u = out[:, :inter], out[:, inter:]
    if activation == "silu":
        a = g / (1.0 + np.exp(-g))
    elif activation == "gelu_tanh":
        a = 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    else:
        raise ValueError(f"unknown activation {activation!r}")
    return (a * u).astype(np.float32)


# ----------------------------------------------------------------------- MoE
def moe_route(logits, top_k: int, norm_topk: bool = True):
    """softmax -> top-k -> renormalise (moe.rs:472-487)."""
    logits = _c(logits, np.float32)
    t, e = logits.shape
    idx = np.empty((t, top_k), np.int32)
    vals = np.empty((t, top_k), np.float32)
    lib().orc_moe_route(_p(logits), ctypes.c_int64(t), ctypes.c_int(e), ctypes.c_int(top_k),
                        ctypes.c_int(int(norm_topk)), _p(idx), _p(vals))
    return idx, vals


def gptoss_expert(x, w_gu, b_gu, w_dn, b_dn, limit: float = 7.0) -> np.ndarray:
    """One GPT-OSS expert on dequantized weights (moe.rs:152-173)."""
    x = _c(x, np.float32)
    w_gu, b_gu, w_dn, b_dn = (_c(a, np.float32) for a in (w_gu, b_gu, w_dn, b_dn))
    m, hidden = x.shape
    inter = w_dn.shape[1]
    out = np.empty((m, hidden), np.float32)
    lib().orc_gptoss_expert_f32(_p(x), _p(w_gu), _p(b_gu), _p(w_dn), _p(b_dn), ctypes.c_float(limit),
                                ctypes.c_int64(m), ctypes.c_int64(hidden), ctypes.c_int64(inter), _p(out))
    return out


def gptoss_moe(x, top_idx, top_vals, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias,
               hidden: int, inter: int, limit: float = 7.0, expert_range=None) -> np.ndarray:
    """``dispatch_sparse`` over MXFP4 GPT-OSS experts (moe.rs:563-607)."""
    x = _c(x, np.float32)
    top_idx = _c(top_idx, np.int32)
    top_vals = _c(top_vals, np.float32)
    t, top_k = top_idx.shape
    e = np.asarray(gu_bias).shape[0]
    gu_blocks, gu_scales, dn_blocks, dn_scales = (_c(a, np.uint8) for a in (gu_blocks, gu_scales, dn_blocks, dn_scales))
    gu_bias, dn_bias = _c(gu_bias, np.float32), _c(dn_bias, np.float32)
    lo, hi = (0, e) if expert_range is None else expert_range
    out = np.empty((t, hidden), np.float32)
    rc = lib().orc_gptoss_moe_f32(_p(x), _p(top_idx), _p(top_vals), ctypes.c_int64(t), ctypes.c_int(top_k),
                                  ctypes.c_int(e), ctypes.c_int64(hidden), ctypes.c_int64(inter), _p(gu_blocks),
                                  _p(gu_scales), _p(gu_bias), _p(dn_blocks), _p(dn_scales), _p(dn_bias),
                                  ctypes.c_float(limit), ctypes.c_int(lo), ctypes.c_int(hi), _p(out))
    if rc:
        raise ValueError(f"orc_gptoss_moe_f32 rc={rc}")
    return out

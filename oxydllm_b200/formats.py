"""Packed weight formats consumed by the kernels, and host-side encoders for them.

The layouts are the reference's, unchanged:

* AWQ 4-bit (awq.rs:7-12,23-24): ``qweight`` u32 ``[in, out/8]``, nibble slot
  ``k`` of word ``(i, j)`` holds out column ``8j + AWQ_PACK_ORDER[k]``;
  ``qzeros`` ``[in/g, out/8]`` packed the same way; ``scales`` ``[in/g, out]``.
* GPTQ 4/8-bit (awq.rs:10-12): ``qweight`` ``[in/pf, out]`` sequential
  LSB-first along in; ``qzeros`` ``[in/g, out/pf]`` sequential along out,
  storing zero-1.
* GGUF blocks along in, rows contiguous (metal_ops.rs:5228-5241): Q4_0 18 B/32,
  Q8_0 34 B/32, Q4_K 144 B/256, Q6_K 210 B/256.
* FP8 E4M3 bytes ``[out, in]`` + f32 scale grid (weights.rs:207-234).
* MXFP4 (mxfp4.rs:3-6): ``blocks`` u8 ``[rows, in/32, 16]`` low nibble first,
  ``scales`` u8 ``[rows, in/32]`` E8M0.

The encoders exist to make well-formed synthetic weights; only
``rtn_quantize_awq``, ``compressed_to_awq`` and ``concat_awq_along_out`` mirror
reference functions. The Q4_K/Q6_K encoders are this project's own (candle's
quantizer is not part of the reference tree); any encoder that emits valid
blocks exercises the kernels identically.
"""
from __future__ import annotations

import numpy as np

AWQ_PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)
AWQ_PACK_FACTOR = 8

GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 2, 8, 12, 14
GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q5_K = 3, 6, 7, 13
GGML_Q2_K, GGML_Q3_K = 10, 11
#: ggml type id -> (elements per block, bytes per block)
GGML_BLOCK = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210),
              GGML_Q4_1: (32, 20), GGML_Q5_0: (32, 22), GGML_Q5_1: (32, 24), GGML_Q5_K: (256, 176), GGML_Q2_K: (256, 84), GGML_Q3_K: (256, 110)}
GGML_NAME = {GGML_Q4_0: "Q4_0", GGML_Q8_0: "Q8_0", GGML_Q4_K: "Q4_K", GGML_Q6_K: "Q6_K",
             GGML_Q4_1: "Q4_1", GGML_Q5_0: "Q5_0", GGML_Q5_1: "Q5_1", GGML_Q5_K: "Q5_K", GGML_Q2_K: "Q2_K", GGML_Q3_K: "Q3_K"}


# ----------------------------------------------------------------------- AWQ
def pack_awq(values: np.ndarray) -> np.ndarray:
    """Pack int4 values ``[rows, out]`` into AWQ words ``[rows, out/8]`` (awq.rs:913-929)."""
    values = np.asarray(values)
    rows, out = values.shape
    if out % AWQ_PACK_FACTOR:
        raise ValueError(f"AWQ out_features ({out}) not divisible by pack factor 8")
    v = (values.astype(np.uint32) & 0xF).reshape(rows, out // 8, 8)
    word = np.zeros((rows, out // 8), np.uint32)
    for k, off in enumerate(AWQ_PACK_ORDER):
        word |= v[:, :, off] << np.uint32(4 * k)
    return word


def pack_w8a16(values: np.ndarray) -> np.ndarray:
    """Pack uint8 values ``[rows, out]`` into the 8-bit AWQ layout ``[rows, out/4]``: byte c of word j is out
    column ``4 j + c`` (identity order at 8 bits, quant_kernels.metal:1-16)."""
    values = np.asarray(values)
    rows, out = values.shape
    if out % 4:
        raise ValueError(f"W8A16 out_features ({out}) not divisible by pack factor 4")
    v = (values.astype(np.uint32) & 0xFF).reshape(rows, out // 4, 4)
    return v[:, :, 0] | (v[:, :, 1] << np.uint32(8)) | (v[:, :, 2] << np.uint32(16)) | (v[:, :, 3] << np.uint32(24))


def unpack_awq(words: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_awq`: ``[rows, out/8]`` words -> ``[rows, out]`` uint8."""
    words = np.asarray(words).astype(np.int64).astype(np.uint32) if words.dtype != np.uint32 else words
    rows, packed = words.shape
    out = np.empty((rows, packed, 8), np.uint8)
    for k, off in enumerate(AWQ_PACK_ORDER):
        out[:, :, off] = (words >> np.uint32(4 * k)) & 0xF
    return out.reshape(rows, packed * 8)


def _round_half_away(x: np.ndarray) -> np.ndarray:
    """Rust ``f32::round``: halves round away from zero (numpy's ``round`` is half-to-even)."""
    return np.sign(x) * np.floor(np.abs(x) + np.float32(0.5))


def rtn_quantize_awq(weight: np.ndarray, group_size: int):
    """Round-to-nearest 4-bit group quantizer in AWQ layout (awq.rs:637-742).

    ``weight`` is ``[out, in]`` f32. Returns ``(qweight, qzeros, scales_f32)``.
    """
    w = np.ascontiguousarray(weight, np.float32)
    out_f, in_f = w.shape
    if out_f % 8:
        raise ValueError(f"rtn_quantize_awq: out_features ({out_f}) must be a multiple of 8")
    if group_size == 0 or in_f % group_size:
        raise ValueError(f"rtn_quantize_awq: in_features ({in_f}) not divisible by group_size ({group_size})")
    groups = in_f // group_size
    grp = w.reshape(out_f, groups, group_size)
    xmin = np.minimum(grp.min(axis=2), np.float32(0.0))
    xmax = np.maximum(grp.max(axis=2), np.float32(0.0))
    flat = (xmax - xmin) < np.float32(1e-12)
    scale = ((xmax - xmin) / np.float32(15.0)).astype(np.float32)
    safe = np.where(flat, np.float32(1.0), scale)
    zero = np.clip(_round_half_away(-xmin / safe), 0.0, 15.0).astype(np.float32)
    q = np.clip(_round_half_away(grp / safe[:, :, None] + zero[:, :, None]), 0.0, 15.0)
    q = np.where(flat[:, :, None], 1.0, q)
    zero = np.where(flat, 0.0, zero)
    scale = np.where(flat, xmin, scale).astype(np.float32)
    qnib = q.reshape(out_f, in_f).astype(np.uint8)
    qweight = pack_awq(qnib.T.copy())
    qzeros = pack_awq(zero.astype(np.uint8).T.copy())
    return qweight, qzeros, np.ascontiguousarray(scale.T)


def compressed_to_awq(weight_packed: np.ndarray, weight_scale: np.ndarray):
    """compressed-tensors pack-quantized int4 -> AWQ layout (awq.rs:187-254).

    ``weight_packed`` ``[out, in/8]`` holds sequential LSB-first offset-binary
    nibbles; ``weight_scale`` is ``[out, groups]``. Zero points become the
    constant 8 (``0x88888888`` words).
    """
    ct = np.asarray(weight_packed).astype(np.int64).astype(np.uint32) if weight_packed.dtype != np.uint32 else weight_packed
    if ct.ndim != 2:
        raise ValueError("weight_packed must be 2-D [out, in/8]")
    out_f, packed_in = ct.shape
    in_f = packed_in * 8
    if weight_scale.ndim != 2:
        raise ValueError("weight_scale must be 2-D [out, groups]")
    scale_out, groups = weight_scale.shape
    if scale_out != out_f:
        raise ValueError(f"weight_scale dim0 {scale_out} != weight_packed out_features {out_f}")
    if groups == 0 or in_f % groups:
        raise ValueError(f"in_features {in_f} not divisible by scale groups {groups}")
    if out_f % 8:
        raise ValueError(f"out_features {out_f} not divisible by pack factor 8")
    nib = np.empty((out_f, packed_in, 8), np.uint8)
    for k in range(8):
        nib[:, :, k] = (ct >> np.uint32(4 * k)) & 0xF
    nib = nib.reshape(out_f, in_f)
    qweight = pack_awq(nib.T.copy())
    qzeros = np.full((groups, out_f // 8), 0x88888888, np.uint32)
    scales = np.ascontiguousarray(np.asarray(weight_scale).T)
    return qweight, qzeros, scales


def concat_awq_along_out(parts):
    """Fuse AWQ triplets along out features (awq.rs:256-323). ``parts`` = [(qweight, qzeros, scales), ...]."""
    if not parts:
        raise ValueError("concat_awq_along_out: no parts")
    k0 = parts[0][0].shape[0]
    g0 = parts[0][2].shape[0]
    for i, (qw, qz, sc) in enumerate(parts[1:], 1):
        if qw.shape[0] != k0:
            raise ValueError(f"AWQ fuse: in_features mismatch at part {i}: expected {k0}, got {qw.shape[0]}")
        if sc.shape[0] != g0:
            raise ValueError(f"AWQ fuse: group_size mismatch at part {i}")
    for i, (qw, qz, sc) in enumerate(parts):
        if sc.shape[1] % 8:
            raise ValueError(f"AWQ fuse: part {i} out_features {sc.shape[1]} not divisible by pack_factor 8")
    return (np.concatenate([p[0] for p in parts], axis=1), np.concatenate([p[1] for p in parts], axis=1),
            np.concatenate([p[2] for p in parts], axis=1))


# ---------------------------------------------------------------------- GPTQ
def pack_gptq_qweight(values: np.ndarray, bits: int) -> np.ndarray:
    """``[in, out]`` ints -> ``[in/pf, out]`` words, sequential along in (awq.rs:1123-1143)."""
    pf = 32 // bits
    k, n = values.shape
    v = (np.asarray(values).astype(np.uint32) & ((1 << bits) - 1)).reshape(k // pf, pf, n)
    word = np.zeros((k // pf, n), np.uint32)
    for s in range(pf):
        word |= v[:, s, :] << np.uint32(bits * s)
    return word


def pack_gptq_qzeros(values: np.ndarray, bits: int) -> np.ndarray:
    """``[groups, out]`` ints -> ``[groups, out/pf]`` words, sequential along out (awq.rs:1145-1167)."""
    pf = 32 // bits
    g, n = values.shape
    v = (np.asarray(values).astype(np.uint32) & ((1 << bits) - 1)).reshape(g, n // pf, pf)
    word = np.zeros((g, n // pf), np.uint32)
    for s in range(pf):
        word |= v[:, :, s] << np.uint32(bits * s)
    return word


# ----------------------------------------------------------------------- FP8
def _e4m3_table() -> np.ndarray:
    t = np.empty(127, np.float64)
    for c in range(127):
        e, m = c >> 3, c & 7
        t[c] = m / 8.0 * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
    return t


_E4M3_POS = _e4m3_table()
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """f32 -> E4M3fn bytes, round-to-nearest-even, saturating at +-448."""
    x = np.asarray(x, np.float64)
    a = np.minimum(np.abs(x), 448.0)
    code = np.searchsorted(_E4M3_MID, a, side="left")  # midpoints strictly below a
    tie = (code < 126) & (a == _E4M3_MID[np.minimum(code, 125)])
    code = np.where(tie & (code % 2 == 1), code + 1, code)
    return (code.astype(np.uint8) | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


def quantize_fp8_block(weight: np.ndarray, block: int = 128):
    """Per-``block x block`` scale = blockmax/448, q = e4m3(W/scale). Returns (bytes [out,in], scale_inv f32 grid)."""
    w = np.ascontiguousarray(weight, np.float32)
    n, k = w.shape
    if n % block or k % block:
        raise ValueError("weight does not tile into blocks")
    t = w.reshape(n // block, block, k // block, block)
    amax = np.abs(t).max(axis=(1, 3))
    scale = (np.maximum(amax, np.float32(1e-12)) / np.float32(448.0)).astype(np.float32)
    q = e4m3_encode((t / scale[:, None, :, None]).astype(np.float32)).reshape(n, k)
    return q, scale


# --------------------------------------------------------------------- MXFP4
_E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_E2M1_MID = (_E2M1[:-1] + _E2M1[1:]) / 2.0


def quantize_mxfp4(weight: np.ndarray):
    """``[rows, in]`` f32 -> (blocks u8 [rows, in/32, 16], scales u8 [rows, in/32]).

    Own round-to-nearest-even encoder: shared exponent floor(log2(amax)) - 2 so
    the block maximum lands in the top binade of E2M1 (max magnitude 6).
    """
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    if k % 32:
        raise ValueError("in_features must be a multiple of 32")
    b = w.reshape(rows, k // 32, 32).astype(np.float64)
    amax = np.abs(b).max(axis=2)
    e = np.where(amax > 0, np.floor(np.log2(np.maximum(amax, 1e-300))) - 2.0, -127.0)
    e = np.clip(e, -127.0, 127.0)
    scaled = np.minimum(np.abs(b) / (2.0 ** e)[:, :, None], 6.0)
    code = np.searchsorted(_E2M1_MID, scaled, side="left")
    tie = (code < 7) & (scaled == _E2M1_MID[np.minimum(code, 6)])
    code = np.where(tie & (code % 2 == 1), code + 1, code).astype(np.uint8)
    code |= (np.signbit(b).astype(np.uint8) << 3)
    blocks = (code[:, :, 0::2] | (code[:, :, 1::2] << 4)).astype(np.uint8)
    scales = (e + 127.0).astype(np.uint8)
    return blocks, scales


# ---------------------------------------------------------------------- GGUF
def _f16(x):
    return np.asarray(x, np.float32).astype(np.float16)


def quantize_q8_0(weight: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    d = _f16(np.abs(b).max(axis=2) / 127.0)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1.0), 0.0)
    q = np.clip(np.round(b * inv[:, :, None]), -127, 127).astype(np.int8)
    out = np.empty((rows, k // 32, 34), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(weight: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    idx = np.abs(b).argmax(axis=2)
    mx = np.take_along_axis(b, idx[:, :, None], axis=2)[:, :, 0]
    d = _f16(mx / -8.0)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1.0), 0.0)
    q = np.clip(np.floor(b * inv[:, :, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((rows, k // 32, 18), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 2:] = q[:, :, :16] | (q[:, :, 16:] << 4)
    return out.reshape(-1)


def quantize_q4_k(weight: np.ndarray) -> np.ndarray:
    """Own Q4_K encoder: affine 4-bit per 32-element sub-block, 6-bit sub-block scales/mins."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    nb = k // 256
    sb = w.reshape(rows, nb, 8, 32)
    mn = np.minimum(sb.min(axis=3), 0.0)
    mxv = np.maximum(sb.max(axis=3), 0.0)
    sub_scale = (mxv - mn) / 15.0
    sub_min = -mn
    d = _f16(sub_scale.max(axis=2) / 63.0)
    dmin = _f16(sub_min.max(axis=2) / 63.0)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.clip(np.round(sub_scale / np.where(df > 0, df, 1.0)[:, :, None]), 0, 63).astype(np.uint8)
    mq = np.clip(np.round(sub_min / np.where(dmf > 0, dmf, 1.0)[:, :, None]), 0, 63).astype(np.uint8)
    eff_s = df[:, :, None] * sc.astype(np.float32)
    eff_m = dmf[:, :, None] * mq.astype(np.float32)
    q = np.clip(np.round((sb + eff_m[:, :, :, None]) / np.where(eff_s > 0, eff_s, 1.0)[:, :, :, None]), 0, 15)
    q = q.astype(np.uint8)
    out = np.empty((rows, nb, 144), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:4] = dmin.view(np.uint8).reshape(rows, nb, 2)
    s12 = np.empty((rows, nb, 12), np.uint8)
    for j in range(4):
        s12[:, :, j] = sc[:, :, j] | ((sc[:, :, j + 4] >> 4) << 6)
        s12[:, :, j + 4] = mq[:, :, j] | ((mq[:, :, j + 4] >> 4) << 6)
        s12[:, :, j + 8] = (sc[:, :, j + 4] & 0xF) | ((mq[:, :, j + 4] & 0xF) << 4)
    out[:, :, 4:16] = s12
    qp = q.reshape(rows, nb, 4, 2, 32)
    out[:, :, 16:] = (qp[:, :, :, 0, :] | (qp[:, :, :, 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(-1)


def quantize_q6_k(weight: np.ndarray) -> np.ndarray:
    """Own Q6_K encoder: symmetric 6-bit per 16-element sub-block, int8 sub-block scales."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    nb = k // 256
    sb = w.reshape(rows, nb, 16, 16)
    sub = np.abs(sb).max(axis=3) / 31.0
    d = _f16(sub.max(axis=2) / 127.0)
    df = d.astype(np.float32)
    sc = np.clip(np.round(sub / np.where(df > 0, df, 1.0)[:, :, None]), 0, 127).astype(np.int8)
    eff = df[:, :, None] * sc.astype(np.float32)
    q = np.clip(np.round(sb / np.where(eff > 0, eff, 1.0)[:, :, :, None]), -32, 31).astype(np.int32) + 32
    q = q.reshape(rows, nb, 2, 4, 32).astype(np.uint8)  # [half, quadrant, l]
    out = np.empty((rows, nb, 210), np.uint8)
    ql = np.empty((rows, nb, 2, 64), np.uint8)
    ql[:, :, :, 0:32] = (q[:, :, :, 0, :] & 0xF) | ((q[:, :, :, 2, :] & 0xF) << 4)
    ql[:, :, :, 32:64] = (q[:, :, :, 1, :] & 0xF) | ((q[:, :, :, 3, :] & 0xF) << 4)
    qh = ((q[:, :, :, 0, :] >> 4) | ((q[:, :, :, 1, :] >> 4) << 2) | ((q[:, :, :, 2, :] >> 4) << 4)
          | ((q[:, :, :, 3, :] >> 4) << 6)).astype(np.uint8)
    out[:, :, 0:128] = ql.reshape(rows, nb, 128)
    out[:, :, 128:192] = qh.reshape(rows, nb, 64)
    # scale index = 8*half + 2*quadrant + l/16; sub-block t covers elements 16t..16t+15 = (half, quadrant, l/16)
    out[:, :, 192:208] = sc.view(np.uint8)
    out[:, :, 208:210] = d.view(np.uint8).reshape(rows, nb, 2)
    return out.reshape(-1)


def _pack5(q: np.ndarray):
    """5-bit codes [rows, nb, 32] -> (qh u8 [rows, nb, 4], qs u8 [rows, nb, 16]): bit j of qh is the fifth bit of element j."""
    hi = (q >> 4).astype(np.uint32)
    qh = (hi << np.arange(32, dtype=np.uint32)).sum(axis=2, dtype=np.uint32)
    qh4 = np.ascontiguousarray(qh).view(np.uint8).reshape(q.shape[0], q.shape[1], 4)
    lo = (q & 0xF).astype(np.uint8)
    return qh4, lo[:, :, :16] | (lo[:, :, 16:] << 4)


def quantize_q4_1(weight: np.ndarray) -> np.ndarray:
    """Q4_1 {f16 d; f16 m; u8 qs[16]}: affine 4-bit per 32 elements, w = q * d + m."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    mn, mx = b.min(axis=2), b.max(axis=2)
    d, m = _f16((mx - mn) / 15.0), _f16(mn)
    df, mf = d.astype(np.float32), m.astype(np.float32)
    q = np.clip(np.round((b - mf[:, :, None]) / np.where(df > 0, df, 1.0)[:, :, None]), 0, 15).astype(np.uint8)
    out = np.empty((rows, k // 32, 20), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 2:4] = m.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 4:] = q[:, :, :16] | (q[:, :, 16:] << 4)
    return out.reshape(-1)


def quantize_q5_0(weight: np.ndarray) -> np.ndarray:
    """Q5_0 {f16 d; u8 qh[4]; u8 qs[16]}: symmetric 5-bit per 32 elements, w = (q - 16) * d."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    idx = np.abs(b).argmax(axis=2)
    mx = np.take_along_axis(b, idx[:, :, None], axis=2)[:, :, 0]
    d = _f16(mx / -16.0)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1.0), 0.0)
    q = np.clip(np.floor(b * inv[:, :, None] + 16.5), 0, 31).astype(np.uint8)
    qh4, qs = _pack5(q)
    out = np.empty((rows, k // 32, 22), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 2:6] = qh4
    out[:, :, 6:] = qs
    return out.reshape(-1)


def quantize_q5_1(weight: np.ndarray) -> np.ndarray:
    """Q5_1 {f16 d; f16 m; u8 qh[4]; u8 qs[16]}: affine 5-bit per 32 elements, w = q * d + m."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    mn, mx = b.min(axis=2), b.max(axis=2)
    d, m = _f16((mx - mn) / 31.0), _f16(mn)
    df, mf = d.astype(np.float32), m.astype(np.float32)
    q = np.clip(np.round((b - mf[:, :, None]) / np.where(df > 0, df, 1.0)[:, :, None]), 0, 31).astype(np.uint8)
    qh4, qs = _pack5(q)
    out = np.empty((rows, k // 32, 24), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 2:4] = m.view(np.uint8).reshape(rows, k // 32, 2)
    out[:, :, 4:8] = qh4
    out[:, :, 8:] = qs
    return out.reshape(-1)


def quantize_q5_k(weight: np.ndarray) -> np.ndarray:
    """Own Q5_K encoder: Q4_K's layout with 5-bit codes; bit j of qh[el] is the fifth bit of sub-block j's element el."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    nb = k // 256
    sb = w.reshape(rows, nb, 8, 32)
    mn = np.minimum(sb.min(axis=3), 0.0)
    mxv = np.maximum(sb.max(axis=3), 0.0)
    sub_scale = (mxv - mn) / 31.0
    sub_min = -mn
    d = _f16(sub_scale.max(axis=2) / 63.0)
    dmin = _f16(sub_min.max(axis=2) / 63.0)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.clip(np.round(sub_scale / np.where(df > 0, df, 1.0)[:, :, None]), 0, 63).astype(np.uint8)
    mq = np.clip(np.round(sub_min / np.where(dmf > 0, dmf, 1.0)[:, :, None]), 0, 63).astype(np.uint8)
    eff_s = df[:, :, None] * sc.astype(np.float32)
    eff_m = dmf[:, :, None] * mq.astype(np.float32)
    q = np.clip(np.round((sb + eff_m[:, :, :, None]) / np.where(eff_s > 0, eff_s, 1.0)[:, :, :, None]), 0, 31)
    q = q.astype(np.uint8)
    out = np.empty((rows, nb, 176), np.uint8)
    out[:, :, 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:4] = dmin.view(np.uint8).reshape(rows, nb, 2)
    s12 = np.empty((rows, nb, 12), np.uint8)
    for j in range(4):
        s12[:, :, j] = sc[:, :, j] | ((sc[:, :, j + 4] >> 4) << 6)
        s12[:, :, j + 4] = mq[:, :, j] | ((mq[:, :, j + 4] >> 4) << 6)
        s12[:, :, j + 8] = (sc[:, :, j + 4] & 0xF) | ((mq[:, :, j + 4] & 0xF) << 4)
    out[:, :, 4:16] = s12
    qh = np.zeros((rows, nb, 32), np.uint8)
    for j in range(8):
        qh |= ((q[:, :, j, :] >> 4) << j).astype(np.uint8)
    out[:, :, 16:48] = qh
    lo = (q & 0xF).reshape(rows, nb, 4, 2, 32)
    out[:, :, 48:] = (lo[:, :, :, 0, :] | (lo[:, :, :, 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(-1)

def quantize_q2_k(weight: np.ndarray) -> np.ndarray:
    """Own Q2_K encoder (block_q2_K: ``scales[16]``, ``qs[64]``, f16 ``d``, f16 ``dmin``): sixteen sub-blocks of 16
    with a 4-bit scale and a 4-bit min each; element e sits in ``qs[(e >> 7) * 32 + (e & 31)]`` at bit ``2 * ((e >> 5) & 3)``."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    assert k % 256 == 0
    nb = k // 256
    x = w.reshape(rows, nb, 16, 16)
    mins = np.maximum(-x.min(axis=3), 0.0)                    # [rows, nb, 16]
    scl = (x.max(axis=3) + mins) / 3.0
    d = (scl.max(axis=2) / 15.0).astype(np.float16).astype(np.float32)
    dmin = (mins.max(axis=2) / 15.0).astype(np.float16).astype(np.float32)
    sc = np.where(d[..., None] > 0, np.clip(np.rint(scl / np.where(d > 0, d, 1.0)[..., None]), 0, 15), 0).astype(np.uint8)
    mn = np.where(dmin[..., None] > 0, np.clip(np.rint(mins / np.where(dmin > 0, dmin, 1.0)[..., None]), 0, 15), 0).astype(np.uint8)
    dl = d[..., None] * sc
    ml = dmin[..., None] * mn
    q = np.where(dl[..., None] > 0, np.clip(np.rint((x + ml[..., None]) / np.where(dl > 0, dl, 1.0)[..., None]), 0, 3), 0).astype(np.uint8)
    q = q.reshape(rows, nb, 2, 4, 32)                          # [half, shift index, byte]
    qs = (q[:, :, :, 0] | (q[:, :, :, 1] << 2) | (q[:, :, :, 2] << 4) | (q[:, :, :, 3] << 6)).astype(np.uint8)
    out = np.empty((rows, nb, 84), np.uint8)
    out[:, :, 0:16] = sc | (mn << 4)
    out[:, :, 16:80] = qs.reshape(rows, nb, 64)
    out[:, :, 80:82] = d.astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 82:84] = dmin.astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return out.reshape(-1)


def quantize_q3_k(weight: np.ndarray) -> np.ndarray:
    """Own Q3_K encoder (block_q3_K: ``hmask[32]``, ``qs[64]``, ``scales[12]``, f16 ``d``): sixteen sub-blocks of 16 with
    a signed 6-bit scale each; a 3-bit code is two bits in ``qs`` (as in Q2_K) and bit ``e >> 5`` of ``hmask[e & 31]``."""
    w = np.ascontiguousarray(weight, np.float32)
    rows, k = w.shape
    assert k % 256 == 0
    nb = k // 256
    x = w.reshape(rows, nb, 16, 16)
    scl = np.abs(x).max(axis=3) / 4.0                          # codes -4..3
    d = (scl.max(axis=2) / 31.0).astype(np.float16).astype(np.float32)
    sc = np.where(d[..., None] > 0, np.clip(np.rint(scl / np.where(d > 0, d, 1.0)[..., None]), 0, 31), 0).astype(np.int32)
    dl = d[..., None] * sc
    q = np.where(dl[..., None] > 0, np.clip(np.rint(x / np.where(dl > 0, dl, 1.0)[..., None]), -4, 3), 0).astype(np.int32) + 4
    q = q.reshape(rows, nb, 2, 4, 32).astype(np.uint8)        # [half, shift index, byte]
    lo = q & 3
    qs = (lo[:, :, :, 0] | (lo[:, :, :, 1] << 2) | (lo[:, :, :, 2] << 4) | (lo[:, :, :, 3] << 6)).astype(np.uint8)
    hb = (q >> 2).reshape(rows, nb, 8, 32)                     # bit index = half * 4 + shift index
    hmask = np.zeros((rows, nb, 32), np.uint8)
    for b in range(8):
        hmask |= (hb[:, :, b] << b).astype(np.uint8)
    s6 = (sc + 32).astype(np.uint8)                            # stored scale
    scales = np.zeros((rows, nb, 12), np.uint8)
    scales[:, :, 0:8] = (s6[:, :, 0:8] & 0x0F) | ((s6[:, :, 8:16] & 0x0F) << 4)
    for i in range(16):
        scales[:, :, 8 + (i & 3)] |= ((s6[:, :, i] >> 4) & 3) << (2 * (i >> 2))
    out = np.empty((rows, nb, 110), np.uint8)
    out[:, :, 0:32] = hmask
    out[:, :, 32:96] = qs.reshape(rows, nb, 64)
    out[:, :, 96:108] = scales
    out[:, :, 108:110] = d.astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return out.reshape(-1)


GGML_QUANTIZE = {GGML_Q4_0: quantize_q4_0, GGML_Q8_0: quantize_q8_0, GGML_Q4_K: quantize_q4_k,
                 GGML_Q6_K: quantize_q6_k, GGML_Q4_1: quantize_q4_1, GGML_Q5_0: quantize_q5_0,
                 GGML_Q5_1: quantize_q5_1, GGML_Q5_K: quantize_q5_k, GGML_Q2_K: quantize_q2_k,
                 GGML_Q3_K: quantize_q3_k}

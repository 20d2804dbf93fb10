"""The CPU oracle replays every CPU known-answer test the reference holds for the
quantized-matmul path. Inputs are built by the formulas in the reference's own
tests; expected values by the independent scalar formula each test states."""
import numpy as np
import pytest

import oracle
from oxydllm_b200 import formats as F


def _awq_case(k, n, g, wf, zf, sf):
    iw = np.array([[wf(i, j) for j in range(n)] for i in range(k)], np.uint8)
    iz = np.array([[zf(gi, j) for j in range(n)] for gi in range(k // g)], np.uint8)
    sc = np.array([[sf(gi, j) for j in range(n)] for gi in range(k // g)], np.float32)
    expected = np.empty((n, k), np.float32)
    for i in range(k):
        for j in range(n):
            expected[j, i] = np.float32(int(iw[i, j]) - int(iz[i // g, j])) * sc[i // g, j]
    return F.pack_awq(iw), F.pack_awq(iz), sc, expected


def test_dequantize_awq_recovers_original_matrix():
    # awq.rs:953-1011
    qw, qz, sc, expected = _awq_case(8, 16, 4, lambda i, j: (i * 3 + j * 5 + 1) & 0xF, lambda g, j: (g * 7 + j) & 0xF,
                                     lambda g, j: np.float32(0.01) * np.float32(g + 1) + np.float32(0.001) * np.float32(j + 1))
    got = oracle.awq_dequant(qw, qz, sc)
    assert got.shape == (16, 8)
    assert np.abs(got - expected).max() < 1e-6
    assert np.array_equal(got, expected)  # same operations, same bits


def test_any_linear_from_awq_matches_reference_linear():
    # linear.rs:687-787
    k, n, g = 4, 8, 2
    qw, qz, sc, w_ref = _awq_case(k, n, g, lambda i, j: (i * 5 + j) & 0xF, lambda gi, j: (gi + j) & 0xF,
                                  lambda gi, j: np.float32(0.05) * np.float32(gi + 1.0) + np.float32(0.01) * np.float32(j))
    bias = np.array([0.1 * j for j in range(n)], np.float32)
    x = np.array([[0.1 * v - 0.05 for v in range(k)]], np.float32)
    out = oracle.linear(x, oracle.awq_dequant(qw, qz, sc), bias)
    ref = x @ w_ref.T + bias
    assert np.abs(out - ref).max() < 1e-6


def test_concat_awq_along_out_matches_separate_dequant():
    # awq.rs:1031-1093
    k, g = 8, 4
    parts, seps = [], []
    for idx, n in enumerate([16, 8, 8]):
        qw, qz, sc, _ = _awq_case(k, n, g, lambda i, j: (i + j + idx * 3) & 0xF, lambda gi, j: (gi * 2 + j + idx) & 0xF,
                                  lambda gi, j: 0.02 * (gi + 1) + 0.005 * (j + 1) + 0.001 * idx)
        parts.append((qw, qz, sc))
        seps.append(oracle.awq_dequant(qw, qz, sc))
    fqw, fqz, fsc = F.concat_awq_along_out(parts)
    assert fsc.shape == (2, 32)
    fused = oracle.awq_dequant(fqw, fqz, fsc)
    assert np.abs(fused - np.concatenate(seps, axis=0)).max() < 1e-6


def test_concat_awq_rejects_in_features_mismatch():
    # awq.rs:1095-1110
    def mk(k):
        return (np.zeros((k, 1), np.uint32), np.zeros((1, 1), np.uint32), np.zeros((1, 8), np.float32))
    with pytest.raises(ValueError):
        F.concat_awq_along_out([mk(4), mk(8)])


def test_dequantize_awq_rejects_wrong_shapes():
    # awq.rs:1112-1121: qweight [8,2] implies 16 outputs, scales say 8
    with pytest.raises(ValueError):
        oracle.awq_dequant(np.zeros((8, 2), np.uint32), np.zeros((2, 2), np.uint32), np.zeros((2, 8), np.float32))


def test_compressed_to_awq_matches_direct_dequant():
    # awq.rs:753-800
    out_f, in_f, group = 16, 64, 32
    groups = in_f // group
    q = np.array([(i % 16) - 8 for i in range(out_f * in_f)], np.int32).reshape(out_f, in_f)
    scale = np.array([0.01 + (i % 7) * 0.003 for i in range(out_f * groups)], np.float32).reshape(out_f, groups)
    packed = np.zeros((out_f, in_f // 8), np.uint32)
    for kk in range(8):
        packed |= ((q[:, kk::8] + 8).astype(np.uint32) & 0xF) << np.uint32(4 * kk)
    qw, qz, sc = F.compressed_to_awq(packed.view(np.int32), scale)
    assert qw.shape == (in_f, out_f // 8) and sc.shape == (groups, out_f)
    dq = oracle.awq_dequant(qw, qz, sc)
    expected = q.astype(np.float32) * np.repeat(scale, group, axis=1)
    assert np.abs(dq - expected).max() < 1e-6


def test_rtn_quantize_awq_round_trips():
    # awq.rs:802-835
    out_f, in_f, group = 16, 64, 32
    data = np.sin(np.arange(out_f * in_f, dtype=np.float32) * np.float32(0.013)).reshape(out_f, in_f)
    qw, qz, sc = F.rtn_quantize_awq(data, group)
    assert qw.shape == (in_f, out_f // 8) and qz.shape == (in_f // group, out_f // 8) and sc.shape == (in_f // group, out_f)
    dq = oracle.awq_dequant(qw, qz, sc)
    rel = np.sqrt(((dq - data).astype(np.float64) ** 2).sum() / (data.astype(np.float64) ** 2).sum())
    assert rel < 0.05


@pytest.mark.parametrize("bits,wf,zf,sf,tol", [
    (8, lambda i, j: (i * 11 + j * 7) & 0xFF, lambda g, j: (g * 31 + j * 17 + 1) & 0xFF,
     lambda g, j: 0.02 * (g + 1) + 0.003 * (j + 1), 1e-5),   # awq.rs:1169-1228
    (4, lambda i, j: (i * 3 + j * 5) & 0xF, lambda g, j: (g * 2 + j) & 0xF,
     lambda g, j: 0.01 * (g + 1) + 0.002 * (j + 1), 1e-5),   # awq.rs:1230-1283
])
def test_dequantize_gptq_matches_reference(bits, wf, zf, sf, tol):
    k, n, g = 32, 16, 16
    iw = np.array([[wf(i, j) for j in range(n)] for i in range(k)], np.uint32)
    iz = np.array([[zf(gi, j) for j in range(n)] for gi in range(k // g)], np.uint32)
    sc = np.array([[sf(gi, j) for j in range(n)] for gi in range(k // g)], np.float32)
    expected = np.empty((n, k), np.float32)
    for i in range(k):
        for j in range(n):
            expected[j, i] = np.float32(int(iw[i, j]) - (int(iz[i // g, j]) + 1)) * sc[i // g, j]
    got = oracle.gptq_dequant(F.pack_gptq_qweight(iw, bits), F.pack_gptq_qzeros(iz, bits), sc, bits)
    assert got.shape == (n, k)
    assert np.abs(got - expected).max() < tol


def test_gptq_symmetric_zero_point():
    # awq.rs:567,580-586: sym or missing qzeros -> zero = 2^(bits-1) - 1 before the +1
    k, n, g = 16, 8, 8
    iw = (np.arange(k * n).reshape(k, n) % 16).astype(np.uint32)
    sc = np.full((k // g, n), 0.5, np.float32)
    got = oracle.gptq_dequant(F.pack_gptq_qweight(iw, 4), None, sc, 4, sym=True)
    assert np.array_equal(got, ((iw.astype(np.float32) - 8.0) * 0.5).T)


def test_e4m3_decode_every_byte_matches_spec():
    # metal_ops.rs:2944-2989
    def spec(v):
        s, e, m = v >> 7, (v >> 3) & 0xF, v & 7
        if e == 0:
            val = m * 0.125 * 2.0 ** -6
        elif e == 15 and m == 7:
            val = float("nan")
        else:
            val = (1.0 + m * 0.125) * 2.0 ** (e - 7)
        return -val if s else val
    b = np.arange(256, dtype=np.uint8)
    got = oracle.e4m3_decode(b)
    exp = np.array([spec(int(v)) for v in b], np.float32)
    nan = np.isnan(exp)
    assert nan.sum() == 2 and np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), exp[~nan].view(np.uint32))
    # encode -> decode round trip of every representable value (the candle cast the test pins)
    assert np.array_equal(F.e4m3_encode(exp[~nan]) & 0x7F, b[~nan] & 0x7F)


def _f8(vals):
    return F.e4m3_encode(np.asarray(vals, np.float32))


def test_fp8_linear_matches_reference_dequant_path():
    # linear.rs:800-832: [2,1] scale broadcast + bias
    w = _f8([[1.0, -2.0, 3.0], [0.5, -0.25, 2.5]])
    scale = np.array([[0.5], [2.0]], np.float32)
    bias = np.array([0.1, -0.2], np.float32)
    x = np.array([[0.75, -1.0, 0.25], [1.5, 0.5, -0.5]], np.float32)
    out = oracle.linear(x, oracle.fp8_dequant(w, scale), bias)
    ref = x @ (np.array([[1.0, -2.0, 3.0], [0.5, -0.25, 2.5]], np.float32) * scale).T + bias
    assert np.abs(out - ref).max() < 1e-5


def test_fp8_rank1_and_scalar_scale_inv():
    # linear.rs:834-897
    w = _f8([[1.0, 2.0], [3.0, 4.0]])
    x = np.array([[1.0, -1.0], [0.5, 2.0]], np.float32)
    dq = oracle.fp8_dequant(w, np.array([0.5, 2.0], np.float32))
    assert np.array_equal(dq, np.array([[0.5, 1.0], [6.0, 8.0]], np.float32))
    assert np.abs(oracle.linear(x, dq) - x @ dq.T).max() < 1e-5
    w2 = _f8([[1.0, -2.0], [0.25, 4.0]])
    assert np.array_equal(oracle.fp8_dequant(w2, np.array([0.5], np.float32)),
                          np.array([[0.5, -1.0], [0.125, 2.0]], np.float32))
    assert np.array_equal(oracle.fp8_dequant(w2, np.float32(0.5)), np.array([[0.5, -1.0], [0.125, 2.0]], np.float32))


def test_fp8_rejects_invalid_rank1_scale_inv_shape():
    # linear.rs:899-914
    with pytest.raises(ValueError, match="invalid FP8 scale_inv shape"):
        oracle.fp8_dequant(_f8([[1.0, -2.0], [0.25, 4.0]]), np.array([0.5, 1.0, 2.0], np.float32))


def test_fp8_block_wise_scale_grid():
    # linear.rs:916-947 and weights.rs:620-657 (exact integers)
    w = _f8(np.arange(1, 17, dtype=np.float32).reshape(4, 4))
    dq = oracle.fp8_dequant(w, np.array([[0.5, 2.0], [4.0, 0.25]], np.float32))
    expanded = np.kron(np.array([[0.5, 2.0], [4.0, 0.25]], np.float32), np.ones((2, 2), np.float32))
    assert np.array_equal(dq, np.arange(1, 17, dtype=np.float32).reshape(4, 4) * expanded)
    out = oracle.linear(np.ones((1, 4), np.float32), dq)
    assert np.abs(out - dq.sum(axis=1)).max() < 1e-4
    dq2 = oracle.fp8_dequant(w, np.array([[10.0, 100.0], [1000.0, 10000.0]], np.float32))
    assert dq2.tolist() == [[10.0, 20.0, 300.0, 400.0], [50.0, 60.0, 700.0, 800.0],
                            [9000.0, 10000.0, 110000.0, 120000.0], [13000.0, 14000.0, 150000.0, 160000.0]]
    with pytest.raises(ValueError):
        oracle.fp8_dequant(w, np.ones((3, 2), np.float32))  # weights.rs:220-225


def test_mxfp4_dequantize_known_values():
    # mxfp4.rs:178-196
    data = [(2 * i) | ((2 * i + 1) << 4) for i in range(8)] + [0] * 8
    out = oracle.mxfp4_dequant(np.array(data, np.uint8), np.array([128], np.uint8), 1, 32)[0]
    exp = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)
    assert np.array_equal(out[:16], exp * 2.0)
    assert np.all(out[16:] == 0.0)
    assert np.isnan(oracle.mxfp4_dequant(np.full(16, 0x22, np.uint8), np.array([255], np.uint8), 1, 32)).all()


def test_mxfp4_linear_matches_manual_dot():
    # mxfp4.rs:198-214
    blocks = np.array([0x22] * 16 + [0x44] * 16, np.uint8)
    w = oracle.mxfp4_dequant(blocks, np.array([127, 126], np.uint8), 2, 32)
    y = oracle.linear(np.ones((1, 32), np.float32), w)
    assert y.tolist() == [[32.0, 32.0]]


def test_gpt_oss_expert_matches_scalar_reference():
    # moe.rs:704-788
    hidden = inter = 32
    limit = np.float32(7.0)
    gu_out, nb = 2 * inter, hidden // 32
    gu_blocks = np.array([(i * 23 + 7) & 0xFF for i in range(gu_out * nb * 16)], np.uint8)
    gu_scales = np.array([125 + (i % 5) for i in range(gu_out * nb)], np.uint8)
    dn_blocks = np.array([(i * 41 + 3) & 0xFF for i in range(hidden * nb * 16)], np.uint8)
    dn_scales = np.array([126 + (i % 3) for i in range(hidden * nb)], np.uint8)
    gu_bias = (np.sin(np.arange(gu_out, dtype=np.float32) * np.float32(0.7)) * 2.0).astype(np.float32)
    dn_bias = (np.cos(np.arange(hidden, dtype=np.float32) * np.float32(0.3)) * 0.5).astype(np.float32)
    x = (np.sin(np.arange(hidden, dtype=np.float32) * np.float32(0.21)) * 3.0).astype(np.float32)[None, :]
    w_gu = oracle.mxfp4_dequant(gu_blocks, gu_scales, gu_out, hidden)
    w_dn = oracle.mxfp4_dequant(dn_blocks, dn_scales, hidden, inter)
    y = oracle.gptoss_expert(x, w_gu, gu_bias, w_dn, dn_bias, float(limit))[0]
    # independent scalar reference
    gate_up = gu_bias + (w_gu.astype(np.float64) @ x[0].astype(np.float64)).astype(np.float32)
    gate = np.minimum(gate_up[0::2], limit)
    up = np.clip(gate_up[1::2], -limit, limit)
    glu = gate * (1.0 / (1.0 + np.exp(-gate * np.float32(1.702))))
    h = (up + 1.0) * glu
    expected = dn_bias + (w_dn.astype(np.float64) @ h.astype(np.float64)).astype(np.float32)
    tol = 1e-3 * np.abs(expected).max() + 1e-3
    assert np.abs(y - expected).max() < tol


def test_moe_route_and_dispatch_agree_with_dense_evaluation():
    # moe.rs:472-487 routing; moe.rs:793-817 naive == sparse (both are evaluations of the same sum)
    rng = np.random.default_rng(0xBEEF)
    t, e, k, hidden, inter = 6, 4, 2, 32, 32
    logits = rng.standard_normal((t, e)).astype(np.float32)
    idx, vals = oracle.moe_route(logits, k, True)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    assert np.array_equal(idx, order)
    top = np.take_along_axis(p, order, axis=1)
    assert np.allclose(vals, top / top.sum(axis=1, keepdims=True), atol=1e-6)
    assert np.allclose(vals.sum(axis=1), 1.0, atol=1e-6)
    gu_b, gu_s, dn_b, dn_s = [], [], [], []
    for _ in range(e):
        b, s = F.quantize_mxfp4(rng.standard_normal((2 * inter, hidden)).astype(np.float32) * 0.5)
        gu_b.append(b); gu_s.append(s)
        b, s = F.quantize_mxfp4(rng.standard_normal((hidden, inter)).astype(np.float32) * 0.5)
        dn_b.append(b); dn_s.append(s)
    gu_b, gu_s, dn_b, dn_s = (np.stack(a) for a in (gu_b, gu_s, dn_b, dn_s))
    gu_bias = rng.standard_normal((e, 2 * inter)).astype(np.float32) * 0.1
    dn_bias = rng.standard_normal((e, hidden)).astype(np.float32) * 0.1
    x = rng.standard_normal((t, hidden)).astype(np.float32)
    sparse = oracle.gptoss_moe(x, idx, vals, gu_b, gu_s, gu_bias, dn_b, dn_s, dn_bias, hidden, inter)
    naive = np.zeros_like(sparse)
    for ex in range(e):
        w_gu = oracle.mxfp4_dequant(gu_b[ex], gu_s[ex], 2 * inter, hidden)
        w_dn = oracle.mxfp4_dequant(dn_b[ex], dn_s[ex], hidden, inter)
        full = oracle.gptoss_expert(x, w_gu, gu_bias[ex], w_dn, dn_bias[ex])
        wt = np.where(idx == ex, vals, 0.0).sum(axis=1, keepdims=True).astype(np.float32)
        naive += full * wt
    assert np.abs(naive - sparse).max() < 1e-5 * max(1.0, np.abs(sparse).max())
    # expert-range partition sums to the whole (the property expert parallelism relies on)
    lo = oracle.gptoss_moe(x, idx, vals, gu_b, gu_s, gu_bias, dn_b, dn_s, dn_bias, hidden, inter, expert_range=(0, 2))
    hi = oracle.gptoss_moe(x, idx, vals, gu_b, gu_s, gu_bias, dn_b, dn_s, dn_bias, hidden, inter, expert_range=(2, 4))
    assert np.abs((lo + hi) - sparse).max() < 1e-5 * max(1.0, np.abs(sparse).max())


def test_w8a16_dequant_known_answer():
    """8-bit AWQ layout (quant_kernels.metal:1-16,40-48): byte c of word j is out column 4 j + c, W = (q - z) * s."""
    k, n, g = 4, 8, 2
    iw = (np.arange(k * n, dtype=np.uint32).reshape(k, n) * 7 + 3) % 256
    iz = np.array([[1, 2, 3, 4, 5, 6, 7, 8], [250, 128, 0, 9, 10, 11, 12, 13]], np.uint32)
    sc = np.array([[0.5, 0.25, 1.0, 2.0, 0.125, 1.5, 0.75, 3.0], [1.0, 0.5, 2.0, 4.0, 0.25, 3.0, 1.5, 6.0]], np.float16)
    qw, qz = F.pack_w8a16(iw), F.pack_w8a16(iz)
    assert qw.shape == (k, n // 4) and int(qw[0, 0]) == (3 | (10 << 8) | (17 << 16) | (24 << 24))
    got = oracle.w8a16_dequant(qw, qz, sc)
    want = np.empty((n, k), np.float32)
    for o in range(n):
        for i in range(k):
            want[o, i] = (float(int(iw[i, o]) - int(iz[i // g, o]))) * float(sc[i // g, o])
    assert np.array_equal(got, want)

"""Parity of the CUDA kernels (through the C ABI) against the CPU oracle.

Dequantization is bit-exact. Matmul outputs are compared with the oracle's f32
``x @ deq(W)^T`` under  max|err| <= 2e-2 * ||row||_inf  (bf16 activations, f32
accumulation, bf16 output rounding) plus the reference tests' own looser bound
``0.06 * max|ref| + 1e-2`` (metal_ops.rs:3713-3716) as a sanity ceiling.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from oxydllm_b200 import formats as F
from oxydllm_b200 import linear as L
from oxydllm_b200 import synth

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gguf_blocks.npz")
TORCH_OUT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def words(a):
    return dev(a.view(np.int32))


def narrowed(ref_f32: np.ndarray, kind: str) -> np.ndarray:
    """The oracle's f32 result narrowed once (RNE), as bit patterns."""
    if kind == "f32":
        return ref_f32.view(np.uint32)
    if kind == "bf16":
        return oracle.to_bf16_bits(ref_f32)
    return oracle.to_f16_bits(ref_f32)


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float32:
        return t.cpu().numpy().view(np.uint32)
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def assert_matmul_close(y: torch.Tensor, ref: np.ndarray, label=""):
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all(), f"{label}: non-finite output"
    err = np.abs(got - ref)
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (err <= 2e-2 * row_inf + 1e-6).all(), f"{label}: max err {err.max()} vs row_inf {row_inf.max()}"
    assert err.max() < 0.06 * np.abs(ref).max() + 1e-2


# ------------------------------------------------------------------ dequant
@pytest.mark.parametrize("k,n,g", [(8, 16, 4), (4, 8, 2), (256, 128, 64), (512, 256, 128), (96, 200, 32)])
@pytest.mark.parametrize("out", ["f32", "bf16", "f16"])
def test_awq_dequant_bit_exact(cuda, k, n, g, out):
    qw, qz, sc = synth.awq_layer(k, n, g, seed=k + n)
    ref = oracle.awq_dequant(qw, qz, sc)
    raw = L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc))
    got = L.dequantize_awq(raw, TORCH_OUT[out])
    assert got.shape == (n, k)
    assert np.array_equal(bits(got), narrowed(ref, out))


def test_awq_dequant_reference_golden_case(cuda):
    # awq.rs:953-1011 inputs, f32 scales
    k, n, g = 8, 16, 4
    iw = np.array([[(i * 3 + j * 5 + 1) & 0xF for j in range(n)] for i in range(k)], np.uint8)
    iz = np.array([[(gi * 7 + j) & 0xF for j in range(n)] for gi in range(k // g)], np.uint8)
    sc = np.array([[np.float32(0.01) * np.float32(gi + 1) + np.float32(0.001) * np.float32(j + 1) for j in range(n)]
                   for gi in range(k // g)], np.float32)
    raw = L.QuantWeight.new_awq(4, words(F.pack_awq(iw)), words(F.pack_awq(iz)), dev(sc))
    got = L.dequantize_awq(raw).cpu().numpy()
    exp = ((iw.astype(np.int32) - np.repeat(iz, g, axis=0).astype(np.int32)).astype(np.float32) * np.repeat(sc, g, axis=0)).T
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("bits_,sym", [(4, False), (8, False), (4, True)])
def test_gptq_dequant_bit_exact(cuda, bits_, sym):
    rng = np.random.default_rng(bits_)
    k, n, g = 128, 64, 32
    iw = rng.integers(0, 1 << bits_, size=(k, n), dtype=np.uint32)
    iz = rng.integers(0, 1 << bits_, size=(k // g, n), dtype=np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n))) * 0.01 + 1e-3).astype(np.float16)
    qw, qz = F.pack_gptq_qweight(iw, bits_), F.pack_gptq_qzeros(iz, bits_)
    ref = oracle.gptq_dequant(qw, None if sym else qz, sc, bits_, sym)
    raw = L.QuantWeight.new_gptq(bits_, sym, words(qw), None if sym else words(qz), dev(sc))
    for out in ("f32", "bf16"):
        assert np.array_equal(bits(L.dequantize_gptq(raw, TORCH_OUT[out])), narrowed(ref, out))


@pytest.mark.parametrize("ggml_type", [F.GGML_Q4_0, F.GGML_Q8_0, F.GGML_Q4_K, F.GGML_Q6_K, F.GGML_Q4_1, F.GGML_Q5_0, F.GGML_Q5_1, F.GGML_Q5_K,
                                       F.GGML_Q2_K, F.GGML_Q3_K])
def test_gguf_dequant_bit_exact_golden_and_oracle(cuda, ggml_type):
    z = np.load(GOLDEN)
    rows, cols = (int(v) for v in z[f"shape_{ggml_type}"])
    lin = L.QLinear(ggml_type, dev(z[f"blocks_{ggml_type}"]), rows, cols)
    got = lin.dequantize(torch.float32)
    assert np.array_equal(bits(got), z[f"deq_{ggml_type}"].view(np.uint32))  # gguf-py fixture
    ref = oracle.gguf_dequant(ggml_type, z[f"blocks_{ggml_type}"], rows, cols)
    assert np.array_equal(bits(lin.dequantize(torch.bfloat16)), oracle.to_bf16_bits(ref))
    # a larger encoded matrix
    data = synth.gguf_layer(ggml_type, 96, 1024, seed=7)
    lin = L.QLinear(ggml_type, dev(data), 96, 1024)
    assert np.array_equal(bits(lin.dequantize()), oracle.gguf_dequant(ggml_type, data, 96, 1024).view(np.uint32))


def test_fp8_dequant_bit_exact(cuda):
    # every byte, F8 chain of metal_ops.rs:4310-4371: 8 x 256 bytes (37 i + 11), 2 x 2 grid
    w = np.array([(37 * i + 11) & 0xFF for i in range(8 * 256)], np.uint8).reshape(8, 256)
    w[(w & 0x7F) == 0x7F] = 0x3C  # no NaN encodings
    scale = np.array([[0.5, 1.25], [3.0, 0.0625]], np.float32)
    lin = L.Fp8Linear(dev(w), dev(scale))
    for out in ("f32", "bf16", "f16"):
        assert np.array_equal(bits(lin.dequantize(TORCH_OUT[out])), narrowed(oracle.fp8_dequant(w, scale), out))
    allb = np.arange(256, dtype=np.uint8).reshape(4, 64)
    got = L.Fp8Linear(dev(allb)).dequantize().cpu().numpy()
    ref = oracle.e4m3_decode(allb)
    ok = ~np.isnan(ref)
    assert np.array_equal(np.isnan(got), ~ok) and np.array_equal(got[ok].view(np.uint32), ref[ok].view(np.uint32))
    # block grid on quantized gaussian weights + per-row and scalar scales
    q, s = synth.fp8_layer(256, 384, seed=3)
    assert np.array_equal(bits(L.Fp8Linear(dev(q), dev(s)).dequantize()), oracle.fp8_dequant(q, s).view(np.uint32))
    srow = np.linspace(0.5, 2.0, 256).astype(np.float32)
    assert np.array_equal(bits(L.Fp8Linear(dev(q), dev(srow)).dequantize()), oracle.fp8_dequant(q, srow).view(np.uint32))
    assert np.array_equal(bits(L.Fp8Linear(dev(q), dev(np.float32(0.3))).dequantize()),
                          oracle.fp8_dequant(q, np.float32(0.3)).view(np.uint32))


def test_mxfp4_dequant_bit_exact(cuda):
    rng = np.random.default_rng(0)
    blocks = rng.integers(0, 256, size=(10, 4, 16), dtype=np.uint8)
    scales = rng.integers(0, 255, size=(10, 4), dtype=np.uint8)  # 0 (2^-127) included, NaN code excluded
    scales[0, 0] = 0
    scales[1, 1] = 254
    lin = L.Mxfp4Linear(dev(blocks), dev(scales), None, 128, 10)
    ref = oracle.mxfp4_dequant(blocks, scales, 10, 128)
    assert np.array_equal(bits(lin.dequantize()), ref.view(np.uint32))
    assert np.array_equal(bits(lin.dequantize(torch.bfloat16)), oracle.to_bf16_bits(ref))
    # reference known-answer vector (mxfp4.rs:178-196) and NaN scale
    data = np.array([(2 * i) | ((2 * i + 1) << 4) for i in range(8)] + [0] * 8, np.uint8)
    got = L.Mxfp4Linear(dev(data), dev(np.array([128], np.uint8)), None, 32, 1).dequantize().cpu().numpy()[0]
    assert got[:16].tolist() == [0.0, 1.0, 2.0, 3.0, 4.0, 6.0, 8.0, 12.0, -0.0, -1.0, -2.0, -3.0, -4.0, -6.0, -8.0, -12.0]
    nan = L.Mxfp4Linear(dev(data), dev(np.array([255], np.uint8)), None, 32, 1).dequantize().cpu().numpy()
    assert np.isnan(nan).all()


# --------------------------------------------------------------------- GEMV
def _awq_ref_case(k, n, g):
    # weights/zeros/scales/x patterns of the reference's Metal parity tests (metal_ops.rs:3660-3720)
    iw = np.array([[(5 * i + 3 * j + 1) & 0xF for j in range(n)] for i in range(k)], np.uint8)
    iz = np.array([[(7 * gi + j + 2) & 0xF for j in range(n)] for gi in range(k // g)], np.uint8)
    sc = np.array([[0.01 + 0.003 * ((gi + j) % 5) for j in range(n)] for gi in range(k // g)], np.float32)
    return F.pack_awq(iw), F.pack_awq(iz), sc


@pytest.mark.parametrize("k,n,g", [(256, 128, 64), (512, 256, 128), (256, 256, 64), (3072, 128, 64)])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 12, 20, 32])
def test_awq_gemv_reference_patterns(cuda, k, n, g, m):
    qw, qz, sc = _awq_ref_case(k, n, g)
    sc16 = sc.astype(np.float16)
    x = synth.bf16_round(np.array([((i % 17) - 8) * 0.03 for i in range(m * k)], np.float32).reshape(m, k))
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc16))
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc16)))
    y = lin.forward(dev(x, torch.bfloat16))
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    assert_matmul_close(y, ref, f"awq k={k} n={n} g={g} m={m}")


@pytest.mark.parametrize("m", [1, 7, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("k,n,g,scale_dtype", [(1024, 2048, 128, "f16"), (4096, 1792, 128, "f16"),
                                               (512, 1000 * 8 // 8, 32, "bf16"), (2048, 72, 64, "f32")])
def test_awq_gemv_random(cuda, m, k, n, g, scale_dtype):
    qw, qz, sc = synth.awq_layer(k, n, g, seed=m)
    x = synth.activations(m, k, seed=m + 100)
    bias = synth.bf16_round(np.random.default_rng(9).standard_normal(n).astype(np.float32))
    if scale_dtype == "bf16":
        sc_np = synth.bf16_round(sc.astype(np.float32))
        sc_t = dev(sc_np, torch.bfloat16)
    elif scale_dtype == "f32":
        sc_np = sc.astype(np.float32)
        sc_t = dev(sc_np)
    else:
        sc_np, sc_t = sc, dev(sc)
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc_np), bias)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), sc_t), dev(bias, torch.bfloat16))
    y = lin.forward(dev(x, torch.bfloat16))
    assert_matmul_close(y, ref, f"awq random m={m} k={k} n={n}")


def test_awq_gemv_leading_dims_and_determinism(cuda):
    k, n, g = 3072, 128, 64  # metal_ops.rs:4562-4625: same bits over 48 runs
    qw, qz, sc = synth.awq_layer(k, n, g, seed=5)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    x = dev(synth.activations(6, k, seed=2), torch.bfloat16)
    y0 = lin.forward(x.reshape(2, 3, k))
    assert y0.shape == (2, 3, n)
    for _ in range(47):
        assert torch.equal(lin.forward(x.reshape(2, 3, k)), y0)
    y1 = lin.forward(x[:1])
    assert torch.equal(y1[0], y0.reshape(6, n)[0])  # batch-size invariant summation order per row


@pytest.mark.parametrize("m", [1, 5, 8])
def test_awq_gemv_dependent_launches_back_to_back(cuda, m):
    # The decode kernel lets the next launch on the stream start early and orders itself behind the
    # previous one before it reads x: a chain y -> x of launches without host synchronisation (eager and
    # replayed from a CUDA graph) must give the bits of the same chain with a synchronisation per step.
    from oxydllm_b200 import _lib
    k = n = 2048
    layers = []
    for seed in range(5):
        qw, qz, sc = synth.awq_layer(k, n, 128, seed=40 + seed)
        layers.append(L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc))))
    x0 = dev(synth.activations(m, k, seed=3), torch.bfloat16)

    def chain(sync):
        x = x0
        for lin in layers:
            x = lin.forward(x)
            if sync:
                torch.cuda.synchronize()
        return x

    want = chain(True)
    assert torch.isfinite(want.float()).all()
    for _ in range(3):
        assert torch.equal(chain(False), want)
    bufs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in layers]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        def run():
            x = x0
            for lin, y in zip(layers, bufs):
                lin._gemv(x, y, m)
                x = y
        run()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        for _ in range(3):
            bufs[-1].zero_()
            graph.replay()
            stream.synchronize()
            assert torch.equal(bufs[-1], want)
    torch.cuda.current_stream().wait_stream(stream)
    assert _lib.load().oxq_awq_gemv_check(None) == 0


def test_awq_prefill_sized_batch_matches_oracle(cuda):
    k, n, g, m = 512, 256, 128, 70
    qw, qz, sc = synth.awq_layer(k, n, g, seed=11)
    x = synth.activations(m, k, seed=12)
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc))
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    assert_matmul_close(lin.forward(dev(x, torch.bfloat16)), ref, "awq m=70")


@pytest.mark.parametrize("ggml_type", [F.GGML_Q4_0, F.GGML_Q8_0, F.GGML_Q4_K, F.GGML_Q6_K, F.GGML_Q4_1, F.GGML_Q5_0, F.GGML_Q5_1, F.GGML_Q5_K,
                                       F.GGML_Q2_K, F.GGML_Q3_K])
@pytest.mark.parametrize("n,k,m", [(128, 256, 1), (100, 2560, 2), (256, 512, 4), (1001, 512, 8), (64, 4096, 1),
                                   (512, 2048, 9), (96, 1024, 32)])
def test_gguf_gemv(cuda, ggml_type, n, k, m):
    # shapes from metal_ops.rs:6386-6617 (odd n = 1001, 100; m across the 8-row boundary)
    w = np.array([((i % 23) - 11) * 0.04 for i in range(n * k)], np.float32).reshape(n, k)
    data = F.GGML_QUANTIZE[ggml_type](w)
    x = synth.activations(m, k, seed=n + m)
    ref = oracle.linear(x, oracle.gguf_dequant(ggml_type, data, n, k))
    lin = L.QLinear(ggml_type, dev(data), n, k)
    y = lin.forward(dev(x, torch.bfloat16))
    assert y.shape == (m, n)
    assert_matmul_close(y, ref, f"gguf type={ggml_type} n={n} k={k} m={m}")


def test_gguf_q4k_config0_shape_and_bias(cuda):
    n = k = 4096
    data = synth.gguf_layer(F.GGML_Q4_K, n, k, seed=0)
    x = synth.activations(1, k, seed=1)
    bias = synth.bf16_round(np.random.default_rng(3).standard_normal(n).astype(np.float32) * 0.1)
    ref = oracle.linear(x, oracle.gguf_dequant(F.GGML_Q4_K, data, n, k), bias)
    lin = L.QLinear(F.GGML_Q4_K, dev(data), n, k, dev(bias, torch.bfloat16))
    assert_matmul_close(lin.forward(dev(x, torch.bfloat16)), ref, "C0")
    lin32 = L.QLinear(F.GGML_Q4_K, dev(data), n, k, out_dtype=torch.float32)
    y32 = lin32.forward(dev(x, torch.bfloat16))
    assert y32.dtype == torch.float32
    ref32 = oracle.linear(x, oracle.gguf_dequant(F.GGML_Q4_K, data, n, k))
    assert np.abs(y32.cpu().numpy() - ref32).max() <= 5e-3 * np.abs(ref32).max()  # f32 out: tighter


@pytest.mark.parametrize("n,k,grid,m", [(512, 2048, (4, 16), 1), (2048, 512, (16, 4), 1), (512, 2048, (4, 16), 4),
                                        (96, 160, (3, 5), 2), (256, 1024, (2, 8), 32), (1792, 4096, (14, 32), 16)])
def test_fp8_gemv(cuda, n, k, grid, m):
    # shapes of metal_ops.rs:4373-4452; tolerance there: < 0.02 * max(1, max|ref|)
    rng = np.random.default_rng(n + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    bo, bi = n // grid[0], k // grid[1]
    t = w.reshape(grid[0], bo, grid[1], bi)
    scale = (np.abs(t).max(axis=(1, 3)) / 448.0).astype(np.float32)
    q = F.e4m3_encode(t / scale[:, None, :, None]).reshape(n, k)
    x = synth.activations(m, k, seed=5)
    ref = oracle.linear(x, oracle.fp8_dequant(q, scale))
    y = L.Fp8Linear(dev(q), dev(scale)).forward(dev(x, torch.bfloat16))
    assert_matmul_close(y, ref, f"fp8 n={n} k={k} m={m}")
    assert np.abs(y.float().cpu().numpy() - ref).max() < 0.02 * max(1.0, np.abs(ref).max())


def test_fp8_gemv_scale_variants_and_bias(cuda):
    n, k, m = 128, 256, 3
    q, _ = synth.fp8_layer(n, k, seed=1)
    x = synth.activations(m, k, seed=2)
    bias = synth.bf16_round(np.linspace(-1, 1, n).astype(np.float32))
    for s in (None, np.float32(0.01), np.linspace(0.005, 0.02, n).astype(np.float32)):
        ref = oracle.linear(x, oracle.fp8_dequant(q, s), bias)
        y = L.Fp8Linear(dev(q), None if s is None else dev(np.asarray(s)), dev(bias, torch.bfloat16)).forward(
            dev(x, torch.bfloat16))
        assert_matmul_close(y, ref, "fp8 scale variant")


@pytest.mark.parametrize("n,k,m", [(10, 64, 1), (10, 64, 4), (10, 64, 8), (10, 64, 32), (2880, 2880, 5), (5760, 2880, 1)])
def test_mxfp4_gemv(cuda, n, k, m):
    # N=10, K=64 from metal_ops.rs:6621-6670; 2880 = GPT-OSS hidden (90 blocks: not a multiple of 128)
    b, s = synth.mxfp4_layer(n, k, seed=n)
    bias = synth.bf16_round(np.random.default_rng(1).standard_normal(n).astype(np.float32) * 0.02)
    x = synth.activations(m, k, seed=3)
    ref = oracle.linear(x, oracle.mxfp4_dequant(b, s, n, k), bias)
    y = L.Mxfp4Linear(dev(b), dev(s), dev(bias, torch.bfloat16), k, n).forward(dev(x, torch.bfloat16))
    assert_matmul_close(y, ref, f"mxfp4 n={n} k={k} m={m}")


def test_mxfp4_manual_dot(cuda):
    # mxfp4.rs:198-214
    blocks = np.array([0x22] * 16 + [0x44] * 16, np.uint8)
    lin = L.Mxfp4Linear(dev(blocks), dev(np.array([127, 126], np.uint8)), None, 32, 2)
    y = lin.forward(torch.ones((1, 32), dtype=torch.bfloat16, device="cuda"))
    assert y.float().cpu().tolist() == [[32.0, 32.0]]


def test_full_size_config1_linearity(cuda):
    """Full C1 shape: y(x1 + x2) == y(x1) + y(x2) up to rounding, and a row subset against the oracle."""
    k, n, g = 4096, 14336, 128
    qw, qz, sc = synth.awq_layer(k, n, g, seed=0)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    x1 = synth.activations(4, k, seed=1)
    x2 = synth.bf16_round(x1 * 2.0)  # exact in bf16
    y1 = lin.forward(dev(x1, torch.bfloat16)).float()
    y2 = lin.forward(dev(x2, torch.bfloat16)).float()
    assert torch.allclose(y2, 2.0 * y1, rtol=2 ** -7, atol=1e-6)
    cols = slice(4096, 4096 + 512)
    ref = oracle.linear(x1, oracle.awq_dequant(qw[:, 512:576], qz[:, 512:576], sc[:, cols]))
    assert_matmul_close(y1[:, cols], ref, "C1 column slice")


# ------------------------------------------------- edge cases of the tuned kernels
@pytest.mark.parametrize("k,n,g", [(192, 264, 32), (384, 40, 64), (128, 1032, 128), (1040, 96, 16)])
def test_awq_slab_producer_ragged_shapes_bit_exact(cuda, k, n, g):
    # bf16 output takes the tensor-core path's producer: k not a multiple of its 128-row tile, a word
    # count that is not a multiple of 4 (no 16-byte loads) or of the 32-word tile
    qw, qz, sc = synth.awq_layer(k, n, g, seed=k + n)
    raw = L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc))
    ref = oracle.awq_dequant(qw, qz, sc)
    assert np.array_equal(bits(L.dequantize_awq(raw, torch.bfloat16)), oracle.to_bf16_bits(ref))


def test_mxfp4_slab_producer_extreme_scales_bit_exact(cuda):
    rng = np.random.default_rng(5)
    sc_list = [0, 1, 2, 3, 4, 5, 127, 249, 250, 251, 252, 253, 254]
    blocks = rng.integers(0, 256, size=(len(sc_list), 2, 16), dtype=np.uint8)
    scales = np.repeat(np.array(sc_list, np.uint8)[:, None], 2, axis=1)
    lin = L.Mxfp4Linear(dev(blocks), dev(scales), None, 64, len(sc_list))
    ref = oracle.mxfp4_dequant(blocks, scales, len(sc_list), 64)
    assert np.array_equal(bits(lin.dequantize(torch.bfloat16)), oracle.to_bf16_bits(ref))


def test_fp8_slab_producer_nan_bytes(cuda):
    allb = np.tile(np.arange(256, dtype=np.uint8), 4).reshape(4, 256)
    scale = np.array([[0.75, 2.0]], np.float32)
    got = L.Fp8Linear(dev(allb), dev(scale)).dequantize(torch.bfloat16)
    ref = oracle.fp8_dequant(allb, scale)
    ok = ~np.isnan(ref)
    g = got.float().cpu().numpy()
    assert np.array_equal(np.isnan(g), ~ok)
    assert np.array_equal(bits(got)[ok], oracle.to_bf16_bits(ref)[ok])


@pytest.mark.parametrize("m", [9, 17, 24, 32])
def test_fp8_gemv_tuned_kernel_many_tokens(cuda, m):
    n, k = 200, 1024  # a ragged last row tile
    q, s = synth.fp8_layer(256, k, seed=m)
    q = np.ascontiguousarray(q[:n])
    srow = np.ascontiguousarray(np.repeat(s, 128, axis=0)[:n])  # one scale per (row, 128-wide k block)
    x = synth.activations(m, k, seed=3)
    bias = synth.bf16_round(np.linspace(-0.5, 0.5, n).astype(np.float32))
    y = L.Fp8Linear(dev(q), dev(srow), dev(bias, torch.bfloat16)).forward(dev(x, torch.bfloat16))
    assert_matmul_close(y, oracle.linear(x, oracle.fp8_dequant(q, srow), bias), f"fp8 tuned m={m}")


@pytest.mark.parametrize("n,k,m", [(72, 512, 11), (40, 768, 3), (16, 256, 16)])
def test_q4k_gemv_tuned_kernel_ragged(cuda, n, k, m):
    data = synth.gguf_layer(F.GGML_Q4_K, n, k, seed=n + m)
    x = synth.activations(m, k, seed=9)
    ref = oracle.linear(x, oracle.gguf_dequant(F.GGML_Q4_K, data, n, k))
    y = L.QLinear(F.GGML_Q4_K, dev(data), n, k).forward(dev(x, torch.bfloat16))
    assert_matmul_close(y, ref, f"q4k n={n} k={k} m={m}")


@pytest.mark.parametrize("k,n,g,sym", [(320, 72, 40, False), (512, 200, 128, True), (2048, 96, 64, False)])
def test_gptq4_slab_producer_ragged_shapes_bit_exact(cuda, k, n, g, sym):
    # bf16 output takes the transposing 4-bit producer: word rows and columns that do not fill its 32 x 32 tile
    rng = np.random.default_rng(k + n)
    iw = rng.integers(0, 16, size=(k, n), dtype=np.uint32)
    iz = rng.integers(0, 16, size=(k // g, n), dtype=np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n))) * 0.01 + 1e-3).astype(np.float16)
    qw, qz = F.pack_gptq_qweight(iw, 4), F.pack_gptq_qzeros(iz, 4)
    ref = oracle.gptq_dequant(qw, None if sym else qz, sc, 4, sym)
    raw = L.QuantWeight.new_gptq(4, sym, words(qw), None if sym else words(qz), dev(sc))
    assert np.array_equal(bits(L.dequantize_gptq(raw, torch.bfloat16)), oracle.to_bf16_bits(ref))

"""The fused unpack + tcgen05 AWQ matmul (batches of 17..256 tokens through ``oxq_awq_gemm``).

The kernel builds the bf16 weight tile in shared memory; with one-hot activations an output row is a
row of that tile, so the in-kernel dequantization and the operand layout are checked bit for bit against
the oracle's dequantized weight rounded to bf16 (what the dequantization kernel writes, awq.rs:360-367).
General inputs are checked under the matmul tolerance of the other parity tests.
"""
import numpy as np
import pytest
import torch

import oracle
from oxydllm_b200 import gemm, synth
from oxydllm_b200 import linear as L

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dtype) if dtype is not None else t).cuda()


def layer(k, n, g, seed, scale_dtype="f16", bias=False):
    qw, qz, sc = synth.awq_layer(k, n, g, seed=seed)
    if scale_dtype == "bf16":
        sc_np = synth.bf16_round(sc.astype(np.float32))
        sc_t = dev(sc_np, torch.bfloat16)
    else:
        sc_np, sc_t = sc, dev(sc)
    b = synth.bf16_round(np.random.default_rng(seed).standard_normal(n).astype(np.float32)) if bias else None
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, dev(qw.view(np.int32)), dev(qz.view(np.int32)), sc_t),
                              dev(b, torch.bfloat16) if bias else None)
    return lin, oracle.awq_dequant(qw, qz, sc_np), b


def close(y, ref):
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - ref)
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (err <= 2e-2 * row_inf + 1e-6).all(), f"max err {err.max()} vs row_inf {row_inf.max()}"


@pytest.mark.parametrize("scale_dtype", ["f16", "bf16"])
@pytest.mark.parametrize("k,n,g", [(256, 128, 64), (512, 384, 128), (1024, 256, 256)])
def test_fused_weight_tile_bit_exact_with_one_hot_rows(cuda, k, n, g, scale_dtype):
    lin, w, _ = layer(k, n, g, seed=k + n, scale_dtype=scale_dtype)
    assert lin.gemv_max_m() == 8  # narrow layers of these shapes take the fused kernel (with k splits) from 9 tokens on
    want = oracle.to_bf16_bits(w)  # [n, k]
    for k0 in range(0, k, 256):
        m = min(256, k - k0)
        x = np.zeros((m, k), np.float32)
        x[np.arange(m), k0 + np.arange(m)] = 1.0
        y = lin.forward(dev(x, torch.bfloat16))
        got = y.cpu().view(torch.int16).numpy().view(np.uint16)  # [m, n]: row i is input row k0 + i of the weight
        assert np.array_equal(got, want[:, k0:k0 + m].T)
    gemm.check(gemm.workspace(n, k, "cuda"))


@pytest.mark.parametrize("m", [17, 32, 33, 64, 100, 128, 255, 256])
@pytest.mark.parametrize("k,n,g,scale_dtype,bias", [(512, 256, 128, "f16", True), (2048, 1152, 128, "bf16", False),
                                                   (1024, 128, 512, "f16", False)])
def test_fused_matmul_matches_oracle(cuda, m, k, n, g, scale_dtype, bias):
    lin, w, b = layer(k, n, g, seed=m + n, scale_dtype=scale_dtype, bias=bias)
    x = synth.activations(m, k, seed=m)
    ref = oracle.linear(x, synth.bf16_round(w), b)
    y = lin.forward(dev(x, torch.bfloat16))
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    close(y, ref)
    assert torch.equal(lin.forward(dev(x, torch.bfloat16)), y)  # same bits on the same workspace
    gemm.check(gemm.workspace(n, k, "cuda"))


@pytest.mark.parametrize("m", [32, 64, 256])
def test_fused_matmul_benchmark_layer(cuda, m):
    k, n, g = 4096, 14336, 128
    lin, w, _ = layer(k, n, g, seed=7)
    x = synth.activations(m, k, seed=m)
    y = lin.forward(dev(x, torch.bfloat16))
    rows = [0, m // 2, m - 1]
    ref = oracle.linear(x[rows], synth.bf16_round(w))
    close(y[rows], ref)
    y32 = torch.empty((m, n), dtype=torch.float32, device="cuda")  # f32 output through the entry point itself
    gemm.awq_matmul(lin, dev(x, torch.bfloat16), y32)
    close(y32[rows], ref)
    gemm.check(gemm.workspace(n, k, "cuda"))


def test_shapes_outside_the_fused_kernel_keep_their_paths(cuda):
    # out_features not a multiple of 128 and f32 scales: the GEMV up to 32 tokens, the slab GEMM above
    lin, w, _ = layer(512, 200, 128, seed=3)
    assert lin.gemv_max_m() == L.GEMV_MAX_M
    for m in (20, 40):
        x = synth.activations(m, 512, seed=m)
        close(lin.forward(dev(x, torch.bfloat16)), oracle.linear(x, synth.bf16_round(w)))


# ------------------------------------------------------------------ GPTQ 4-bit through the same kernel (K-major operand)
def gptq_layer(k, n, g, seed, sym=False, scale_dtype="f16"):
    rng = np.random.default_rng(seed)
    qw = rng.integers(0, 2**32, size=(k // 8, n), dtype=np.uint64).astype(np.uint32)
    qz = None if sym else rng.integers(0, 2**32, size=(k // g, n // 8), dtype=np.uint64).astype(np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n)) * 0.02) / 7 + 1e-4).astype(np.float16)
    if scale_dtype == "bf16":
        sc_np = synth.bf16_round(sc.astype(np.float32))
        sc_t = dev(sc_np, torch.bfloat16)
    else:
        sc_np, sc_t = sc, dev(sc)
    raw = L.QuantWeight.new_gptq(4, sym, dev(qw.view(np.int32)), None if sym else dev(qz.view(np.int32)), sc_t)
    return L.PackedQuantLinear(raw), oracle.gptq_dequant(qw, qz, sc_np, 4, sym)


@pytest.mark.parametrize("k,n,g,sym,scale_dtype", [(256, 128, 64, False, "f16"), (512, 384, 128, True, "f16"),
                                                  (1024, 256, 256, False, "bf16")])
def test_gptq_fused_weight_tile_bit_exact_with_one_hot_rows(cuda, k, n, g, sym, scale_dtype):
    lin, w = gptq_layer(k, n, g, seed=k + n, sym=sym, scale_dtype=scale_dtype)
    assert lin.gemv_max_m() == L.GPTQ_FUSED_MIN_M - 1
    want = oracle.to_bf16_bits(w)
    for k0 in range(0, k, 256):
        m = min(256, k - k0)
        x = np.zeros((m, k), np.float32)
        x[np.arange(m), k0 + np.arange(m)] = 1.0
        y = lin.forward(dev(x, torch.bfloat16))
        got = y.cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got, want[:, k0:k0 + m].T)
    gemm.check(gemm.workspace(n, k, "cuda"))


@pytest.mark.parametrize("m", [3, 8, 17, 64, 200, 256])
@pytest.mark.parametrize("k,n,g,sym", [(512, 256, 128, False), (2048, 640, 64, True), (4096, 1792, 128, False)])
def test_gptq_fused_matmul_matches_oracle(cuda, m, k, n, g, sym):
    lin, w = gptq_layer(k, n, g, seed=m + n, sym=sym)
    x = synth.activations(m, k, seed=m)
    y = lin.forward(dev(x, torch.bfloat16))
    close(y, oracle.linear(x, synth.bf16_round(w)))
    gemm.check(gemm.workspace(n, k, "cuda"))


# ------------------------------------------------------------------ FP8 E4M3 block-scaled through the same kernel
@pytest.mark.parametrize("k,n,block", [(256, 128, 128), (1024, 384, 128), (512, 256, None)])
def test_fp8_fused_weight_tile_bit_exact_with_one_hot_rows(cuda, k, n, block):
    w8, sinv = synth.fp8_layer(n, k, seed=k + n)
    if block is None:
        sinv = None  # unscaled weight
    lin = L.Fp8Linear(dev(w8), None if sinv is None else dev(sinv))
    want = oracle.to_bf16_bits(oracle.fp8_dequant(w8, sinv)).copy()
    want[want == 0x8000] = 0  # a -0 weight leaves the sum of +0 products at +0
    for k0 in range(0, k, 256):
        m = min(256, k - k0)
        x = np.zeros((m, k), np.float32)
        x[np.arange(m), k0 + np.arange(m)] = 1.0
        y = lin.forward(dev(x, torch.bfloat16))
        got = y.cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got, want[:, k0:k0 + m].T)
    gemm.check(gemm.workspace(n, k, "cuda"))


@pytest.mark.parametrize("m", [17, 32, 64, 130, 256])
@pytest.mark.parametrize("k,n,bias", [(512, 256, True), (2048, 640, False), (4096, 1792, False)])
def test_fp8_fused_matmul_matches_oracle(cuda, m, k, n, bias):
    w8, sinv = synth.fp8_layer(n, k, seed=m + n)
    b = synth.bf16_round(np.random.default_rng(m).standard_normal(n).astype(np.float32)) if bias else None
    lin = L.Fp8Linear(dev(w8), dev(sinv), dev(b, torch.bfloat16) if bias else None)
    s, s_out, s_in = lin._grid()
    assert lin.gemv_max_m(s_out, s_in) == L.AWQ_FUSED_MIN_M - 1
    x = synth.activations(m, k, seed=m)
    y = lin.forward(dev(x, torch.bfloat16))
    close(y, oracle.linear(x, synth.bf16_round(oracle.fp8_dequant(w8, sinv)), b))
    gemm.check(gemm.workspace(n, k, "cuda"))


# ------------------------------------------------------------------ narrow layers: k split over grid y, ticketed reduction
@pytest.mark.parametrize("m,k,n,g,bias", [(9, 4096, 4096, 128, True), (64, 14336, 4096, 128, False), (17, 1024, 128, 128, False),
                                          (200, 2048, 1024, 64, True), (256, 4096, 1024, 128, False), (40, 1024, 8064, 128, False)])
def test_fused_split_k_matches_oracle_and_is_reproducible(cuda, m, k, n, g, bias):
    lin, w, b = layer(k, n, g, seed=m + n, bias=bias)
    x = synth.activations(m, k, seed=m)
    xd = dev(x, torch.bfloat16)
    ys = [lin.forward(xd) for _ in range(3)]
    close(ys[0], oracle.linear(x, synth.bf16_round(w), b))
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[1], ys[2])  # partial tiles are added in split order
    ws = gemm.workspace(n, k, "cuda")
    gemm.check(ws)
    assert not ws[:256].view(torch.int32).any()  # the tickets in the workspace header are back at zero


def test_fused_split_k_other_layouts(cuda):
    w8, sinv = synth.fp8_layer(1024, 4096, seed=5)
    lin = L.Fp8Linear(dev(w8), dev(sinv))
    x = synth.activations(32, 4096, seed=6)
    close(lin.forward(dev(x, torch.bfloat16)), oracle.linear(x, synth.bf16_round(oracle.fp8_dequant(w8, sinv))))
    glin, gw = gptq_layer(4096, 1024, 128, seed=8)
    close(glin.forward(dev(x, torch.bfloat16)), oracle.linear(x, synth.bf16_round(gw)))
    gemm.check(gemm.workspace(1024, 4096, "cuda"))

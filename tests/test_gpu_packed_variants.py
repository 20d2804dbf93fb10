"""The packed-int layouts next to 4-bit AWQ through the resident operator (PackedQuantLinear, linear.rs:403-534):
GPTQ 4/8-bit (PackDim::In; awq.rs:442-590) and the 8-bit AWQ layout W8A16 (quant_kernels.metal:1-16,40-48),
decode GEMV and prefill GEMM, against the CPU oracle. Dequantization is bit-exact; matmuls within
max|err| <= 2e-2 * ||row||_inf of the oracle's f32 result."""
import numpy as np
import pytest
import torch

import oracle
from oxydllm_b200 import formats as F
from oxydllm_b200 import gemm
from oxydllm_b200 import linear as L
from oxydllm_b200 import synth

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dtype) if dtype is not None else t).cuda()


def words(a):
    return dev(a.view(np.int32))


def close(y, ref, label):
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all(), f"{label}: non-finite"
    err = np.abs(got - ref)
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (err <= 2e-2 * row_inf + 1e-6).all(), f"{label}: max err {err.max()} row_inf {row_inf.max()}"


def gptq_case(k, n, g, bits, seed):
    rng = np.random.default_rng(seed)
    iw = rng.integers(0, 1 << bits, size=(k, n), dtype=np.uint32)
    iz = rng.integers(0, (1 << bits) - 1, size=(k // g, n), dtype=np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n)) * 0.02) / 7.0 + 1e-4).astype(np.float16)
    bias = synth.bf16_round(rng.standard_normal(n).astype(np.float32))
    return F.pack_gptq_qweight(iw, bits), F.pack_gptq_qzeros(iz, bits), sc, bias


@pytest.mark.parametrize("bits,sym", [(4, False), (4, True), (8, False), (8, True)])
@pytest.mark.parametrize("m,k,n,g", [(1, 256, 256, 128), (2, 192, 104, 64), (3, 1024, 520, 128), (4, 64, 8, 32),
                                     (5, 512, 1000, 128), (8, 4096, 1024, 128), (1, 4096, 4096, 128)])
def test_gptq_gemv_matches_oracle(cuda, bits, sym, m, k, n, g):
    qw, qz, sc, bias = gptq_case(k, n, g, bits, seed=m + n + bits)
    x = synth.activations(m, k, seed=m)
    ref = oracle.linear(x, oracle.gptq_dequant(qw, None if sym else qz, sc, bits, sym), bias)
    raw = L.QuantWeight.new_gptq(bits, sym, words(qw), None if sym else words(qz), dev(sc))
    lin = L.PackedQuantLinear(raw, dev(bias, torch.bfloat16))
    y = lin.forward(dev(x, torch.bfloat16))
    assert y.shape == (m, n)
    close(y, ref, f"gptq gemv bits={bits} sym={sym} m={m}")


@pytest.mark.parametrize("bits", [4, 8])
def test_gptq_operator_dispatch_gemv_and_gemm_agree_with_oracle(cuda, bits):
    """AnyLinear.from_quant keeps GPTQ packed; m <= 8 runs the GEMV, larger m the tensor-core GEMM."""
    k, n, g = 1024, 768, 128
    qw, qz, sc, bias = gptq_case(k, n, g, bits, seed=5)
    any_lin = L.AnyLinear.from_quant(L.QuantWeight.new_gptq(bits, False, words(qw), words(qz), dev(sc)), dev(bias, torch.bfloat16))
    assert any_lin.variant == "PackedQuant" and any_lin.inner.pack_dim == "in"
    w = oracle.gptq_dequant(qw, qz, sc, bits)
    for m in (8, 9, 70):
        x = synth.activations(m, k, seed=m)
        y = any_lin.forward(dev(x, torch.bfloat16))
        close(y, oracle.linear(x, oracle.round_bf16(w) if m > 8 else w, bias), f"gptq operator m={m}")
    gemm.check(gemm.workspace(n, k, "cuda"))


def w8_case(k, n, g, seed):
    rng = np.random.default_rng(seed)
    iw = rng.integers(0, 256, size=(k, n), dtype=np.uint32)
    iz = rng.integers(0, 256, size=(k // g, n), dtype=np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n)) * 0.02) / 127.0 + 1e-5).astype(np.float16)
    return F.pack_w8a16(iw), F.pack_w8a16(iz), sc


@pytest.mark.parametrize("out", ["f32", "bf16", "f16"])
def test_w8a16_dequant_bit_exact(cuda, out):
    k, n, g = 192, 100, 64
    qw, qz, sc = w8_case(k, n, g, seed=1)
    ref = oracle.w8a16_dequant(qw, qz, sc)
    raw = L.QuantWeight(8, "out", "sequential", "signed", words(qw), words(qz), dev(sc))
    t = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[out]
    got = L.dequantize_quant(raw, t)
    if out == "f32":
        assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    else:
        want = oracle.to_bf16_bits(ref) if out == "bf16" else oracle.to_f16_bits(ref)
        assert np.array_equal(got.cpu().view(torch.int16).numpy().view(np.uint16), want)


@pytest.mark.parametrize("m,k,n,g", [(1, 256, 256, 128), (2, 192, 100, 64), (3, 1024, 520, 128), (8, 2048, 1024, 128),
                                     (33, 256, 64, 32), (70, 512, 520, 128)])
def test_w8a16_linear_matches_oracle(cuda, m, k, n, g):
    qw, qz, sc = w8_case(k, n, g, seed=m + n)
    bias = synth.bf16_round(np.random.default_rng(3).standard_normal(n).astype(np.float32))
    x = synth.activations(m, k, seed=m)
    w = oracle.w8a16_dequant(qw, qz, sc)
    raw = L.QuantWeight(8, "out", "sequential", "signed", words(qw), words(qz), dev(sc))
    lin = L.PackedQuantLinear(raw, dev(bias, torch.bfloat16))
    y = lin.forward(dev(x, torch.bfloat16))
    close(y, oracle.linear(x, oracle.round_bf16(w) if m > 8 else w, bias), f"w8a16 m={m}")
    if m > 8:
        gemm.check(gemm.workspace(n, k, "cuda"))

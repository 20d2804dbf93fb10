"""Tensor-core (tcgen05) prefill matmuls against the CPU oracle: y = x @ deq(W)^T in f32 with the
weights first rounded to bf16 (what the tensor cores are fed; the reference's GPU paths round the
dequantized weight to the activation dtype too, linear.rs:143, mpp_gemm.metal:143). Tolerance:
max|err| <= 2e-2 * ||row||_inf."""
import ctypes

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


def check(y, ref, label):
    gemm.check(gemm.workspace(1, 8, y.device))  # no bounded wait ran out
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all(), f"{label}: non-finite"
    err = np.abs(got - ref)
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (err <= 2e-2 * row_inf + 1e-6).all(), f"{label}: max err {err.max()} row_inf {row_inf.max()}"


@pytest.mark.parametrize("m,k,n,g", [(70, 192, 104, 64), (70, 160, 104, 32), (128, 256, 256, 128), (33, 64, 8, 64),
                                     (300, 1024, 520, 128), (2048, 512, 768, 128)])
def test_awq_gemm(cuda, m, k, n, g):
    # (70,192,104,64), (70,160,104,32): partial tiles of metal_ops.rs:5004-5055
    qw, qz, sc = synth.awq_layer(k, n, g, seed=m)
    x = synth.activations(m, k, seed=m + 1)
    bias = synth.bf16_round(np.random.default_rng(2).standard_normal(n).astype(np.float32))
    ref = oracle.linear(x, oracle.round_bf16(oracle.awq_dequant(qw, qz, sc)), bias)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)), dev(bias, torch.bfloat16))
    y = lin.forward(dev(x, torch.bfloat16))
    assert y.shape == (m, n)
    check(y, ref, f"awq gemm {m}x{k}x{n}")


def test_awq_gemm_matches_gemv_rows(cuda):
    k, n, g = 512, 512, 128
    qw, qz, sc = synth.awq_layer(k, n, g, seed=3)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    x = dev(synth.activations(64, k, seed=4), torch.bfloat16)
    big = lin.forward(x).float()
    small = lin.forward(x[:8]).float()
    assert torch.allclose(big[:8], small, rtol=2e-2, atol=2e-2 * float(small.abs().max()))


@pytest.mark.parametrize("ggml_type", [F.GGML_Q4_0, F.GGML_Q8_0, F.GGML_Q4_K, F.GGML_Q6_K, F.GGML_Q4_1, F.GGML_Q5_0, F.GGML_Q5_1, F.GGML_Q5_K,
                                       F.GGML_Q2_K, F.GGML_Q3_K])
@pytest.mark.parametrize("n,k,m", [(512, 2048, 33), (1001, 512, 70), (2048, 2048, 9 * 8)])
def test_gguf_gemm(cuda, ggml_type, n, k, m):
    # shapes/m of metal_ops.rs:6386-6470 (m in {33, 70}, odd n = 1001)
    w = np.array([((i % 17) - 8) * 0.05 for i in range(n * k)], np.float32).reshape(n, k)
    data = F.GGML_QUANTIZE[ggml_type](w)
    x = synth.activations(m, k, seed=n)
    ref = oracle.linear(x, oracle.round_bf16(oracle.gguf_dequant(ggml_type, data, n, k)))
    y = L.QLinear(ggml_type, dev(data), n, k).forward(dev(x, torch.bfloat16))
    check(y, ref, f"gguf gemm type={ggml_type}")


@pytest.mark.parametrize("n,k,m", [(256, 1024, 64), (1792, 4096, 2048 // 8), (384, 128, 40)])
def test_fp8_gemm(cuda, n, k, m):
    q, s = synth.fp8_layer(n, k, seed=n)
    x = synth.activations(m, k, seed=7)
    ref = oracle.linear(x, oracle.round_bf16(oracle.fp8_dequant(q, s)))
    y = L.Fp8Linear(dev(q), dev(s)).forward(dev(x, torch.bfloat16))
    check(y, ref, f"fp8 gemm {n}x{k} m={m}")


@pytest.mark.parametrize("n,k,m", [(10, 64, 33), (2880, 2880, 200), (5760, 2880, 64)])
def test_mxfp4_gemm(cuda, n, k, m):
    # (10, 64, 33) from metal_ops.rs:6621-6670; 2880 = GPT-OSS hidden (k tail of 64 inside a 128 tile)
    b, s = synth.mxfp4_layer(n, k, seed=n)
    bias = synth.bf16_round(np.random.default_rng(1).standard_normal(n).astype(np.float32) * 0.02)
    x = synth.activations(m, k, seed=3)
    ref = oracle.linear(x, oracle.mxfp4_dequant(b, s, n, k), bias)  # MXFP4 values are exact in bf16
    y = L.Mxfp4Linear(dev(b), dev(s), dev(bias, torch.bfloat16), k, n).forward(dev(x, torch.bfloat16))
    check(y, ref, f"mxfp4 gemm {n}x{k} m={m}")


def test_workspace_too_small_is_rejected(cuda):
    import ctypes
    from oxydllm_b200 import _lib
    one = ctypes.c_void_p(256)
    with pytest.raises(_lib.OxqError, match="workspace of"):
        _lib.call("oxq_awq_gemm", one, 2, one, one, one, 1, None, 0, one, 2, 64, 256, 256, 128, one, 16, None)


@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("m,k,inter,g", [(1, 256, 64, 64), (7, 512, 200, 128), (33, 256, 64, 32), (300, 1024, 1000, 128),
                                         (2048, 512, 1024, 128), (64, 4096, 9216, 128),  # the last needs two slabs
                                         (24, 512, 256, 128), (200, 1024, 1024, 64), (256, 2048, 9216, 128)])
def test_gated_ffn_gate_up_matches_oracle(cuda, activation, m, k, inter, g):
    """act(gate) * up on the fused [gate | up] AWQ weight: GEMV route for m <= 16, the kernel that unpacks inside the
    tensor-core loop for 17 .. 256 tokens on the shapes it takes (GEMV up to 32 elsewhere), GEMM epilogue above."""
    from oxydllm_b200 import gemm
    qw, qz, sc = synth.awq_layer(k, 2 * inter, g, seed=m + inter)
    sc = (sc.astype(np.float32) * 8.0).astype(sc.dtype)  # larger pre-activations: both tails of the activations
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    x = synth.activations(m, k, seed=3)
    w = oracle.awq_dequant(qw, qz, sc)
    if m > 32 or (m > 16 and g >= 64 and inter % 64 == 0 and k % 128 == 0):
        w = oracle.round_bf16(w)  # the tensor-core paths multiplies the bf16-rounded dense weight
    ref = oracle.gated_ffn(x, w, activation)
    y = L.GatedFfnProjection(lin, activation).forward(dev(x, torch.bfloat16))
    gemm.check(gemm.workspace(1, 8, "cuda"))
    got = y.float().cpu().numpy()
    assert got.shape == (m, inter) and np.isfinite(got).all()
    # products of two projections: tolerance relative to the row's largest |gate| * |up| scale
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (np.abs(got - ref) <= 3e-2 * row_inf + 1e-4).all(), float(np.abs(got - ref).max())


def test_bounded_wait_expiry_is_reported_and_the_workspace_stays_usable(cuda):
    # A wait that nothing satisfies gives up after its limit (50 ms in the self-test), records its code and the
    # kernel ends; the check reports it once, and the same workspace then serves a normal call.
    from oxydllm_b200 import _lib
    k, n, m = 512, 256, 70
    ws = gemm.workspace(n, k, "cuda")
    gemm.check(ws)
    _lib.call("oxq_selftest_wait_expiry", ctypes.c_void_p(ws.data_ptr()), 9, None)
    with pytest.raises(_lib.OxqError, match="bounded wait 9") as e:
        gemm.check(ws)
    assert e.value.status < 0
    gemm.check(ws)  # reported once, clean again
    qw, qz, sc = synth.awq_layer(k, n, 128, seed=3)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    x = synth.activations(m, k, seed=4)
    y = lin.forward(dev(x, torch.bfloat16))
    check(y, oracle.linear(x, synth.bf16_round(oracle.awq_dequant(qw, qz, sc))), "after an expired wait")
    gemm.check(ws)


@pytest.mark.parametrize("m", [100, 200])  # one-CTA kernel, two-CTA kernel
def test_gemm_kernel_survives_a_producer_that_never_loads(cuda, m):
    # The kernel's own roles: with no tile data ever arriving the MMA issuer gives up after the 2 s limit, everybody
    # falls through, tensor memory is freed, the kernel returns, the check reports code 2 and the workspace still works.
    from oxydllm_b200 import _lib
    k, n = 1024, 1024
    ws = gemm.workspace(n, k, "cuda")
    gemm.check(ws)
    _lib.call("oxq_selftest_gemm_wait_expiry", ctypes.c_void_p(ws.data_ptr()), ws.numel(), m, None)
    with pytest.raises(_lib.OxqError, match=r"bounded wait [23]"):  # the issuer (2) or an epilogue warp (3) gives up first
        gemm.check(ws)
    gemm.check(ws)
    qw, qz, sc = synth.awq_layer(k, n, 128, seed=9)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc.astype(np.float32))))  # f32 scales: slab path
    x = synth.activations(300, k, seed=10)
    y = lin.forward(dev(x, torch.bfloat16))
    check(y, oracle.linear(x, synth.bf16_round(oracle.awq_dequant(qw, qz, sc.astype(np.float32)))), "after an aborted GEMM")

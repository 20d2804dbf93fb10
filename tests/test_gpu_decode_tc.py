"""oxq_awq_decode_matmul: the decode-batch AWQ matmul on tcgen05 with one-byte (E4M3-coded) weights and
three-piece E5M2 activations, against the CPU oracle's f32 ``x @ deq(W)^T`` (awq.rs:391-417,612-633;
linear.rs:450-505). The arithmetic is exact up to f32 accumulation, so the error budget is the bf16 rounding
of the output: max|err| <= 2e-2 * ||row||_inf as everywhere. Same inputs give the same bits (fixed-order sums)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oxydllm_b200 import _lib, gemm
from oxydllm_b200 import linear as L
from oxydllm_b200 import synth

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dtype) if dtype is not None else t).cuda()


def layer(k, n, g, seed, bias=False, scales_dtype=np.float16):
    qw, qz, sc = synth.awq_layer(k, n, g, seed=seed)
    b = synth.bf16_round(np.random.default_rng(seed).standard_normal(n).astype(np.float32)) if bias else None
    sc_t = dev(sc) if scales_dtype == np.float16 else dev(sc.astype(np.float32), torch.bfloat16 if scales_dtype == "bf16" else torch.float32)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, dev(qw.view(np.int32)), dev(qz.view(np.int32)), sc_t),
                              dev(b, torch.bfloat16) if bias else None)
    return lin, qw, qz, sc_t.float().cpu().numpy(), b


def run(lin, x, m, n, dtype=torch.bfloat16):
    y = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    gemm.awq_decode_matmul(lin, dev(x, torch.bfloat16), y)
    gemm.check(gemm.decode_workspace(m, lin.in_features, n, "cuda"))
    return y


@pytest.mark.parametrize("m,k,n,g,bias", [
    (1, 128, 128, 128, False), (1, 512, 256, 128, True), (2, 256, 32, 128, False), (3, 1024, 1056, 128, True),
    (4, 4096, 4096, 128, False), (7, 384, 544, 128, True), (8, 1024, 2048, 256, False), (9, 512, 544, 256, True),
    (16, 2048, 2048, 128, False), (17, 1024, 1024, 512, True), (24, 1024, 2048, 128, False), (32, 4096, 1024, 128, True)])
def test_decode_matmul_matches_oracle(cuda, m, k, n, g, bias):
    lin, qw, qz, sc, b = layer(k, n, g, seed=m + n, bias=bias)
    x = synth.activations(m, k, seed=m)
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc.astype(np.float16)), b)
    got = run(lin, x, m, n).float().cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-6).all()


def test_decode_matmul_wide_dynamic_range_and_rerun(cuda):
    """Tokens with very different magnitudes, outlier channels inside a k group, zeros: the per-(token, group)
    power-of-two scaling keeps the three-piece split exact. A second call on the same workspace gives the same bits."""
    m, k, n, g = 5, 1024, 1056, 128
    lin, qw, qz, sc, _ = layer(k, n, g, seed=3)
    x = synth.activations(m, k, seed=4)
    x[1] *= 1e-3
    x[2, ::7] *= 300.0
    x[3] *= 2.0 ** 40
    x[4, 128:256] = 0.0
    x = synth.bf16_round(x)
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc.astype(np.float16)))
    y1 = run(lin, x, m, n)
    got = y1.float().cpu().numpy()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-6).all()
    y2 = run(lin, x, m, n)
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("scales_dtype", ["bf16", "f32"])
def test_decode_matmul_other_scale_dtypes_and_f32_output(cuda, scales_dtype):
    m, k, n, g = 6, 512, 512, 128
    lin, qw, qz, sc, _ = layer(k, n, g, seed=9, scales_dtype=scales_dtype)
    x = synth.activations(m, k, seed=2)
    w = oracle.awq_dequant(qw, qz, sc)  # scales as the kernel sees them (bf16-rounded or f32)
    got = run(lin, x, m, n, torch.float32).cpu().numpy()
    ref = oracle.linear(x, w)
    assert (np.abs(got - ref) <= 1e-4 * np.abs(ref).max(axis=1, keepdims=True) + 1e-6).all()  # f32 out: only f32 accumulation error


def test_decode_matmul_full_c1_shape_and_lm_head_width(cuda):
    """K = 4096, N = 14336 (every SM shares tiles with its neighbours) and N = 128256 (partial last tile)."""
    for m, n in ((5, 14336), (32, 14336), (7, 128256)):
        lin, qw, qz, sc, _ = layer(4096, n, 128, seed=n % 101)
        x = synth.activations(m, 4096, seed=m)
        y = run(lin, x, m, n)
        for a, b in ((0, 64), (n // 2 - 32, n // 2 + 32), (n - 64, n)):
            ref = oracle.linear(x, oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b].astype(np.float16)))
            got = y[:, a:b].float().cpu().numpy()
            assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-6).all()


def test_decode_matmul_rejections(cuda):
    one = ctypes.c_void_p(256)
    args = lambda m, k, n, g, ws=one, wsb=1 << 30: (one, _lib.OXQ_BF16, one, one, one, _lib.OXQ_F16, None, 0, one, _lib.OXQ_BF16,
                                                    m, k, n, g, ws, wsb, None)
    with pytest.raises(_lib.OxqError, match="outside 1.."):
        _lib.call("oxq_awq_decode_matmul", *args(33, 256, 256, 128))
    with pytest.raises(_lib.OxqError, match="needs out_features"):
        _lib.call("oxq_awq_decode_matmul", *args(4, 256, 264, 128))
    with pytest.raises(_lib.OxqError, match="needs out_features"):
        _lib.call("oxq_awq_decode_matmul", *args(4, 256, 256, 64))
    with pytest.raises(_lib.OxqError, match="workspace of"):
        _lib.call("oxq_awq_decode_matmul", *args(4, 256, 256, 128, one, 16))
    assert int(_lib.load().oxq_decode_max_m()) == 32

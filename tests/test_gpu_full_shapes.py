"""Code paths that only large or odd shapes reach, against the CPU oracle: weights cut into several
dequantization slabs (more than 128 MiB as bf16), the GPTQ prefill matmul, and the benchmark
configurations at their full sizes (checked on column / token subsets, since the oracle is a CPU
restatement: a pure column slice of a packed weight is itself a valid packed weight, awq.rs:256-323).
Tolerance as everywhere: max|err| <= 2e-2 * ||row||_inf against the oracle's f32 result on the
bf16-rounded weight (what the tensor cores are fed; linear.rs:143, mpp_gemm.metal:143)."""
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


def close(got, ref, label, tol=2e-2):
    got = got.float().cpu().numpy()
    assert np.isfinite(got).all(), f"{label}: non-finite"
    err = np.abs(got - ref)
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (err <= tol * row_inf + 1e-6).all(), f"{label}: max err {err.max()} row_inf {row_inf.max()}"


def col_windows(n, boundary=None, width=64):
    """Column windows (multiples of 8): both ends, and both sides of a slab boundary."""
    w = [(0, width), (n - width, n)]
    if boundary is not None and width <= boundary <= n - width:
        w.append((boundary - width, boundary + width))
    return w


# ------------------------------------------------------------------ GPTQ prefill matmul
@pytest.mark.parametrize("bits_,sym", [(4, False), (4, True), (8, False), (8, True)])
@pytest.mark.parametrize("m,k,n,g", [(64, 256, 256, 128), (70, 192, 104, 64), (300, 1024, 520, 128), (33, 64, 8, 32)])
def test_gptq_gemm_matches_oracle(cuda, bits_, sym, m, k, n, g):
    rng = np.random.default_rng(m + n + bits_)
    iw = rng.integers(0, 1 << bits_, size=(k, n), dtype=np.uint32)
    iz = rng.integers(0, (1 << bits_) - 1, size=(k // g, n), dtype=np.uint32)
    sc = (np.abs(rng.standard_normal((k // g, n)) * 0.02) / 7.0 + 1e-4).astype(np.float16)
    qw, qz = F.pack_gptq_qweight(iw, bits_), F.pack_gptq_qzeros(iz, bits_)
    bias = synth.bf16_round(rng.standard_normal(n).astype(np.float32))
    x = synth.activations(m, k, seed=m)
    ref = oracle.linear(x, oracle.round_bf16(oracle.gptq_dequant(qw, None if sym else qz, sc, bits_, sym)), bias)
    raw = L.QuantWeight.new_gptq(bits_, sym, words(qw), None if sym else words(qz), dev(sc))
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    gemm.gptq_matmul(raw, dev(x, torch.bfloat16), y, dev(bias, torch.bfloat16))
    gemm.check(gemm.workspace(n, k, "cuda"))
    close(y, ref, f"gptq gemm bits={bits_} sym={sym}")


# ------------------------------------------------------------------ several slabs
MULTI_K, MULTI_N, MULTI_M = 4096, 20480, 64  # 160 MiB as bf16: two slabs, boundary at row 16384


def test_awq_gemm_two_slabs(cuda):
    k, n, m = MULTI_K, MULTI_N, MULTI_M
    assert gemm.workspace_bytes(n, k) < n * k * 2
    qw, qz, sc = synth.awq_layer(k, n, 128, seed=7)
    x = synth.activations(m, k, seed=8)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    gemm.awq_matmul(lin, dev(x, torch.bfloat16), y)
    gemm.check(gemm.workspace(n, k, "cuda"))
    for a, b in col_windows(n, 16384):
        ref = oracle.linear(x, oracle.round_bf16(oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b])))
        close(y[:, a:b], ref, f"awq two slabs cols {a}:{b}")


def test_noalloc_gemm_four_slabs_against_oracle(cuda):
    """k = 4096 leaves 1024 rows per slab in the built-in 8 MiB array: n = 4096 runs four slabs; m > 128 takes the
    two-CTA kernel. Also checks that the entry point leaves the amount of free device memory unchanged."""
    import ctypes
    from oxydllm_b200 import _lib
    k, n, m = 4096, 4096, 200
    qw, qz, sc = synth.awq_layer(k, n, 128, seed=11)
    x = synth.activations(m, k, seed=12)
    xd, qwd, qzd, scd = dev(x, torch.bfloat16), words(qw), words(qz), dev(sc)
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def call():
        _lib.call("oxq_awq_gemm_noalloc", p(xd), _lib.OXQ_BF16, p(qwd), p(qzd), p(scd), _lib.OXQ_F16, None, 0, p(y),
                  _lib.OXQ_BF16, m, k, n, 128, st)
    call()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    call()
    _lib.call("oxq_awq_gemm_noalloc_check", st)
    assert torch.cuda.mem_get_info()[0] == free0
    for a, b in col_windows(n, 1024) + col_windows(n, 3072):
        ref = oracle.linear(x, oracle.round_bf16(oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b])))
        close(y[:, a:b], ref, f"noalloc four slabs cols {a}:{b}")


def test_fp8_gemm_two_slabs(cuda):
    k, n, m = MULTI_K, MULTI_N, MULTI_M
    q, s = synth.fp8_layer(n, k, seed=9)
    x = synth.activations(m, k, seed=10)
    y = L.Fp8Linear(dev(q), dev(s)).forward(dev(x, torch.bfloat16))
    gemm.check(gemm.workspace(n, k, "cuda"))
    w = oracle.fp8_dequant(q, s)
    for a, b in col_windows(n, 16384):
        close(y[:, a:b], oracle.linear(x, oracle.round_bf16(w[a:b])), f"fp8 two slabs rows {a}:{b}")


def test_mxfp4_gemm_two_slabs(cuda):
    k, n, m = MULTI_K, MULTI_N, MULTI_M
    rng = np.random.default_rng(3)
    blocks = rng.integers(0, 256, size=(n, k // 32, 16), dtype=np.uint8)
    scales = rng.integers(118, 126, size=(n, k // 32), dtype=np.uint8)
    x = synth.activations(m, k, seed=4)
    y = L.Mxfp4Linear(dev(blocks), dev(scales), None, k, n).forward(dev(x, torch.bfloat16))
    gemm.check(gemm.workspace(n, k, "cuda"))
    for a, b in col_windows(n, 16384):
        ref = oracle.linear(x, oracle.mxfp4_dequant(blocks[a:b], scales[a:b], b - a, k))
        close(y[:, a:b], ref, f"mxfp4 two slabs rows {a}:{b}")


def test_gguf_q8_0_gemm_two_slabs(cuda):
    k, n, m = MULTI_K, MULTI_N, MULTI_M
    rng = np.random.default_rng(5)
    nb = k // 32
    data = np.zeros((n, nb, 34), np.uint8)
    data[:, :, :2] = (np.abs(rng.standard_normal((n, nb))) * 1e-3 + 1e-4).astype(np.float16).view(np.uint8).reshape(n, nb, 2)
    data[:, :, 2:] = rng.integers(0, 256, size=(n, nb, 32), dtype=np.uint8)
    x = synth.activations(m, k, seed=6)
    y = L.QLinear(F.GGML_Q8_0, dev(data.reshape(-1)), n, k).forward(dev(x, torch.bfloat16))
    gemm.check(gemm.workspace(n, k, "cuda"))
    for a, b in col_windows(n, 16384):
        ref = oracle.linear(x, oracle.round_bf16(oracle.gguf_dequant(F.GGML_Q8_0, data[a:b].reshape(-1), b - a, k)))
        close(y[:, a:b], ref, f"q8_0 two slabs rows {a}:{b}")


# ------------------------------------------------------------------ benchmark configurations at full size
@pytest.fixture(scope="module")
def c1_layer():
    qw, qz, sc = synth.awq_layer(4096, 14336, 128, seed=0)
    return qw, qz, sc, L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16, 32])
def test_c1_every_m_of_the_sweep(cuda, c1_layer, m):
    qw, qz, sc, lin = c1_layer
    x = synth.activations(m, 4096, seed=m)
    y = lin.forward(dev(x, torch.bfloat16))
    for a, b in col_windows(14336) + [(7168 - 64, 7168 + 64)]:
        ref = oracle.linear(x, oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b]))
        close(y[:, a:b], ref, f"C1 m={m} cols {a}:{b}")


@pytest.mark.parametrize("n", [4096, 14336, 128256])
def test_c2_full_m_every_n(cuda, n):
    """C2: M = 2048, K = 4096, N in {4096, 14336, 128256}; N = 128256 is eight slabs and ends in a partial tile."""
    k, m = 4096, 2048
    qw, qz, sc = synth.awq_layer(k, n, 128, seed=n % 97)
    x = synth.activations(m, k, seed=5)
    lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, words(qw), words(qz), dev(sc)))
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    gemm.awq_matmul(lin, dev(x, torch.bfloat16), y)
    gemm.check(gemm.workspace(n, k, "cuda"))
    rows = np.r_[0:16, 1000:1016, 2032:2048]
    bnd = 16384 if n > 16384 else None
    for a, b in col_windows(n, bnd) + ([(n // 2 - 32, n // 2 + 32)] if n > 16384 else []):
        ref = oracle.linear(x[rows], oracle.round_bf16(oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b])))
        close(y[rows][:, a:b], ref, f"C2 n={n} cols {a}:{b}")


@pytest.mark.parametrize("m", [1, 32, 2048])
def test_c3_every_m(cuda, m):
    n, k = 14336, 4096
    q, s = synth.fp8_layer(n, k, seed=3)
    x = synth.activations(m, k, seed=m)
    y = L.Fp8Linear(dev(q), dev(s)).forward(dev(x, torch.bfloat16))
    if m > 32:
        gemm.check(gemm.workspace(n, k, "cuda"))
    rows = np.arange(m) if m <= 32 else np.r_[0:16, 2032:2048]
    w = oracle.fp8_dequant(q, s)
    for a, b in col_windows(n) + [(7168 - 64, 7168 + 64)]:
        wa = oracle.round_bf16(w[a:b]) if m > 32 else w[a:b]
        close(y[rows][:, a:b], oracle.linear(x[rows], wa), f"C3 m={m} rows {a}:{b}")


def test_awq_gemm_tp_entry_places_tile_in_local_and_peer_outputs(cuda):
    """oxq_awq_gemm_tp on one GPU: a second buffer of the same GPU stands in for a peer's output. Both receive this
    shard's columns [col_base, col_base + n_local) of an n_full-wide output and nothing else."""
    import ctypes
    from oxydllm_b200 import _lib
    m, k, n_full, g = 200, 512, 1024, 128
    a, b = 256, 768
    qw, qz, sc = synth.awq_layer(k, n_full, g, seed=21)
    bias = synth.bf16_round(np.random.default_rng(4).standard_normal(n_full).astype(np.float32))
    x = synth.activations(m, k, seed=22)
    xd, qwd, qzd, scd = dev(x, torch.bfloat16), words(qw[:, a // 8:b // 8]), words(qz[:, a // 8:b // 8]), dev(sc[:, a:b])
    bd = dev(bias, torch.bfloat16)
    y_local = torch.full((m, n_full), 7.0, dtype=torch.bfloat16, device="cuda")
    y_peer = torch.full((m, n_full), 7.0, dtype=torch.bfloat16, device="cuda")
    peers = (ctypes.c_void_p * 1)(y_peer.data_ptr())
    ws = gemm.workspace(b - a, k, "cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.call("oxq_awq_gemm_tp", p(xd), _lib.OXQ_BF16, p(qwd), p(qzd), p(scd), _lib.OXQ_F16, p(bd), _lib.OXQ_BF16, p(y_local),
              ctypes.cast(peers, ctypes.c_void_p), 1, _lib.OXQ_BF16, m, k, b - a, a, n_full, g, p(ws), ws.numel(),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    gemm.check(ws)
    ref = oracle.linear(x, oracle.round_bf16(oracle.awq_dequant(qw[:, a // 8:b // 8], qz[:, a // 8:b // 8], sc[:, a:b])), bias[a:b])
    for y in (y_local, y_peer):
        close(y[:, a:b], ref, "tp tile")
        assert bool((y[:, :a] == 7.0).all()) and bool((y[:, b:] == 7.0).all())
    assert torch.equal(y_local, y_peer)

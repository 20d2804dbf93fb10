"""Second opinions on the oracle from implementations independent of it:
committed gguf-py dequantization fixtures (tests/golden/make_golden.py) and
torch's float8_e4m3fn cast."""
import os

import numpy as np
import pytest

import oracle
from oxydllm_b200 import formats as F

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gguf_blocks.npz")


@pytest.mark.parametrize("ggml_type", [F.GGML_Q4_0, F.GGML_Q8_0, F.GGML_Q4_K, F.GGML_Q6_K, F.GGML_Q4_1, F.GGML_Q5_0, F.GGML_Q5_1, F.GGML_Q5_K,
                                       F.GGML_Q2_K, F.GGML_Q3_K])
def test_gguf_dequant_bit_exact_against_gguf_py_fixture(ggml_type):
    z = np.load(GOLDEN)
    rows, cols = (int(v) for v in z[f"shape_{ggml_type}"])
    got = oracle.gguf_dequant(ggml_type, z[f"blocks_{ggml_type}"], rows, cols)
    assert np.array_equal(got.view(np.uint32), z[f"deq_{ggml_type}"].view(np.uint32))


@pytest.mark.parametrize("ggml_type,max_rel", [(F.GGML_Q4_0, 0.12), (F.GGML_Q8_0, 0.01), (F.GGML_Q4_K, 0.11),
                                               (F.GGML_Q6_K, 0.03), (F.GGML_Q4_1, 0.11), (F.GGML_Q5_0, 0.06),
                                               (F.GGML_Q5_1, 0.05), (F.GGML_Q5_K, 0.05), (F.GGML_Q2_K, 0.45), (F.GGML_Q3_K, 0.25)])
def test_encoders_emit_valid_blocks(ggml_type, max_rel):
    w = (np.random.default_rng(3).standard_normal((8, 512)) * 0.02).astype(np.float32)
    data = F.GGML_QUANTIZE[ggml_type](w)
    bel, bby = F.GGML_BLOCK[ggml_type]
    assert data.dtype == np.uint8 and data.size == 8 * (512 // bel) * bby
    dq = oracle.gguf_dequant(ggml_type, data, 8, 512)
    assert np.linalg.norm(dq - w) / np.linalg.norm(w) < max_rel


def test_gguf_rejects_bad_sizes():
    with pytest.raises(ValueError):
        oracle.gguf_dequant(F.GGML_Q4_K, np.zeros(144, np.uint8), 1, 128)
    with pytest.raises(ValueError):
        oracle.gguf_dequant(F.GGML_Q8_0, np.zeros(33, np.uint8), 1, 32)


def test_e4m3_against_torch():
    torch = pytest.importorskip("torch")
    b = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(b).view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_decode(b)
    ok = ~np.isnan(ref)
    assert np.array_equal(np.isnan(got), ~ok)
    assert np.array_equal(got[ok].view(np.uint32), ref[ok].view(np.uint32))
    x = (np.random.default_rng(0).standard_normal(4096) * 100).astype(np.float32)
    enc = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(F.e4m3_encode(x), enc)


def test_roundings_against_numpy_and_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 1e4)])
    assert np.array_equal(oracle.to_f16_bits(x), x.astype(np.float16).view(np.uint16))
    tb = torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.to_bf16_bits(x), tb)
    h = rng.integers(0, 1 << 16, size=4096).astype(np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = oracle.f16_bits_to_f32(h)
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok].view(np.uint32), ref[ok].view(np.uint32))


def test_mxfp4_and_fp8_quantizers_reconstruct():
    w = (np.random.default_rng(2).standard_normal((16, 256)) * 0.02).astype(np.float32)
    b, s = F.quantize_mxfp4(w)
    assert b.shape == (16, 8, 16) and s.shape == (16, 8)
    dq = oracle.mxfp4_dequant(b, s, 16, 256)
    assert np.linalg.norm(dq - w) / np.linalg.norm(w) < 0.15
    q, sc = F.quantize_fp8_block(w.reshape(32, 128).repeat(4, axis=0), 128)
    assert q.shape == (128, 128) and sc.shape == (1, 1)
    dq = oracle.fp8_dequant(q, sc)
    assert np.linalg.norm(dq - w.reshape(32, 128).repeat(4, axis=0)) / np.linalg.norm(w) < 0.1

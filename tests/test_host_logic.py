"""Host-side mirror of the reference operator surface: container arithmetic,
shape rejection and variant selection (CPU tensors; nothing is launched)."""
import numpy as np
import pytest
import torch

from oxydllm_b200 import formats as F
from oxydllm_b200 import linear as L


def _awq(k=8, n=16, g=4):
    return L.QuantWeight.new_awq(4, torch.zeros((k, n // 8), dtype=torch.int32),
                                 torch.zeros((k // g, n // 8), dtype=torch.int32), torch.zeros((k // g, n)))


def test_quant_weight_geometry():
    raw = _awq()
    assert (raw.in_features(), raw.out_features(), raw.group_size(), raw.pack_factor()) == (8, 16, 4, 8)
    g = L.QuantWeight.new_gptq(8, False, torch.zeros((8, 16), dtype=torch.int32),
                               torch.zeros((2, 4), dtype=torch.int32), torch.zeros((2, 16)))
    assert (g.in_features(), g.out_features(), g.group_size(), g.pack_factor()) == (32, 16, 16, 4)
    assert g.zero_point == "plus_one" and L.QuantWeight.new_gptq(4, True, g.qweight, None, g.scales).zero_point == "symmetric"


def test_dequantize_awq_rejects_wrong_shapes():
    # awq.rs:1112-1121
    raw = L.QuantWeight.new_awq(4, torch.zeros((8, 2), dtype=torch.int32), torch.zeros((2, 2), dtype=torch.int32),
                                torch.zeros((2, 8)))
    with pytest.raises(ValueError):
        L.dequantize_awq(raw)


def test_no_cpu_path():
    with pytest.raises(ValueError, match="CUDA tensors only"):
        L.dequantize_awq(_awq())
    lin = L.PackedQuantLinear(_awq(k=16, n=16, g=16))
    with pytest.raises(ValueError, match="CUDA tensors only"):
        lin.forward(torch.zeros((1, 16), dtype=torch.bfloat16))


def test_any_linear_selects_fp8_variant_for_fp8_weights():
    # linear.rs:789-798
    w = torch.tensor([[0.5, -1.0], [1.5, 0.25]]).to(torch.float8_e4m3fn)
    assert L.AnyLinear.from_weight(w).variant == "Fp8"
    assert L.AnyLinear.from_weight(torch.zeros(2, 2)).variant == "Float"


def test_fp8_scale_inv_shapes():
    # linear.rs:115-138, weights.rs:220-225
    w = torch.zeros((4, 4)).to(torch.float8_e4m3fn)
    for s in (torch.ones(()), torch.ones(1), torch.ones(4), torch.ones(4, 1), torch.ones(2, 2)):
        grid, s_out, s_in = L.Fp8Linear(w, s)._grid()
        assert grid.shape == (s_out, s_in)
    with pytest.raises(ValueError, match="invalid FP8 scale_inv shape"):
        L.Fp8Linear(w, torch.ones(3))._grid()
    with pytest.raises(ValueError, match="invalid FP8 scale_inv rank"):
        L.Fp8Linear(w, torch.ones(1, 1, 1))._grid()
    with pytest.raises(ValueError, match="does not tile weight"):
        L.Fp8Linear(w, torch.ones(3, 2))._grid()


def test_mxfp4_and_gguf_constructor_checks():
    # mxfp4.rs:85-106, linear.rs:216-236
    with pytest.raises(ValueError, match="must be U8"):
        L.Mxfp4Linear(torch.zeros(32), torch.zeros(2, dtype=torch.uint8), None, 32, 2)
    with pytest.raises(ValueError, match="multiple of 32"):
        L.Mxfp4Linear(torch.zeros(32, dtype=torch.uint8), torch.zeros(2, dtype=torch.uint8), None, 48, 2)
    with pytest.raises(ValueError, match="don't match"):
        L.Mxfp4Linear(torch.zeros(31, dtype=torch.uint8), torch.zeros(2, dtype=torch.uint8), None, 32, 2)
    L.Mxfp4Linear(torch.zeros(32, dtype=torch.uint8), torch.zeros(2, dtype=torch.uint8), None, 32, 2)
    with pytest.raises(ValueError, match="multiple of the block size"):
        L.QLinear(F.GGML_Q4_K, torch.zeros(144, dtype=torch.uint8), 1, 128)
    with pytest.raises(ValueError, match="expected 288"):
        L.QLinear(F.GGML_Q4_K, torch.zeros(144, dtype=torch.uint8), 2, 256)
    with pytest.raises(ValueError, match="last dim"):
        L.QLinear(F.GGML_Q4_K, torch.zeros(288, dtype=torch.uint8), 2, 256).forward(torch.zeros(1, 128))


def test_pack_unpack_awq_roundtrip_and_order():
    v = np.arange(3 * 16).reshape(3, 16) % 16
    w = F.pack_awq(v)
    assert np.array_equal(F.unpack_awq(w), v)
    # slot k of a word holds column AWQ_PACK_ORDER[k] (awq.rs:23, 391-400)
    for k, col in enumerate(F.AWQ_PACK_ORDER):
        assert ((w[0, 0] >> (4 * k)) & 0xF) == v[0, col]


def test_oracle_gated_ffn_known_values():
    """act(gate) * up on a hand-built fused weight: identity gate rows, constant up rows."""
    import oracle
    inter, k = 4, 4
    w = np.zeros((2 * inter, k), np.float32)
    w[:inter] = np.eye(inter, dtype=np.float32)      # gate = x
    w[inter:] = 0.5 * np.eye(inter, dtype=np.float32)  # up = x / 2
    x = np.array([[0.0, 1.0, -2.0, 3.0]], np.float32)
    silu = oracle.gated_ffn(x, w, "silu")[0]
    want = [g / (1.0 + np.exp(-g)) * (g / 2) for g in x[0]]
    assert np.allclose(silu, want, rtol=1e-6, atol=1e-7)
    gelu = oracle.gated_ffn(x, w, "gelu_tanh")[0]
    want = [0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * (g / 2) for g in x[0]]
    assert np.allclose(gelu, want, rtol=1e-6, atol=1e-7)
    with pytest.raises(ValueError):
        oracle.gated_ffn(x, w, "relu")

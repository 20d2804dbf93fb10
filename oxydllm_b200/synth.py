"""Seeded synthetic inputs shaped like the five benchmark configurations.

No checkpoint or dataset is involved: weights and activations are drawn from
the stated distributions with ``numpy.random.default_rng(seed)`` and quantized
by the encoders in :mod:`formats`. All arrays are numpy; callers move them to
the GPU. bf16 tensors are returned as f32 arrays already rounded to bf16.
"""
from __future__ import annotations

import numpy as np

from . import formats as F


def bf16_round(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest-even bf16 -> f32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)


def activations(m: int, k: int, seed: int = 1) -> np.ndarray:
    """bf16-representable N(0, 1) activations ``[m, k]``."""
    return bf16_round(np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32))


def awq_layer(k: int = 4096, n: int = 14336, group_size: int = 128, seed: int = 0):
    """Config 1/2: uniform int4 weights and zeros, f16 scales |N(0, 0.02)|/7 + 1e-4."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    z = rng.integers(0, 16, size=(k // group_size, n), dtype=np.uint8)
    scales = (np.abs(rng.standard_normal((k // group_size, n)) * 0.02) / 7.0 + 1e-4).astype(np.float16)
    return F.pack_awq(q), F.pack_awq(z), scales


def gguf_layer(ggml_type: int, n: int = 4096, k: int = 4096, seed: int = 0) -> np.ndarray:
    """Config 0: W ~ N(0, 0.02) quantized to GGML blocks (this project's encoder)."""
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return F.GGML_QUANTIZE[ggml_type](w)


def fp8_layer(n: int = 14336, k: int = 4096, seed: int = 0, block: int = 128):
    """Config 3: W ~ N(0, 0.02), one f32 scale = blockmax/448 per 128x128 block."""
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return F.quantize_fp8_block(w, block)


def mxfp4_layer(n: int, k: int, seed: int = 0):
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return F.quantize_mxfp4(w)


def gptoss_moe(num_experts: int = 32, hidden: int = 2880, inter: int = 2880, tokens: int = 4096, seed: int = 0):
    """Config 4: MXFP4 experts from N(0, 0.02), bf16 biases N(0, 0.02), router logits N(0, 1), bf16 x N(0, 1)."""
    rng = np.random.default_rng(seed)
    out = {"gu_blocks": [], "gu_scales": [], "dn_blocks": [], "dn_scales": []}
    for _ in range(num_experts):
        b, s = F.quantize_mxfp4((rng.standard_normal((2 * inter, hidden)) * 0.02).astype(np.float32))
        out["gu_blocks"].append(b); out["gu_scales"].append(s)
        b, s = F.quantize_mxfp4((rng.standard_normal((hidden, inter)) * 0.02).astype(np.float32))
        out["dn_blocks"].append(b); out["dn_scales"].append(s)
    out = {k_: np.stack(v) for k_, v in out.items()}
    out["gu_bias"] = bf16_round((rng.standard_normal((num_experts, 2 * inter)) * 0.02).astype(np.float32))
    out["dn_bias"] = bf16_round((rng.standard_normal((num_experts, hidden)) * 0.02).astype(np.float32))
    out["logits"] = rng.standard_normal((tokens, num_experts)).astype(np.float32)
    out["x"] = bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32))
    return out

"""Host-side mirror of the reference's quantized-linear operator surface.

Same names, argument meaning and error behaviour as ``src/common/linear.rs``,
``awq.rs`` and ``mxfp4.rs`` of the reference, with torch CUDA tensors standing
in for candle tensors. Every ``forward`` runs a CUDA kernel of ``liboxq.so``
through the C ABI on the packed weights as stored (nothing is dequantized at
load, unlike the reference's non-Metal path, linear.rs:582-601); there is no
CPU path.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from .formats import GGML_BLOCK

_DT = {torch.float32: _lib.OXQ_F32, torch.float16: _lib.OXQ_F16, torch.bfloat16: _lib.OXQ_BF16}

#: Largest m handled by the decode GEMV kernels; larger batches go to the tensor-core GEMM.
GEMV_MAX_M = 32
#: The same for the GPTQ and 8-bit GEMVs (one 8-token chunk of the reference's batched GEMV, linear.rs:461-478).
PACKED_SIMT_GEMV_MAX_M = 8
# AWQ 4-bit layers whose shape the fused unpack + tcgen05 kernel serves (out_features % 128, in_features % 128,
# group size a power of two >= 64, 16-bit scales) leave the split-k GEMV at this batch: measured on a 4096 x 14336 layer the GEMV
# takes 24 us at 16 tokens and 47 us at 32, the fused kernel 28 to 31 us for any batch up to 128.
AWQ_FUSED_MIN_M = 17
AWQ_FUSED_SPLIT_K_TILES = 74  # at most this many 128-row tiles: the fused kernel runs two or more k splits per tile
# GPTQ 4-bit layers of such shapes: the GEMV takes 25 / 28 / 35 / 48 us at 1 / 2 / 4 / 8 tokens on the same layer, the fused
# kernel 30 us for any batch up to 64.
GPTQ_FUSED_MIN_M = 3


def _dt(t: torch.dtype) -> int:
    try:
        return _DT[t]
    except KeyError:
        raise ValueError(f"unsupported dtype {t}") from None


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # raw handle of torch's current stream on the current device, without building a Stream object
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("oxydllm_b200 operators run on CUDA tensors only (no CPU path)")


def _as_u32_words(t: torch.Tensor) -> torch.Tensor:
    """Packed tensors arrive as I32/U32/I64 (awq.rs:158-179); the kernels read 32-bit words."""
    if t.dtype == torch.int32:
        return t.contiguous()
    if t.dtype == torch.int64:
        return t.to(torch.int32).contiguous()  # wraps modulo 2^32 like `x as u32`
    if t.dtype == torch.uint32:
        return t.contiguous().view(torch.int32)
    raise ValueError(f"Unsupported AWQ packed tensor dtype {t.dtype} (expected I32/U32/I64)")


def _flatten_x(x: torch.Tensor, in_features: int, who: str):
    if x.shape[-1] != in_features:
        raise ValueError(f"{who}: input last dim {x.shape[-1]} != in_features {in_features}")
    if x.dim() == 2 and x.is_contiguous():  # the common case: nothing to reshape
        return x, x.shape[:1], x.shape[0]
    lead = x.shape[:-1]
    m = 1
    for d in lead:
        m *= d
    return x.reshape(m, in_features).contiguous(), lead, m


# ---------------------------------------------------------------------------
# AWQ / GPTQ containers (awq.rs:26-128)
@dataclass
class QuantWeight:
    """Packed-int weight triplet plus the metadata needed to dispatch its dequant (awq.rs:45-54)."""
    bits: int
    pack_dim: str       # "out" (AWQ) or "in" (GPTQ)
    pack_order: str     # "awq_interleaved" or "sequential"
    zero_point: str     # "signed", "plus_one" or "symmetric"
    qweight: torch.Tensor
    qzeros: Optional[torch.Tensor]
    scales: torch.Tensor

    @classmethod
    def new_awq(cls, bits: int, qweight, qzeros, scales) -> "QuantWeight":
        return cls(bits, "out", "awq_interleaved", "signed", qweight, qzeros, scales)

    @classmethod
    def new_gptq(cls, bits: int, sym: bool, qweight, qzeros, scales) -> "QuantWeight":
        return cls(bits, "in", "sequential", "symmetric" if sym else "plus_one", qweight, qzeros, scales)

    def pack_factor(self) -> int:
        return 32 // self.bits

    def in_features(self) -> int:
        if self.qweight.dim() != 2:
            raise ValueError("qweight must be 2D")
        d0 = self.qweight.shape[0]
        return d0 if self.pack_dim == "out" else d0 * self.pack_factor()

    def out_features(self) -> int:
        if self.scales.dim() != 2:
            raise ValueError("scales must be 2D")
        return self.scales.shape[1]

    def group_size(self) -> int:
        in_features = self.in_features()
        groups = self.scales.shape[0]
        if groups == 0:
            raise ValueError("quant scales has zero groups")
        if in_features % groups:
            raise ValueError(f"quant in_features ({in_features}) not divisible by scales groups ({groups})")
        return in_features // groups

    def to(self, device) -> "QuantWeight":
        return QuantWeight(self.bits, self.pack_dim, self.pack_order, self.zero_point, self.qweight.to(device),
                           None if self.qzeros is None else self.qzeros.to(device), self.scales.to(device))


AwqRawTensors = QuantWeight


def _check_awq_shapes(raw: QuantWeight):
    in_f, out_f, g = raw.in_features(), raw.out_features(), raw.group_size()
    groups, packed_out = in_f // g, out_f // 8
    if out_f % 8:
        raise ValueError(f"AWQ out_features ({out_f}) not divisible by pack factor 8")
    if raw.qweight.shape[1] != packed_out:
        raise ValueError(f"AWQ qweight dim1 ({raw.qweight.shape[1]}) != out_features/8 ({packed_out})")
    if raw.qzeros is None:
        raise ValueError("AWQ dequantize: qzeros tensor missing")
    if tuple(raw.qzeros.shape) != (groups, packed_out):
        raise ValueError(f"AWQ qzeros shape {list(raw.qzeros.shape)} != [{groups}, {packed_out}]")
    if tuple(raw.scales.shape) != (groups, out_f):
        raise ValueError(f"AWQ scales shape {list(raw.scales.shape)} != [{groups}, {out_f}]")
    return in_f, out_f, g


def dequantize_awq(raw: QuantWeight, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``dequantize_awq`` (awq.rs:325-440): dense ``[out, in]`` weight, bit-exact, on the GPU."""
    if raw.bits != 4:
        raise ValueError(f"AWQ dequantize: only 4-bit supported, got {raw.bits}")
    in_f, out_f, g = _check_awq_shapes(raw)
    _require_cuda(raw.qweight, raw.qzeros, raw.scales)
    qw, qz, sc = _as_u32_words(raw.qweight), _as_u32_words(raw.qzeros), raw.scales.contiguous()
    out = torch.empty((out_f, in_f), dtype=out_dtype, device=qw.device)
    _lib.call("oxq_awq_dequant", _p(qw), _p(qz), _p(sc), _dt(sc.dtype), _p(out), _dt(out_dtype), in_f, out_f, g,
              _stream())
    return out


def dequantize_gptq(raw: QuantWeight, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``dequantize_gptq`` (awq.rs:442-559): dense ``[out, in]`` weight, bit-exact, on the GPU."""
    if raw.pack_dim != "in" or raw.pack_order != "sequential":
        raise ValueError(f"dequantize_gptq: expected PackDim::In + Sequential, got {raw.pack_dim}/{raw.pack_order}")
    if raw.bits not in (4, 8):
        raise ValueError(f"dequantize_gptq: only 4/8-bit supported, got {raw.bits}")
    pf = raw.pack_factor()
    in_f, out_f, g = raw.in_features(), raw.out_features(), raw.group_size()
    groups = in_f // g
    if tuple(raw.qweight.shape) != (in_f // pf, out_f):
        raise ValueError(f"GPTQ qweight shape {list(raw.qweight.shape)} != [{in_f // pf}, {out_f}]")
    if tuple(raw.scales.shape) != (groups, out_f):
        raise ValueError(f"GPTQ scales shape {list(raw.scales.shape)} != [{groups}, {out_f}]")
    if out_f % pf:
        raise ValueError(f"GPTQ out_features {out_f} not divisible by pack_factor {pf}")
    qz = None
    if raw.qzeros is not None:
        if tuple(raw.qzeros.shape) != (groups, out_f // pf):
            raise ValueError(f"GPTQ qzeros shape {list(raw.qzeros.shape)} != [{groups}, {out_f // pf}]")
        qz = _as_u32_words(raw.qzeros)
    _require_cuda(raw.qweight, raw.scales)
    qw, sc = _as_u32_words(raw.qweight), raw.scales.contiguous()
    sym = raw.qzeros is None or raw.zero_point == "symmetric"
    out = torch.empty((out_f, in_f), dtype=out_dtype, device=qw.device)
    _lib.call("oxq_gptq_dequant", _p(qw), _p(qz), _p(sc), _dt(sc.dtype), _p(out), _dt(out_dtype), in_f, out_f, g,
              raw.bits, int(sym), _stream())
    return out


def dequantize_w8a16(raw: QuantWeight, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``dequantize_w8`` (metal_ops.rs, quant_kernels.metal:335-356): dense ``[out, in]`` weight of the 8-bit AWQ
    layout (``qweight [in, out/4]``, byte c of word j = out column ``4 j + c``), bit-exact, on the GPU."""
    if raw.bits != 8 or raw.pack_dim != "out":
        raise ValueError(f"dequantize_w8a16: expected 8-bit PackDim::Out, got {raw.bits}-bit {raw.pack_dim}")
    if raw.qzeros is None:
        raise ValueError("W8A16 dequantize: qzeros tensor missing")
    in_f, out_f, g = raw.in_features(), raw.out_features(), raw.group_size()
    groups = in_f // g
    if out_f % 4 or tuple(raw.qweight.shape) != (in_f, out_f // 4) or tuple(raw.qzeros.shape) != (groups, out_f // 4):
        raise ValueError(f"W8A16 qweight/qzeros shapes {list(raw.qweight.shape)}/{list(raw.qzeros.shape)} do not match "
                         f"[{in_f}, {out_f // 4}] / [{groups}, {out_f // 4}]")
    _require_cuda(raw.qweight, raw.qzeros, raw.scales)
    qw, qz, sc = _as_u32_words(raw.qweight), _as_u32_words(raw.qzeros), raw.scales.contiguous()
    out = torch.empty((out_f, in_f), dtype=out_dtype, device=qw.device)
    _lib.call("oxq_w8a16_dequant", _p(qw), _p(qz), _p(sc), _dt(sc.dtype), _p(out), _dt(out_dtype), in_f, out_f, g, _stream())
    return out


def dequantize_quant(raw: QuantWeight, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``dequantize_quant`` (awq.rs:592-597)."""
    if raw.pack_dim == "out":
        return dequantize_awq(raw, out_dtype) if raw.bits == 4 else dequantize_w8a16(raw, out_dtype)
    return dequantize_gptq(raw, out_dtype)


# ---------------------------------------------------------------------------
class Linear:
    """Dense ``x @ W^T + b`` (linear.rs:35-79); the Float arm of :class:`AnyLinear`."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight, self.bias = weight, bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x, self.weight.to(x.dtype), self.bias)


class PackedQuantLinear:
    """Resident packed-int linear layer (``PackedQuantLinear``, linear.rs:403-534): AWQ (``pack_dim="out"``) or
    GPTQ (``pack_dim="in"``), 4 or 8 bits, on the packed tensors as stored.

    ``forward`` keeps the reference's dispatch shape: decode-sized batches go to the GEMV kernels (the
    reference chunks them by 8 tokens, linear.rs:450-480), larger ones to the tensor-core GEMM on slabs of the
    dequantized weight (linear.rs:494-524). Scales stay in their stored dtype and are widened to f32 inside
    the kernels (the CPU convention, awq.rs:362-367); pass ``scales.to(dtype)`` yourself to get the Metal
    resident convention (linear.rs:437).
    """

    def __init__(self, raw: QuantWeight, bias: Optional[torch.Tensor] = None, dtype: torch.dtype = torch.bfloat16):
        if raw.bits not in (4, 8):
            raise ValueError(f"PackedQuantLinear: bits must be 4 or 8, got {raw.bits}")
        self.bits, self.pack_dim = raw.bits, raw.pack_dim
        self.sym = raw.pack_dim == "in" and (raw.qzeros is None or raw.zero_point == "symmetric")
        if raw.qzeros is None and not self.sym:
            raise ValueError("PackedQuantLinear: qzeros missing")
        pf = raw.pack_factor()
        if raw.pack_dim == "out" and raw.bits == 4:
            self.in_features, self.out_features, self.group_size = _check_awq_shapes(raw)
        else:
            self.in_features, self.out_features, self.group_size = raw.in_features(), raw.out_features(), raw.group_size()
            groups = self.in_features // self.group_size
            want_qw = (self.in_features, self.out_features // pf) if raw.pack_dim == "out" else (self.in_features // pf, self.out_features)
            if self.out_features % pf or tuple(raw.qweight.shape) != want_qw:
                raise ValueError(f"PackedQuantLinear: qweight shape {list(raw.qweight.shape)} != {list(want_qw)}")
            if raw.qzeros is not None and tuple(raw.qzeros.shape) != (groups, self.out_features // pf):
                raise ValueError(f"PackedQuantLinear: qzeros shape {list(raw.qzeros.shape)} != [{groups}, {self.out_features // pf}]")
            if tuple(raw.scales.shape) != (groups, self.out_features):
                raise ValueError(f"PackedQuantLinear: scales out_features {raw.scales.shape[1]} != derived {self.out_features}")
        self.qweight = _as_u32_words(raw.qweight)
        self.qzeros = None if raw.qzeros is None else _as_u32_words(raw.qzeros)
        self.scales = raw.scales.contiguous()
        self.bias = None if bias is None else bias.contiguous()
        self.dtype = dtype
        self._resident = all(t is None or t.is_cuda for t in (self.qweight, self.qzeros, self.scales, self.bias))
        # constant arguments of the GEMV call, converted once
        b = self.bias
        self._const = (_p(self.qweight), _p(self.qzeros), _p(self.scales), _dt(self.scales.dtype), _p(b),
                       _dt(b.dtype) if b is not None else 0)

    def gemv_max_m(self) -> int:
        """Largest batch the decode kernels take before the tensor-core GEMM is the better tool: 32 for the
        4-bit AWQ tensor-core GEMV (16 where the fused unpack + tcgen05 kernel takes over), 8 (one chunk of the
        reference's batched GEMV) for GPTQ and 8-bit (2 for 4-bit GPTQ shapes the fused kernel serves)."""
        fused = (self.bits == 4 and self.out_features % 128 == 0 and self.in_features % 128 == 0 and self.group_size % 64 == 0
                 and self.group_size & (self.group_size - 1) == 0 and self.scales.dtype in (torch.float16, torch.bfloat16))
        if self.pack_dim == "out" and self.bits == 4:
            if fused and self.out_features // 128 <= AWQ_FUSED_SPLIT_K_TILES:
                return 8  # narrow layer: the fused kernel splits k over the SMs (4096 x 4096: 14 us at 16 tokens, GEMV 23 us)
            return AWQ_FUSED_MIN_M - 1 if fused else GEMV_MAX_M
        if fused:
            return GPTQ_FUSED_MIN_M - 1
        return PACKED_SIMT_GEMV_MAX_M

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out``: optional preallocated contiguous ``[m, out_features]`` result tensor of x's dtype and device."""
        x2, lead, m = _flatten_x(x, self.in_features, "PackedQuantLinear")
        if not (self._resident and x2.is_cuda):
            _require_cuda(x2, self.qweight, self.qzeros, self.scales, self.bias)
        if out is None:
            y = torch.empty((m, self.out_features), dtype=x2.dtype, device=x2.device)
        else:
            if (out.shape != (m, self.out_features) or out.dtype != x2.dtype or out.device != x2.device
                    or not out.is_contiguous()):
                raise ValueError(f"PackedQuantLinear: out must be a contiguous [{m}, {self.out_features}] {x2.dtype} tensor "
                                 f"on {x2.device}")
            y = out
        if m == 0:
            return y.reshape(*lead, self.out_features)
        if m <= self.gemv_max_m():
            self._gemv(x2, y, m)
        else:
            from . import gemm
            if self.pack_dim == "out" and self.bits == 4:
                gemm.awq_matmul(self, x2, y)
            elif self.pack_dim == "out":
                gemm.w8a16_matmul(self, x2, y)
            else:
                gemm.gptq_matmul(self, x2, y, self.bias)
        return y.reshape(*lead, self.out_features)

    def _gemv(self, x2, y, m):
        qw, qz, sc, sc_dt, b, b_dt = self._const
        if self.pack_dim == "out" and self.bits == 4:
            _lib.call("oxq_awq_gemv", _p(x2), _dt(x2.dtype), qw, qz, sc, sc_dt, b, b_dt, _p(y), _dt(y.dtype), m,
                      self.in_features, self.out_features, self.group_size, _stream())
        elif self.pack_dim == "out":
            _lib.call("oxq_w8a16_gemv", _p(x2), _dt(x2.dtype), qw, qz, sc, sc_dt, b, b_dt, _p(y), _dt(y.dtype), m,
                      self.in_features, self.out_features, self.group_size, _stream())
        else:
            _lib.call("oxq_gptq_gemv", _p(x2), _dt(x2.dtype), qw, qz, sc, sc_dt, b, b_dt, _p(y), _dt(y.dtype), m,
                      self.in_features, self.out_features, self.group_size, self.bits, int(self.sym), _stream())

    # the attributes gemm.gptq_matmul reads from a QuantWeight
    def pack_factor(self) -> int:
        return 32 // self.bits

    @property
    def zero_point(self) -> str:
        return "symmetric" if self.sym else ("plus_one" if self.pack_dim == "in" else "signed")


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}


class GatedFfnProjection:
    """Fused gate+up projection and gated activation of ``FeedForward`` (ffn.rs:235-254, 385-470).

    ``gate_up`` is the AWQ linear over ``concat_awq_along_out([gate_proj, up_proj])`` (out features
    ``2 * intermediate``); ``forward`` returns ``act(gate) * up`` with ``act`` SiLU or tanh-GeLU, i.e.
    what the reference's ``GateUpProjection::Fused`` branch feeds to ``down_proj``.
    """

    def __init__(self, gate_up: "PackedQuantLinear", activation: str = "silu"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"GatedFfnProjection: unknown activation {activation!r} (silu, gelu_tanh)")
        if gate_up.out_features % 16:
            raise ValueError(f"GatedFfnProjection: fused out_features {gate_up.out_features} must be 2 * intermediate, "
                             "intermediate a multiple of 8")
        if gate_up.bias is not None:
            raise ValueError("GatedFfnProjection: the fused gate/up projection carries no bias")
        self.gate_up, self.activation = gate_up, activation
        self.intermediate = gate_up.out_features // 2

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lin = self.gate_up
        x2, lead, m = _flatten_x(x, lin.in_features, "GatedFfnProjection")
        _require_cuda(x2, lin.qweight, lin.qzeros, lin.scales)
        if x2.dtype != torch.bfloat16:
            raise ValueError("GatedFfnProjection: activations must be bf16")
        y = torch.empty((m, self.intermediate), dtype=x2.dtype, device=x2.device)
        if m:
            from . import gemm
            gemm.awq_ffn_gate_up(lin, x2, y, ACTIVATIONS[self.activation])
        return y.reshape(*lead, self.intermediate)


class Fp8Linear:
    """``Fp8Linear`` (linear.rs:81-146): E4M3 weight ``[out, in]`` + optional f32 ``scale_inv``.

    ``scale_inv`` may be rank 0, rank 1 (``[out]`` or ``[1]``) or a 2-D grid
    tiling the weight evenly (weights.rs:207-234); anything else raises the
    reference's message at ``forward`` time (linear.rs:115-138).
    """

    def __init__(self, weight: torch.Tensor, scale_inv: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None):
        if weight.dtype == torch.float8_e4m3fn:
            weight = weight.view(torch.uint8)
        if weight.dtype != torch.uint8 or weight.dim() != 2:
            raise ValueError("Fp8Linear: weight must be a 2-D F8E4M3 tensor")
        self.weight = weight.contiguous()
        self.scale_inv = scale_inv
        self.bias = None if bias is None else bias.contiguous()
        self.out_features, self.in_features = weight.shape

    def _grid(self):
        s = self.scale_inv
        if s is None:
            return None, 0, 0
        s = s.to(torch.float32)
        if s.dim() == 2:
            pass
        elif s.dim() == 1:
            if s.shape[0] == self.out_features:
                s = s.reshape(self.out_features, 1)
            elif s.shape[0] == 1:
                s = s.reshape(1, 1)
            else:
                raise ValueError(f"invalid FP8 scale_inv shape {list(s.shape)}: expected [out_features, 1], "
                                 "[out_features], or scalar")
        elif s.dim() == 0:
            s = s.reshape(1, 1)
        else:
            raise ValueError(f"invalid FP8 scale_inv rank {s.dim()}: expected rank 0, 1, or 2")
        s_out, s_in = s.shape
        if s_out == 0 or s_in == 0 or self.out_features % s_out or self.in_features % s_in:
            raise ValueError(f"block-wise FP8 weight_scale_inv [{s_out}, {s_in}] does not tile weight "
                             f"[{self.out_features}, {self.in_features}] evenly")
        return s.contiguous(), s_out, s_in

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """The per-forward dequant of the reference (linear.rs:96-141), bit-exact."""
        s, s_out, s_in = self._grid()
        _require_cuda(self.weight)
        out = torch.empty((self.out_features, self.in_features), dtype=out_dtype, device=self.weight.device)
        _lib.call("oxq_fp8_dequant", _p(self.weight), _p(s), s_out, s_in, _p(out), _dt(out_dtype), self.out_features,
                  self.in_features, _stream())
        return out

    def gemv_max_m(self, s_out: int, s_in: int) -> int:
        """Largest batch for the decode GEMV: 16 where the fused widen + tcgen05 kernel serves the layer (out_features % 128,
        in_features % 128, scale blocks of a multiple of 128 rows and 64 columns; 24 us for up to 32 tokens on a
        14336 x 4096 layer against 25 / 45 us for the GEMV at 16 / 32), else 32."""
        n, k = self.out_features, self.in_features
        bo, bi = (n // s_out, k // s_in) if s_out and s_in else (n, k)
        fused = n % 128 == 0 and k % 128 == 0 and bo % 128 == 0 and bi % 64 == 0
        return AWQ_FUSED_MIN_M - 1 if fused else GEMV_MAX_M

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        s, s_out, s_in = self._grid()
        x2, lead, m = _flatten_x(x, self.in_features, "Fp8Linear")
        _require_cuda(x2, self.weight, self.bias)
        y = torch.empty((m, self.out_features), dtype=x2.dtype, device=x2.device)
        if m == 0:
            return y.reshape(*lead, self.out_features)
        if m <= self.gemv_max_m(s_out, s_in):
            b = self.bias
            _lib.call("oxq_fp8_gemv", _p(x2), _dt(x2.dtype), _p(self.weight), _p(s), s_out, s_in, _p(b),
                      _dt(b.dtype) if b is not None else 0, _p(y), _dt(y.dtype), m, self.in_features,
                      self.out_features, _stream())
        else:
            from . import gemm
            gemm.fp8_matmul(self, s, s_out, s_in, x2, y)
        return y.reshape(*lead, self.out_features)


class QLinear:
    """``QLinear`` (linear.rs:179-394) over raw GGML blocks ``[out, in]``, rows contiguous.

    ``from_blocks`` plays the role of ``from_arc_with_bias``: the byte count is
    checked against the shape and block layout as ``GgufFastPath::build`` does
    (linear.rs:216-236).
    """

    def __init__(self, ggml_type: int, blocks: torch.Tensor, out_features: int, in_features: int,
                 bias: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16):
        if ggml_type not in GGML_BLOCK:
            raise ValueError(f"unsupported GGML type {ggml_type}")
        bel, bby = GGML_BLOCK[ggml_type]
        if in_features % bel:
            raise ValueError(f"GGUF in_features {in_features} is not a multiple of the block size {bel}")
        expected = out_features * (in_features // bel) * bby
        if blocks.dtype != torch.uint8 or blocks.numel() != expected:
            raise ValueError(f"GGUF fast path: got {blocks.numel()} bytes, expected {expected} for shape "
                             f"[{out_features}, {in_features}] type {ggml_type}")
        self.ggml_type, self.blocks = ggml_type, blocks.contiguous().reshape(-1)
        self.out_features, self.in_features = out_features, in_features
        self.bias = None if bias is None else bias.contiguous()
        self.out_dtype = out_dtype

    from_blocks = classmethod(lambda cls, *a, **k: cls(*a, **k))

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _require_cuda(self.blocks)
        out = torch.empty((self.out_features, self.in_features), dtype=out_dtype, device=self.blocks.device)
        _lib.call("oxq_gguf_dequant", self.ggml_type, _p(self.blocks), _p(out), _dt(out_dtype), self.out_features,
                  self.in_features, _stream())
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead, m = _flatten_x(x, self.in_features, "QLinear")
        _require_cuda(x2, self.blocks, self.bias)
        y = torch.empty((m, self.out_features), dtype=self.out_dtype, device=x2.device)
        if m == 0:
            return y.reshape(*lead, self.out_features)
        if m <= GEMV_MAX_M:
            b = self.bias
            _lib.call("oxq_gguf_gemv", self.ggml_type, _p(x2), _dt(x2.dtype), _p(self.blocks), _p(b),
                      _dt(b.dtype) if b is not None else 0, _p(y), _dt(y.dtype), m, self.in_features,
                      self.out_features, _stream())
        else:
            from . import gemm
            gemm.gguf_matmul(self, x2, y)
        return y.reshape(*lead, self.out_features)


class Mxfp4Linear:
    """``Mxfp4Linear`` (mxfp4.rs:67-169): ``y = x @ W^T + bias`` with W kept packed."""

    def __init__(self, blocks: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], in_features: int,
                 out_features: int):
        if blocks.dtype != torch.uint8 or scales.dtype != torch.uint8:
            raise ValueError(f"Mxfp4Linear: blocks/scales must be U8, got {blocks.dtype}/{scales.dtype}")
        if in_features % 32:
            raise ValueError(f"Mxfp4Linear: in_features {in_features} must be a multiple of 32")
        nb = in_features // 32
        if blocks.numel() != out_features * nb * 16 or scales.numel() != out_features * nb:
            raise ValueError(f"Mxfp4Linear: blocks {blocks.numel()} / scales {scales.numel()} elements don't match "
                             f"[{out_features}, {in_features}]")
        self.blocks = blocks.contiguous().reshape(-1)
        self.scales = scales.contiguous().reshape(-1)
        self.bias = None if bias is None else bias.contiguous()
        self.in_features, self.out_features = in_features, out_features

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _require_cuda(self.blocks)
        out = torch.empty((self.out_features, self.in_features), dtype=out_dtype, device=self.blocks.device)
        _lib.call("oxq_mxfp4_dequant", _p(self.blocks), _p(self.scales), _p(out), _dt(out_dtype), self.out_features,
                  self.in_features, _stream())
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead, m = _flatten_x(x, self.in_features, "Mxfp4Linear")
        _require_cuda(x2, self.blocks, self.scales, self.bias)
        y = torch.empty((m, self.out_features), dtype=x2.dtype, device=x2.device)
        if m == 0:
            return y.reshape(*lead, self.out_features)
        if m <= GEMV_MAX_M:
            b = self.bias
            _lib.call("oxq_mxfp4_gemv", _p(x2), _dt(x2.dtype), _p(self.blocks), _p(self.scales), _p(b),
                      _dt(b.dtype) if b is not None else 0, _p(y), _dt(y.dtype), m, self.in_features,
                      self.out_features, _stream())
        else:
            from . import gemm
            gemm.mxfp4_matmul(self, x2, y)
        return y.reshape(*lead, self.out_features)


class AnyLinear:
    """``AnyLinear`` (linear.rs:536-612): one of Float / Fp8 / Quantized / PackedQuant."""

    def __init__(self, inner):
        self.inner = inner

    @classmethod
    def from_weight(cls, weight, bias=None):
        return cls.from_weight_with_scale_inv(weight, None, bias)

    @classmethod
    def from_weight_with_scale_inv(cls, weight, scale_inv=None, bias=None):
        """FP8 variant iff the weight dtype is F8E4M3 (linear.rs:549-559)."""
        if weight.dtype == torch.float8_e4m3fn:
            return cls(Fp8Linear(weight, scale_inv, bias))
        return cls(Linear(weight, bias))

    @classmethod
    def from_awq(cls, raw: QuantWeight, bias=None, device="cuda", dtype=torch.bfloat16):
        """Always resident-packed here (the reference does this on Metal only, linear.rs:561-580)."""
        return cls(PackedQuantLinear(raw.to(device), bias, dtype))

    @classmethod
    def from_quant(cls, raw: QuantWeight, bias=None, device="cuda", dtype=torch.bfloat16):
        """AWQ and GPTQ, 4 or 8 bits, all stay packed and resident (the reference keeps them packed on Metal,
        linear.rs:561-580, and dequantizes at load elsewhere, linear.rs:582-601)."""
        return cls(PackedQuantLinear(raw.to(device), bias, dtype))

    @classmethod
    def from_gguf(cls, ggml_type, blocks, out_features, in_features, bias=None, out_dtype=torch.bfloat16):
        return cls(QLinear(ggml_type, blocks, out_features, in_features, bias, out_dtype))

    @property
    def variant(self) -> str:
        return {Linear: "Float", Fp8Linear: "Fp8", QLinear: "Quantized", PackedQuantLinear: "PackedQuant"}[
            type(self.inner)]

    def forward(self, x):
        return self.inner.forward(x)

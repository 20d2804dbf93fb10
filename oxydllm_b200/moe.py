"""GPT-OSS MoE feed-forward layer: host-side mirror of ``MoeFeedForward`` with ``MoeExpert::GptOss``
experts (moe.rs:366-450 loader layout, 466-499 routing, 563-607 dispatch, 152-173 expert math).

The router is a dense linear (with bias) as in the reference (moe.rs:378-380); its logits feed
``oxq_gptoss_moe_forward``, which does routing, dispatch, both expert GEMMs, the clamped SwiGLU and
the weighted combine on the device. ``expert_range`` restricts a replica to its local experts.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .linear import _dt, _p, _stream

_workspaces: dict = {}


def _workspace(nbytes: int, device) -> torch.Tensor:
    idx = torch.device(device).index
    key = torch.cuda.current_device() if idx is None else idx
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def route(logits: torch.Tensor, top_k: int, norm_topk: bool = True):
    """softmax -> top-k -> renormalise on the device; returns (top_idx int32, top_w f32)."""
    logits = logits.to(torch.float32).contiguous()
    t, e = logits.shape
    idx = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    _lib.call("oxq_moe_route", _p(logits), t, e, top_k, int(norm_topk), _p(idx), _p(w), _stream())
    return idx, w


def combine(rows: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor, pos: torch.Tensor, num_experts: int,
            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``out[t] = sum_s top_w[t, s] * rows[pos[t, s]]`` in ascending expert order (moe.rs:593-605), on the device."""
    t, k = top_idx.shape
    hidden = rows.shape[1]
    out = torch.empty((t, hidden), dtype=out_dtype or rows.dtype, device=rows.device)
    if t:
        _lib.call("oxq_moe_combine", _p(rows.contiguous()), _p(top_idx.to(torch.int32).contiguous()),
                  _p(top_w.to(torch.float32).contiguous()), _p(pos.to(torch.int32).contiguous()), t, k, hidden, num_experts,
                  _p(out), _dt(out.dtype), _stream())
    return out


def dispatch_plan(top_idx: torch.Tensor, num_experts: int):
    """Pairs sorted by expert id (stable) on the device: ``(counts i32 [E], perm i32 [pairs], inv i32 [pairs])``."""
    idx = top_idx.to(torch.int32).contiguous()
    pairs = idx.numel()
    counts = torch.empty(num_experts, dtype=torch.int32, device=idx.device)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=idx.device)
    perm = torch.empty(pairs, dtype=torch.int32, device=idx.device)
    inv = torch.empty(pairs, dtype=torch.int32, device=idx.device)
    _lib.call("oxq_moe_dispatch_plan", _p(idx), pairs, num_experts, _p(counts), _p(offsets), _p(perm), _p(inv), _stream())
    return counts, perm, inv


def gather_rows(x: torch.Tensor, perm: torch.Tensor, top_k: int) -> torch.Tensor:
    """``out[i] = x[perm[i] // top_k]``: the rows of a dispatch in send order (bf16, on the device)."""
    out = torch.empty((perm.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    if perm.numel():
        _lib.call("oxq_moe_gather_rows", _p(x.contiguous()), _p(perm), perm.numel(), top_k, x.shape[1], _p(out), _stream())
    return out


def expand_ids(counts: torch.Tensor, n_local: int, lo: int, total: int) -> torch.Tensor:
    """Expert ids of rows received in groups (source rank major, local expert minor) from the groups' sizes."""
    ids = torch.empty(total, dtype=torch.int32, device=counts.device)
    if total:
        _lib.call("oxq_moe_expand_ids", _p(counts), counts.numel(), n_local, lo, _p(ids), _stream())
    return ids


class GptOssMoe:
    """``gu_*``: fused gate/up projection (even rows gate, odd rows up), ``dn_*``: down projection, per expert."""

    def __init__(self, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias, hidden: int, inter: int,
                 top_k: int = 4, swiglu_limit: float = 7.0, norm_topk: bool = True,
                 router_weight: Optional[torch.Tensor] = None, router_bias: Optional[torch.Tensor] = None):
        e = gu_bias.shape[0]
        for name, t in (("gu_blocks", gu_blocks), ("gu_scales", gu_scales), ("dn_blocks", dn_blocks), ("dn_scales", dn_scales)):
            if t.dtype != torch.uint8:
                raise ValueError(f"Mxfp4Linear: blocks/scales must be U8, got {t.dtype} for {name}")
        if hidden % 32 or inter % 32:
            raise ValueError(f"Mxfp4Linear: in_features ({hidden}, {inter}) must be a multiple of 32")
        if gu_blocks.numel() != e * 2 * inter * (hidden // 32) * 16 or gu_scales.numel() != e * 2 * inter * (hidden // 32):
            raise ValueError("GPT-OSS gate_up blocks/scales elements don't match [E, 2*inter, hidden]")
        if dn_blocks.numel() != e * hidden * (inter // 32) * 16 or dn_scales.numel() != e * hidden * (inter // 32):
            raise ValueError("GPT-OSS down blocks/scales elements don't match [E, hidden, inter]")
        self.num_experts, self.hidden, self.inter, self.top_k = e, hidden, inter, top_k
        self.limit, self.norm_topk = float(swiglu_limit), norm_topk
        self.gu_blocks, self.gu_scales = gu_blocks.contiguous(), gu_scales.contiguous()
        self.dn_blocks, self.dn_scales = dn_blocks.contiguous(), dn_scales.contiguous()
        self.gu_bias, self.dn_bias = gu_bias.contiguous(), dn_bias.contiguous()
        if self.gu_bias.dtype != self.dn_bias.dtype:
            raise ValueError("expert biases must share one dtype")
        self.router_weight, self.router_bias = router_weight, router_bias

    def forward(self, x: torch.Tensor, expert_range=None) -> torch.Tensor:
        if self.router_weight is None:
            raise ValueError("GptOssMoe.forward needs router weights; use forward_with_logits")
        flat = x.reshape(-1, self.hidden)
        logits = torch.nn.functional.linear(flat, self.router_weight.to(flat.dtype),
                                            None if self.router_bias is None else self.router_bias.to(flat.dtype))
        return self.forward_with_logits(x, logits, expert_range)

    def forward_with_logits(self, x: torch.Tensor, logits: torch.Tensor, expert_range=None) -> torch.Tensor:
        if x.shape[-1] != self.hidden:
            raise ValueError(f"Mxfp4Linear: x last dim {x.shape[-1]} != in_features {self.hidden}")
        if not x.is_cuda:
            raise ValueError("oxydllm_b200 operators run on CUDA tensors only (no CPU path)")
        shape = x.shape
        x2 = x.reshape(-1, self.hidden).contiguous()
        t = x2.shape[0]
        logits = logits.reshape(t, self.num_experts).to(torch.float32).contiguous()
        lo, hi = (0, self.num_experts) if expert_range is None else expert_range
        out = torch.empty_like(x2)
        if t == 0:
            return out.reshape(shape)
        need = int(_lib.load().oxq_gptoss_moe_workspace_bytes(t, self.top_k, hi - lo, self.hidden, self.inter))
        ws = _workspace(need, x2.device)
        _lib.call("oxq_gptoss_moe_forward", _p(x2), _dt(x2.dtype), _p(logits), t, self.num_experts, self.top_k,
                  int(self.norm_topk), self.hidden, self.inter, _p(self.gu_blocks), _p(self.gu_scales), _p(self.gu_bias),
                  _p(self.dn_blocks), _p(self.dn_scales), _p(self.dn_bias), _dt(self.gu_bias.dtype),
                  ctypes.c_float(self.limit), lo, hi, _p(out), _dt(out.dtype), _p(ws), ws.numel(), _stream())
        self.last_workspace = ws
        return out.reshape(shape)

    def forward_experts(self, rows: torch.Tensor, expert_ids: torch.Tensor, expert_range=None) -> torch.Tensor:
        """Each row through the expert it is already assigned to, weight one (the owner side of expert parallelism)."""
        if rows.shape[-1] != self.hidden:
            raise ValueError(f"Mxfp4Linear: x last dim {rows.shape[-1]} != in_features {self.hidden}")
        if not rows.is_cuda:
            raise ValueError("oxydllm_b200 operators run on CUDA tensors only (no CPU path)")
        rows = rows.contiguous()
        ids = expert_ids.to(torch.int32).contiguous()
        r = rows.shape[0]
        out = torch.empty_like(rows)
        if r == 0:
            return out
        lo, hi = (0, self.num_experts) if expert_range is None else expert_range
        need = int(_lib.load().oxq_gptoss_moe_workspace_bytes(r, 1, hi - lo, self.hidden, self.inter))
        ws = _workspace(need, rows.device)
        _lib.call("oxq_gptoss_experts_forward", _p(rows), _dt(rows.dtype), _p(ids), r, self.num_experts, self.hidden, self.inter,
                  _p(self.gu_blocks), _p(self.gu_scales), _p(self.gu_bias), _p(self.dn_blocks), _p(self.dn_scales),
                  _p(self.dn_bias), _dt(self.gu_bias.dtype), ctypes.c_float(self.limit), lo, hi, _p(out), _dt(out.dtype),
                  _p(ws), ws.numel(), _stream())
        self.last_workspace = ws
        return out

    def check(self):
        """Synchronise and raise if a tensor-core kernel of the last forward gave up on a wait."""
        _lib.call("oxq_gemm_check", _p(self.last_workspace), _stream())

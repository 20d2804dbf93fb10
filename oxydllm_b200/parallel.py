"""Multi-GPU forms of the two operators that shard naturally (one process per GPU, torch.distributed).

* Tensor parallel column split of a packed linear + all-gather of the outputs. AWQ packs 8
  consecutive out columns per word, so any split at a multiple of 8 columns is a pure slice of
  ``qweight[:, a/8:b/8]``, ``qzeros[:, a/8:b/8]``, ``scales[:, a:b]`` -- the property
  ``concat_awq_along_out`` relies on (awq.rs:256-323). The reference itself has no multi-GPU
  execution; parity is "sharded result == unsharded result".
* Expert parallel GPT-OSS MoE with all-to-all token dispatch and combine: experts are independent
  and the combine is a sum (moe.rs:593-605). Tokens start data-parallel; each rank routes its own
  tokens, sends every (token, slot) row to the rank that owns the expert, runs its local experts
  on what it received, sends the rows back, and the owner of the token adds them in ascending
  expert order.

The index arithmetic lives in plain functions (``column_shard``, ``expert_shard``,
``plan_dispatch``, ``combine_rows``) so that it can be exercised with gloo on CPU; the classes bind
them to the CUDA operators.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------- sharding arithmetic
def column_shard(n: int, world: int, rank: int, multiple: int = 8) -> tuple[int, int]:
    """Out-column range ``[a, b)`` of ``rank``: near-equal shards whose bounds are multiples of ``multiple``."""
    if n % multiple:
        raise ValueError(f"out_features {n} not divisible by {multiple}")
    units = n // multiple
    base, rem = divmod(units, world)
    a = rank * base + min(rank, rem)
    b = a + base + (1 if rank < rem else 0)
    return a * multiple, b * multiple


def expert_shard(num_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous expert range ``[lo, hi)`` owned by ``rank``."""
    base, rem = divmod(num_experts, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def owner_of_expert(expert: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    """Rank that owns each expert id under :func:`expert_shard`."""
    base, rem = divmod(num_experts, world)
    cut = rem * (base + 1)
    if base == 0:
        return expert.clone()
    return torch.where(expert < cut, expert // (base + 1), rem + (expert - cut) // base)


def plan_dispatch(top_idx: torch.Tensor, num_experts: int, world: int):
    """Order in which this rank's (token, slot) pairs are sent: grouped by destination rank, pair order kept.

    Returns ``(send_order, send_counts)``: ``send_order[i]`` is the flat pair index (token * k + slot)
    of the i-th row sent, ``send_counts[r]`` the number of rows going to rank ``r``.
    """
    flat = top_idx.reshape(-1).to(torch.int64)
    dest = owner_of_expert(flat, num_experts, world)
    send_order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)
    return send_order, send_counts


def plan_dispatch_by_expert(top_idx: torch.Tensor, num_experts: int):
    """The same order refined: pairs sorted by expert id (stable), which under the contiguous :func:`expert_shard` also groups
    them by destination rank. Returns ``(send_order, per_expert)`` with ``per_expert[e]`` the number of rows for expert ``e``:
    exchanging these counts tells every owner how many rows of which expert arrive from whom, so the expert ids themselves
    never travel."""
    flat = top_idx.reshape(-1).to(torch.int64)
    send_order = torch.sort(flat, stable=True).indices
    per_expert = torch.bincount(flat, minlength=num_experts)
    return send_order, per_expert


def combine_rows(rows: torch.Tensor, send_order: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor) -> torch.Tensor:
    """out[t] = sum over slots, in ascending expert id, of top_w[t, s] * rows[position of pair (t, s)] (f32 accumulate)."""
    t, k = top_idx.shape
    pos = torch.empty_like(send_order)
    pos[send_order] = torch.arange(send_order.numel(), device=send_order.device)
    per_pair = rows.to(torch.float32)[pos].reshape(t, k, -1)
    order = torch.sort(top_idx.to(torch.int64), dim=1, stable=True).indices
    acc = torch.zeros((t, rows.shape[1]), dtype=torch.float32, device=rows.device)
    for s in range(k):
        sel = order[:, s]
        w = torch.gather(top_w, 1, sel[:, None])
        acc += w * torch.gather(per_pair, 1, sel[:, None, None].expand(t, 1, per_pair.shape[2]))[:, 0]
    return acc


def all_to_all_rows(rows: torch.Tensor, send_counts: Sequence[int], recv_counts: Sequence[int], group=None) -> torch.Tensor:
    """Variable-size all-to-all of matrix rows (works for NCCL and gloo)."""
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=[int(c) for c in recv_counts],
                           input_split_sizes=[int(c) for c in send_counts], group=group)
    return out


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


# ----------------------------------------------------------------------------- tensor parallel linear
class ColumnParallelLinear:
    """Column-split linear: ``local`` computes ``x @ W[a:b]^T``; ``forward`` all-gathers the shards.

    ``local`` is any callable ``x[m, k] -> y[m, b - a]`` (an operator of :mod:`linear` built on the
    sliced tensors). ``chunks`` > 1 cuts the batch into row chunks and overlaps the all-gather of one
    chunk with the matmul of the next; it pays when ``local`` costs the same per row whatever the batch
    (a dense or GEMV-sized operator), not for the dequantize-then-GEMM operators, which would
    dequantize the shard once per chunk.
    """

    def __init__(self, local: Callable[[torch.Tensor], torch.Tensor], out_features: int, group=None, chunks: int = 1,
                 multiple: int = 8):
        self.local, self.n, self.group, self.chunks = local, out_features, group, max(1, chunks)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bounds = [column_shard(out_features, self.world, r, multiple) for r in range(self.world)]
        self.width = max(b - a for a, b in self.bounds)

    @staticmethod
    def slice_awq(qweight, qzeros, scales, a: int, b: int):
        """Columns ``[a, b)`` of an AWQ triplet (pure slices of the packed tensors)."""
        return qweight[:, a // 8:b // 8].contiguous(), qzeros[:, a // 8:b // 8].contiguous(), scales[:, a:b].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        out = x.new_empty((m, self.n))
        step = (m + self.chunks - 1) // self.chunks
        pending = []
        for r0 in range(0, m, step):
            r1 = min(m, r0 + step)
            y = self.local(x[r0:r1])
            if y.shape[1] != self.width:  # uneven shards: pad to the widest so the gather is regular
                y = torch.nn.functional.pad(y, (0, self.width - y.shape[1]))
            flat = y.new_empty((self.world * (r1 - r0), self.width))  # rank-major concatenation
            work = dist.all_gather_into_tensor(flat, y.contiguous(), group=self.group, async_op=True)
            pending.append((work, flat.view(self.world, r1 - r0, self.width), r0, r1))
        even = all(b - a == self.width for a, b in self.bounds)
        for work, gathered, r0, r1 in pending:
            work.wait()
            if even:  # one strided copy: [world, rows, width] -> [rows, world * width]
                out[r0:r1].view(r1 - r0, self.world, self.width).copy_(gathered.permute(1, 0, 2))
            else:
                for r, (a, b) in enumerate(self.bounds):
                    out[r0:r1, a:b] = gathered[r, :, :b - a]
        return out


class PeerStoreColumnLinear:
    """Column-split AWQ linear that places its output block straight into ``out[:, a:b]`` of EVERY rank.

    No all-gather and no re-layout: ``oxq_awq_gemm_tp`` runs the tensor-core GEMM of the shard into the local output
    and copies the finished column block, through peer pointers, to the same place in the other ranks' outputs
    (plain stores over NVLink from a small kernel of the library; nothing is read from a peer). The output buffer ``[m_max, n]`` is symmetric memory
    (``torch.distributed._symmetric_memory``), allocated and exchanged once. Two barriers order the ranks: one
    before the GEMM (nobody still reads the previous result) and one after it (every tile has landed).
    ``forward`` returns a view of that buffer, valid until the next ``forward``.
    """

    def __init__(self, shard, out_features: int, m_max: int, group=None, dtype: torch.dtype = torch.bfloat16):
        import torch.distributed._symmetric_memory as symm_mem
        self.shard, self.n, self.m_max = shard, out_features, m_max
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.a, self.b = column_shard(out_features, self.world, self.rank)
        if shard.out_features != self.b - self.a:
            raise ValueError(f"shard has {shard.out_features} out features, rank {self.rank} owns {self.b - self.a}")
        if self.world > 8:
            raise ValueError("PeerStoreColumnLinear: at most 8 ranks (7 peer outputs)")
        self.out = symm_mem.empty((m_max, out_features), dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        self.hdl = symm_mem.rendezvous(self.out, self.group.group_name)
        import ctypes
        peers = [int(self.hdl.buffer_ptrs[r]) for r in range(self.world) if r != self.rank]
        self._peers = (ctypes.c_void_p * max(1, len(peers)))(*peers)
        self._n_peers = len(peers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import _lib, gemm
        from .linear import _dt, _p, _stream
        m = x.shape[0]
        if m > self.m_max:
            raise ValueError(f"PeerStoreColumnLinear: batch {m} exceeds the buffer ({self.m_max} rows)")
        lin = self.shard
        ws = gemm.workspace(lin.out_features, lin.in_features, x.device)
        y = self.out[:m]
        self.hdl.barrier(channel=0)  # the previous result is no longer read anywhere
        # row stride of the output buffer is n for any m (a leading slice), so peer offsets equal local ones
        import ctypes
        _lib.call("oxq_awq_gemm_tp", _p(x), _dt(x.dtype), _p(lin.qweight), _p(lin.qzeros), _p(lin.scales), _dt(lin.scales.dtype),
                  _p(lin.bias), _dt(lin.bias.dtype) if lin.bias is not None else 0, _p(y),
                  ctypes.cast(self._peers, ctypes.c_void_p), self._n_peers, _dt(y.dtype), m, lin.in_features, lin.out_features,
                  self.a, self.n, lin.group_size, _p(ws), ws.numel(), _stream())
        self.hdl.barrier(channel=1)  # every rank's tiles have landed here
        return y


# ----------------------------------------------------------------------------- expert parallel MoE
class ExpertParallelMoe:
    """All-to-all expert parallelism around a local expert function.

    ``route(logits) -> (top_idx int32 [t, k], top_w f32 [t, k])`` and
    ``local_experts(rows[r, hidden], expert_ids[r]) -> y[r, hidden]`` (each row through its expert,
    weight 1) are supplied by the caller: the CUDA operators in production, anything else in tests.
    """

    def __init__(self, num_experts: int, route: Callable, local_experts: Callable, group=None):
        self.num_experts, self.route, self.local_experts, self.group = num_experts, route, local_experts, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.bounds = [expert_shard(num_experts, self.world, r) for r in range(self.world)]

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        top_idx, top_w = self.route(logits)
        k = top_idx.shape[1]
        on_device = x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
        if on_device:  # counting sort by expert id in three small kernels: counts, send order and its inverse
            from . import moe
            per_expert, send_order, pos = moe.dispatch_plan(top_idx, self.num_experts)
        else:
            send_order, per_expert = plan_dispatch_by_expert(top_idx, self.num_experts)
            pos = None
        sizes = [hi - lo for lo, hi in self.bounds]
        lo, hi = self.bounds[self.rank]
        n_local = hi - lo
        if on_device:
            rows = moe.gather_rows(x, send_order, k)  # needs no size from the host: runs while the counts travel
        # counts per (source rank, local expert): one small all-to-all; the expert ids of the rows follow from them
        recv_pe = per_expert.new_empty((self.world * n_local,))
        dist.all_to_all_single(recv_pe, per_expert, output_split_sizes=[n_local] * self.world, input_split_sizes=sizes,
                               group=self.group)
        both = torch.cat([per_expert, recv_pe]).tolist()  # the one host read-back: buffer sizes (summed on the host)
        sc = [sum(both[a:b]) for a, b in self.bounds]
        rc = [sum(both[self.num_experts + r * n_local:self.num_experts + (r + 1) * n_local]) for r in range(self.world)]
        total = int(sum(rc))
        if on_device:
            got_ids = moe.expand_ids(recv_pe, n_local, lo, total)
        else:
            rows = x[send_order // k]
            local_ids = torch.arange(lo, hi, device=recv_pe.device, dtype=torch.int32).repeat(self.world)
            got_ids = torch.repeat_interleave(local_ids, recv_pe, output_size=total)
        got_rows = all_to_all_rows(rows, sc, rc, self.group)
        y = self.local_experts(got_rows, got_ids) if got_rows.shape[0] else got_rows
        back = all_to_all_rows(y.to(x.dtype), rc, sc, self.group)
        if on_device:  # the device combine: one kernel, ascending expert order, f32 accumulation
            return moe.combine(back, top_idx, top_w, pos, self.num_experts, x.dtype)
        return combine_rows(back, send_order, top_idx, top_w).to(x.dtype)


def gptoss_local_experts(layer) -> Callable:
    """``local_experts`` callable over a :class:`moe.GptOssMoe` holding ALL expert tensors (only the local
    ones are touched): each received row goes through its expert with weight one (``oxq_gptoss_experts_forward``)."""
    def run(rows: torch.Tensor, expert_ids: torch.Tensor) -> torch.Tensor:
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        return layer.forward_experts(rows, expert_ids, expert_shard(layer.num_experts, world, rank))
    return run

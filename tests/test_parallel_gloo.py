"""World-size-2 gloo runs (CPU) of the sharding logic: the column split + all-gather and the
all-to-all expert dispatch/combine must reproduce the unsharded oracle result. The local compute is
the CPU oracle here (the CUDA operators cannot run without a GPU); the GPU tests cover the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oxydllm_b200 import parallel, synth


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), fn, ret), nprocs=world, join=True)
    return [ret[r] for r in range(world)]


def _tp_case(rank, world):
    k, n, g, m = 256, 200, 64, 9          # 25 packed words: uneven shards (13 and 12 words)
    qw, qz, sc = synth.awq_layer(k, n, g, seed=3)
    x = synth.activations(m, k, seed=4)
    a, b = parallel.column_shard(n, world, rank)
    sqw, sqz, ssc = parallel.ColumnParallelLinear.slice_awq(torch.from_numpy(qw.view(np.int32)), torch.from_numpy(qz.view(np.int32)),
                                                            torch.from_numpy(sc), a, b)
    w_local = oracle.awq_dequant(sqw.numpy().view(np.uint32), sqz.numpy().view(np.uint32), ssc.numpy())
    lin = parallel.ColumnParallelLinear(lambda xx: torch.from_numpy(oracle.linear(xx.numpy(), w_local)), n, chunks=2)
    y = lin.forward(torch.from_numpy(x)).numpy()
    ref = oracle.linear(x, oracle.awq_dequant(qw, qz, sc))
    return float(np.abs(y - ref).max()), (a, b)


def test_column_parallel_awq_equals_unsharded():
    res = _run(_tp_case)
    assert [r[1] for r in res] == [(0, 104), (104, 200)]
    assert all(r[0] == 0.0 for r in res)  # same arithmetic per column: identical bits


def _ep_case(rank, world, e=6):
    hidden, inter, t_local, k = 64, 32, 11, 3
    d = synth.gptoss_moe(e, hidden, inter, t_local * world, seed=7)
    x_all, lg_all = d["x"], d["logits"]
    sl = slice(rank * t_local, (rank + 1) * t_local)
    lo, hi = parallel.expert_shard(e, world, rank)

    def route(lg):
        idx, w = oracle.moe_route(lg.numpy(), k, True)
        return torch.from_numpy(idx), torch.from_numpy(w)

    def local_experts(rows, ids):
        out = np.empty((rows.shape[0], hidden), np.float32)
        for i, ex in enumerate(ids.tolist()):
            assert lo <= ex < hi, "row sent to a rank that does not own its expert"
            w_gu = oracle.mxfp4_dequant(d["gu_blocks"][ex], d["gu_scales"][ex], 2 * inter, hidden)
            w_dn = oracle.mxfp4_dequant(d["dn_blocks"][ex], d["dn_scales"][ex], hidden, inter)
            out[i] = oracle.gptoss_expert(rows[i:i + 1].numpy(), w_gu, d["gu_bias"][ex], w_dn, d["dn_bias"][ex])[0]
        return torch.from_numpy(out)

    ep = parallel.ExpertParallelMoe(e, route, local_experts)
    y = ep.forward(torch.from_numpy(x_all[sl]), torch.from_numpy(lg_all[sl])).numpy()
    idx, w = oracle.moe_route(lg_all, k, True)
    ref = oracle.gptoss_moe(x_all, idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], hidden, inter)[sl]
    return float(np.abs(y - ref).max() / max(1e-9, np.abs(ref).max()))


def test_expert_parallel_all_to_all_equals_unsharded():
    res = _run(_ep_case)
    assert all(r < 1e-5 for r in res), res


def _ep_case_uneven(rank, world):
    return _ep_case(rank, world, e=5)  # shards (0, 3) and (3, 5): unequal split sizes in the counts exchange


def test_expert_parallel_with_an_uneven_expert_split():
    res = _run(_ep_case_uneven)
    assert all(r < 1e-5 for r in res), res


def test_shard_arithmetic():
    assert [parallel.column_shard(128256, 8, r) for r in (0, 7)] == [(0, 16032), (112224, 128256)]
    assert [parallel.expert_shard(32, 8, r) for r in (0, 3, 7)] == [(0, 4), (12, 16), (28, 32)]
    assert [parallel.expert_shard(6, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 5), (5, 6)]
    ex = torch.arange(6)
    assert parallel.owner_of_expert(ex, 6, 4).tolist() == [0, 0, 1, 1, 2, 3]
    with pytest.raises(ValueError):
        parallel.column_shard(100, 2, 0)
    top_idx = torch.tensor([[5, 0], [1, 4]])
    order, counts = parallel.plan_dispatch(top_idx, 6, 2)
    assert counts.tolist() == [2, 2] and order.tolist() == [1, 2, 0, 3]
    order, per_expert = parallel.plan_dispatch_by_expert(top_idx, 6)  # sorted by expert id, pair order kept
    assert per_expert.tolist() == [1, 1, 0, 0, 1, 1] and order.tolist() == [1, 2, 3, 0]

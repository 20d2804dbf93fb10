"""torchrun worker: tensor-parallel AWQ linear and expert-parallel GPT-OSS MoE on N GPUs, checked against
the single-GPU operators (rank 0 holds the unsharded result). Launched by tests/test_gpu_multi.py."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxydllm_b200 import linear as L  # noqa: E402
from oxydllm_b200 import moe, parallel, synth  # noqa: E402


def dev(a, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dt) if dt is not None else t).cuda()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # --- tensor parallel column split + all-gather (decode and prefill sized batches)
    k, n, g = 1024, 2056 * 8 // 8, 128
    n = 2048 + 8 * world * 3  # not a multiple of the tile width, even shards
    qw, qz, sc = synth.awq_layer(k, n, g, seed=1)
    full = L.PackedQuantLinear(L.QuantWeight.new_awq(4, dev(qw.view(np.int32)), dev(qz.view(np.int32)), dev(sc)))
    a, b = parallel.column_shard(n, world, rank)
    sqw, sqz, ssc = parallel.ColumnParallelLinear.slice_awq(full.qweight, full.qzeros, full.scales, a, b)
    shard = L.PackedQuantLinear(L.QuantWeight.new_awq(4, sqw, sqz, ssc))
    for m, chunks in ((4, 1), (200, 2)):
        x = dev(synth.activations(m, k, seed=m), torch.bfloat16)
        tp = parallel.ColumnParallelLinear(shard.forward, n, chunks=chunks)
        y = tp.forward(x)
        ref = full.forward(x)
        err = float((y.float() - ref.float()).abs().max())
        tol = 2e-2 * float(ref.float().abs().max())
        assert err <= tol, f"TP m={m}: {err} > {tol}"

    # --- the same split with direct placement: each rank's GEMM stores its tile into every rank's output
    ps = parallel.PeerStoreColumnLinear(shard, n, m_max=320)
    for m in (200, 64, 300, 200):  # fused kernel on the shard up to 256 rows, dequantized slab + GEMM above
        x = dev(synth.activations(m, k, seed=m + 7), torch.bfloat16)
        y = ps.forward(x)
        ref = full.forward(x)
        err = float((y.float() - ref.float()).abs().max())
        tol = 2e-2 * float(ref.float().abs().max())
        assert err <= tol, f"peer-store TP m={m}: {err} > {tol}"
    from oxydllm_b200 import gemm
    gemm.check(gemm.workspace(shard.out_features, k, "cuda"))

    # --- expert parallel all-to-all dispatch / combine
    e, hidden, inter, t_local = 8, 128, 128, 96
    d = synth.gptoss_moe(e, hidden, inter, t_local * world, seed=2)
    layer = moe.GptOssMoe(dev(d["gu_blocks"]), dev(d["gu_scales"]), dev(d["gu_bias"], torch.bfloat16), dev(d["dn_blocks"]),
                          dev(d["dn_scales"]), dev(d["dn_bias"], torch.bfloat16), hidden=hidden, inter=inter, top_k=4)
    sl = slice(rank * t_local, (rank + 1) * t_local)
    x_all, lg_all = dev(d["x"], torch.bfloat16), dev(d["logits"])
    ep = parallel.ExpertParallelMoe(e, lambda lg: moe.route(lg, 4, True), parallel.gptoss_local_experts(layer))
    y = ep.forward(x_all[sl].contiguous(), lg_all[sl].contiguous())
    ref = layer.forward_with_logits(x_all, lg_all)[sl]
    layer.check()
    err = float((y.float() - ref.float()).abs().max())
    tol = 2e-2 * float(ref.float().abs().max())
    assert err <= tol, f"EP: {err} > {tol}"
    dist.barrier()
    if rank == 0:
        print("multi-gpu ok", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

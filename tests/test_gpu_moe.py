"""GPT-OSS MXFP4 MoE layer on the device against the CPU oracle (f32 chain of the reference's CPU path).
Tolerance: max|err| <= 2e-2 * ||row||_inf (bf16 activations between the two expert GEMMs)."""
import numpy as np
import pytest
import torch

import oracle
from oxydllm_b200 import moe, synth

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dtype) if dtype is not None else t).cuda()


def build(d):
    return moe.GptOssMoe(dev(d["gu_blocks"]), dev(d["gu_scales"]), dev(d["gu_bias"], torch.bfloat16),
                         dev(d["dn_blocks"]), dev(d["dn_scales"]), dev(d["dn_bias"], torch.bfloat16),
                         hidden=d["x"].shape[1], inter=d["dn_blocks"].shape[2] * 32, top_k=4)


@pytest.mark.parametrize("tokens,experts", [(1, 4), (5, 32), (64, 32), (777, 8)])
def test_route_matches_oracle(cuda, tokens, experts):
    logits = np.random.default_rng(tokens).standard_normal((tokens, experts)).astype(np.float32)
    k = min(4, experts)
    idx, w = moe.route(dev(logits), k)
    ridx, rw = oracle.moe_route(logits, k, True)
    assert np.array_equal(idx.cpu().numpy(), ridx)  # N(0,1) logits: no ties
    assert np.allclose(w.cpu().numpy(), rw, rtol=1e-5, atol=1e-7)
    idx2, w2 = moe.route(dev(logits), k, norm_topk=False)
    _, rw2 = oracle.moe_route(logits, k, False)
    assert np.allclose(w2.cpu().numpy(), rw2, rtol=1e-5, atol=1e-7)


def test_route_ties_take_lower_index(cuda):
    logits = np.zeros((3, 8), np.float32)
    idx, w = moe.route(dev(logits), 4)
    assert idx.cpu().tolist() == [[0, 1, 2, 3]] * 3
    assert np.allclose(w.cpu().numpy(), 0.25)


@pytest.mark.parametrize("tokens,experts,hidden,inter", [(40, 4, 64, 64), (300, 8, 128, 96), (129, 32, 256, 256),
                                                         (3, 4, 64, 32)])
def test_moe_layer_matches_oracle(cuda, tokens, experts, hidden, inter):
    d = synth.gptoss_moe(experts, hidden, inter, tokens, seed=tokens)
    # larger weights than N(0, 0.02) so that the clamps and the sigmoid gate are exercised
    rng = np.random.default_rng(1)
    d["x"] = synth.bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32) * 4.0)
    layer = build(d)
    y = layer.forward_with_logits(dev(d["x"], torch.bfloat16), dev(d["logits"]))
    layer.check()
    idx, w = oracle.moe_route(d["logits"], 4, True)
    ref = oracle.gptoss_moe(d["x"], idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], hidden, inter, 7.0)
    got = y.float().cpu().numpy()
    assert got.shape == ref.shape and np.isfinite(got).all()
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    assert (np.abs(got - ref) <= 2e-2 * row_inf + 1e-5).all(), np.abs(got - ref).max()


def test_moe_expert_ranges_add_up_and_are_deterministic(cuda):
    d = synth.gptoss_moe(8, 128, 128, 200, seed=5)
    layer = build(d)
    x, lg = dev(d["x"], torch.bfloat16), dev(d["logits"])
    full = layer.forward_with_logits(x, lg).float()
    again = layer.forward_with_logits(x, lg).float()
    assert torch.equal(full, again)
    parts = sum(layer.forward_with_logits(x, lg, (lo, lo + 2)).float() for lo in range(0, 8, 2))
    layer.check()
    assert torch.allclose(parts, full, rtol=2e-2, atol=2e-2 * float(full.abs().max()))
    ref_lo = oracle.gptoss_moe(d["x"], *oracle.moe_route(d["logits"], 4, True), d["gu_blocks"], d["gu_scales"], d["gu_bias"],
                               d["dn_blocks"], d["dn_scales"], d["dn_bias"], 128, 128, 7.0, expert_range=(0, 2))
    got_lo = layer.forward_with_logits(x, lg, (0, 2)).float().cpu().numpy()
    assert (np.abs(got_lo - ref_lo) <= 2e-2 * np.abs(ref_lo).max(axis=1, keepdims=True) + 1e-4).all()


def test_moe_gpt_oss_shape_slice(cuda):
    """GPT-OSS-20B expert shape (hidden = inter = 2880, 45 k blocks of 64) with 4 experts and 256 tokens."""
    d = synth.gptoss_moe(4, 2880, 2880, 256, seed=9)
    layer = build(d)
    y = layer.forward_with_logits(dev(d["x"], torch.bfloat16), dev(d["logits"]))
    layer.check()
    idx, w = oracle.moe_route(d["logits"], 4, True)
    ref = oracle.gptoss_moe(d["x"], idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], 2880, 2880, 7.0)
    got = y.float().cpu().numpy()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all()


@pytest.mark.parametrize("tokens", [1, 4, 16])
def test_moe_decode_path_gpt_oss_shape(cuda, tokens):
    """Few (token, slot) pairs: batched single-token GEMVs on the selected experts' packed weights (no dequantized slab)."""
    d = synth.gptoss_moe(8, 2880, 2880, tokens, seed=20 + tokens)
    layer = build(d)
    x, lg = dev(d["x"], torch.bfloat16), dev(d["logits"])
    y = layer.forward_with_logits(x, lg)
    idx, w = oracle.moe_route(d["logits"], 4, True)
    args = (d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"], d["dn_bias"], 2880, 2880, 7.0)
    ref = oracle.gptoss_moe(d["x"], idx, w, *args)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all(), np.abs(got - ref).max()
    assert torch.equal(y, layer.forward_with_logits(x, lg))  # run-to-run identical
    # a rank's expert range: the other experts' pairs contribute nothing
    got_hi = layer.forward_with_logits(x, lg, (4, 8)).float().cpu().numpy()
    ref_hi = oracle.gptoss_moe(d["x"], idx, w, *args, expert_range=(4, 8))
    assert (np.abs(got_hi - ref_hi) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all()


def test_forward_experts_with_given_ids_matches_oracle(cuda):
    """Rows that already carry their expert (the owner side of expert parallelism): each row through that expert, weight one."""
    e, hidden, inter, rows = 8, 128, 96, 150
    d = synth.gptoss_moe(e, hidden, inter, rows, seed=3)
    layer = build(d)
    lo, hi = 2, 6
    ids = np.random.default_rng(0).integers(lo, hi, size=rows).astype(np.int32)
    y = layer.forward_experts(dev(d["x"], torch.bfloat16), dev(ids), (lo, hi))
    layer.check()
    got = y.float().cpu().numpy()
    for r in range(0, rows, 7):
        ex = int(ids[r])
        w_gu = oracle.mxfp4_dequant(d["gu_blocks"][ex], d["gu_scales"][ex], 2 * inter, hidden)
        w_dn = oracle.mxfp4_dequant(d["dn_blocks"][ex], d["dn_scales"][ex], hidden, inter)
        ref = oracle.gptoss_expert(d["x"][r:r + 1], w_gu, d["gu_bias"][ex], w_dn, d["dn_bias"][ex])[0]
        assert np.abs(got[r] - ref).max() <= 2e-2 * np.abs(ref).max() + 1e-5, r


def test_device_combine_matches_host_combine(cuda):
    from oxydllm_b200 import parallel
    t, k, hidden, e = 37, 4, 64, 16
    rng = np.random.default_rng(1)
    top_idx = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
    top_w = rng.random((t, k)).astype(np.float32)
    rows = synth.bf16_round(rng.standard_normal((t * k, hidden)).astype(np.float32))
    send_order = torch.from_numpy(rng.permutation(t * k))
    pos = torch.empty_like(send_order)
    pos[send_order] = torch.arange(t * k)
    ref = parallel.combine_rows(torch.from_numpy(rows), send_order, torch.from_numpy(top_idx), torch.from_numpy(top_w))
    got = moe.combine(dev(rows, torch.bfloat16), dev(top_idx), dev(top_w), pos.cuda(), e, torch.float32)
    assert torch.allclose(got.cpu(), ref, rtol=1e-6, atol=1e-6)


def test_moe_skewed_routing_many_blocks_and_empty_experts(cuda):
    """One expert takes most rows (several token blocks of the grouped kernel), others take none or a handful."""
    tokens, experts, hidden, inter = 700, 8, 128, 128
    d = synth.gptoss_moe(experts, hidden, inter, tokens, seed=21)
    lg = np.full((tokens, experts), -30.0, dtype=np.float32)
    lg[:, 0] = 5.0                                  # every token picks expert 0 first
    lg[:, 1:4] = np.random.default_rng(3).standard_normal((tokens, 3)).astype(np.float32)
    lg[:5, 6] = 9.0                                 # five rows for expert 6; experts 4, 5, 7 get nothing or ties only
    d["logits"] = lg
    layer = build(d)
    y = layer.forward_with_logits(dev(d["x"], torch.bfloat16), dev(lg))
    layer.check()
    idx, w = oracle.moe_route(lg, 4, True)
    counts = np.bincount(idx.reshape(-1), minlength=experts)
    assert counts[0] == tokens and counts.min() == 0  # more than two blocks of 256 rows, and an empty expert
    ref = oracle.gptoss_moe(d["x"], idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], hidden, inter, 7.0)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all()


def test_moe_tiny_block_scales_take_the_f32_route(cuda):
    """E8M0 bytes below 4 (2^-127 .. 2^-124: products leave the normal bf16 range) in a tenth of the blocks."""
    tokens, experts, hidden, inter = 300, 4, 256, 192
    d = synth.gptoss_moe(experts, hidden, inter, tokens, seed=33)
    rng = np.random.default_rng(8)
    for key in ("gu_scales", "dn_scales"):
        sc = d[key].copy()
        mask = rng.random(sc.shape) < 0.1
        sc[mask] = rng.integers(0, 4, size=int(mask.sum()), dtype=np.uint8)
        d[key] = sc
    layer = build(d)
    y = layer.forward_with_logits(dev(d["x"], torch.bfloat16), dev(d["logits"]))
    layer.check()
    idx, w = oracle.moe_route(d["logits"], 4, True)
    ref = oracle.gptoss_moe(d["x"], idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], hidden, inter, 7.0)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all()


def test_grouped_kernel_survives_a_weight_producer_that_never_loads(cuda):
    # With no packed box ever arriving, the unpack teams, the MMA issuer and the epilogue warps of the grouped kernel each
    # give up after the 2 s limit, tensor memory is freed, the kernel returns, the check reports a code once, and the layer
    # still works afterwards.
    import ctypes
    from oxydllm_b200 import _lib, gemm
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    _lib.call("oxq_selftest_moe_wait_expiry", ctypes.c_void_p(ws.data_ptr()), ws.numel(), None)
    with pytest.raises(_lib.OxqError, match=r"bounded wait \d+"):
        gemm.check(ws)
    gemm.check(ws)
    d = synth.gptoss_moe(4, 128, 128, 200, seed=2)
    layer = build(d)
    y = layer.forward_with_logits(dev(d["x"], torch.bfloat16), dev(d["logits"]))
    layer.check()
    idx, w = oracle.moe_route(d["logits"], 4, True)
    ref = oracle.gptoss_moe(d["x"], idx, w, d["gu_blocks"], d["gu_scales"], d["gu_bias"], d["dn_blocks"], d["dn_scales"],
                            d["dn_bias"], 128, 128, 7.0)
    got = y.float().cpu().numpy()
    assert (np.abs(got - ref) <= 2e-2 * np.abs(ref).max(axis=1, keepdims=True) + 1e-5).all()


@pytest.mark.parametrize("tokens,experts,k", [(1, 4, 4), (37, 8, 2), (1024, 32, 4), (4099, 32, 4)])
def test_dispatch_plan_gather_and_ids_match_torch(cuda, tokens, experts, k):
    """The expert-parallel bookkeeping kernels against their eager equivalents (bit-exact: integer work and row copies)."""
    g = torch.Generator().manual_seed(tokens)
    top_idx = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).to(torch.int32).cuda()
    counts, perm, inv = moe.dispatch_plan(top_idx, experts)
    flat = top_idx.reshape(-1).to(torch.int64)
    ref_perm = torch.sort(flat, stable=True).indices
    assert torch.equal(counts.long(), torch.bincount(flat, minlength=experts))
    assert torch.equal(perm.long(), ref_perm)
    assert torch.equal(inv.long()[ref_perm], torch.arange(flat.numel(), device="cuda"))
    x = torch.randn(tokens, 64, device="cuda").to(torch.bfloat16)
    assert torch.equal(moe.gather_rows(x, perm, k), x[ref_perm // k])
    world, n_local, lo = 4, experts // 4, experts // 4 * 2
    grp = torch.randint(0, 50, (world * n_local,), generator=g).to(torch.int32).cuda()
    grp[1] = 0
    ids = moe.expand_ids(grp, n_local, lo, int(grp.sum()))
    ref_ids = torch.repeat_interleave(torch.arange(lo, lo + n_local, device="cuda", dtype=torch.int32).repeat(world), grp.long())
    assert torch.equal(ids, ref_ids)

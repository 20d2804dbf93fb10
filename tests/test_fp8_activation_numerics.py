"""Why the FP8 block-scaled matmul multiplies bf16 activations (a decision record kept as a test).

A native FP8 x FP8 tensor-core product needs the activations in an 8-bit format. On benchmark configuration 3
(W ~ N(0, 0.02) as E4M3 with one scale per 128 x 128 block, K = 4096, N = 14336, bf16 N(0, 1) activations) rounding x
to E4M3 per (row, 128-wide k block) puts the result outside the stated matmul tolerance
max|err| <= 2e-2 * ||row||_inf against the reference's dequantize-to-f32 product (linear.rs:96-145), while splitting
every activation into two E4M3 pieces is well inside but costs two products per weight. CPU only (torch float8 casts)."""
import torch


def _case(m=2, n=14336, k=4096, blk=128):
    torch.manual_seed(0)
    w = torch.randn(n, k) * 0.02
    wb = w.view(n // blk, blk, k // blk, blk)
    scale = wb.abs().amax(dim=(1, 3), keepdim=True) / 448.0
    wq = (wb / scale).to(torch.float8_e4m3fn).float()
    x = torch.randn(m, k).bfloat16().float()
    ref = x @ (wq * scale).view(n, k).t()
    return wq, scale, x, ref, blk


def _blockwise(pieces, wq, scale, blk):
    """sum over k blocks of (sum_p piece_p . Wq^T * piece_scale_p) * weight block scale, f32 accumulation."""
    n, k = wq.shape[0] * wq.shape[1], wq.shape[2] * wq.shape[3]
    out = torch.zeros(pieces[0][0].shape[0], n)
    for kb in range(k // blk):
        wt = wq[:, :, kb, :].reshape(n, blk).t()
        sc = scale[:, 0, kb, 0].repeat_interleave(blk)[None, :]
        out += sum((xq[:, kb, :] @ wt) * xs[:, kb, :] for xq, xs in pieces) * sc
    return out


def test_one_e4m3_piece_per_activation_misses_the_tolerance_two_pieces_meet_it():
    wq, scale, x, ref, blk = _case()
    row_inf = ref.abs().amax(dim=1)
    xb = x.view(x.shape[0], -1, blk)
    s1 = xb.abs().amax(dim=2, keepdim=True) / 448.0
    q1 = (xb / s1).to(torch.float8_e4m3fn).float()
    one = ((_blockwise([(q1, s1)], wq, scale, blk) - ref).abs().amax(dim=1) / row_inf)
    assert bool((one > 2e-2).all()), one  # 0.023 .. 0.029 on this configuration
    r = xb / s1 - q1
    s2 = r.abs().amax(dim=2, keepdim=True).clamp_min(1e-30) / 448.0
    q2 = (r / s2).to(torch.float8_e4m3fn).float()
    two = ((_blockwise([(q1, s1), (q2, s1 * s2)], wq, scale, blk) - ref).abs().amax(dim=1) / row_inf)
    assert bool((two < 2e-3).all()), two

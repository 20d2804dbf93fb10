"""oxq_awq_gemm_noalloc: the AWQ prefill matmul for callers that cannot allocate device memory.

Some hosts of this library may not call cudaMalloc at the moment they need a matmul: a runtime
that owns the only allocator, a plugin loaded after all free memory went to a pool, or code
running where allocation is forbidden. For them the library carries its own fixed scratch array.
This test drives the entry point through the C ABI exactly as such a caller would (inputs and
outputs are the caller's; no workspace is passed) and checks it, twice in a row because the
scratch keeps the previous call's contents, against the regular workspace-taking entry point.
The file name sorts last so that a run stopping at the first failure has already run every other
test; the test also passes alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from oxydllm_b200 import _lib, gemm, synth

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(m, k, n, g, seed):
    qw, qz, sc = synth.awq_layer(k, n, g, seed=seed)
    x = synth.activations(m, k, seed=seed + 1)
    bias = synth.bf16_round(np.random.default_rng(seed + 2).standard_normal(n).astype(np.float32))
    t = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(dt) if dt else torch.from_numpy(np.ascontiguousarray(a))).cuda()
    return (t(x, torch.bfloat16), t(qw.view(np.int32)), t(qz.view(np.int32)), t(sc), t(bias, torch.bfloat16))


def _run_both(m, k, n, g, seed):
    x, qw, qz, sc, bias = _case(m, k, n, g, seed)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    y_ref = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ws = gemm.workspace(n, k, x.device)
    _lib.call("oxq_awq_gemm", _p(x), _lib.OXQ_BF16, _p(qw), _p(qz), _p(sc), _lib.OXQ_F16, _p(bias), _lib.OXQ_BF16,
              _p(y_ref), _lib.OXQ_BF16, m, k, n, g, _p(ws), ws.numel(), st)
    gemm.check(ws)
    y_new = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    _lib.call("oxq_awq_gemm_noalloc", _p(x), _lib.OXQ_BF16, _p(qw), _p(qz), _p(sc), _lib.OXQ_F16, _p(bias),
              _lib.OXQ_BF16, _p(y_new), _lib.OXQ_BF16, m, k, n, g, st)
    _lib.call("oxq_awq_gemm_noalloc_check", st)
    return y_new.float().cpu().numpy(), y_ref.float().cpu().numpy()


def test_noalloc_matches_workspace_entry_twice_in_a_row(cuda):
    # two different problems back to back: the second must not see anything of the first
    for m, k, n, g, seed in [(96, 1024, 2048, 128, 10), (70, 512, 1032, 64, 20)]:
        got, ref = _run_both(m, k, n, g, seed)
        assert np.isfinite(got).all()
        row_inf = np.abs(ref).max(axis=1, keepdims=True)
        assert (np.abs(got - ref) <= 2e-2 * row_inf + 1e-6).all()


def test_noalloc_rejects_sizes_beyond_its_scratch(cuda):
    max_k = int(_lib.load().oxq_awq_gemm_noalloc_max_k())
    assert max_k == 16384
    one = ctypes.c_void_p(256)
    k = max_k + 128
    with pytest.raises(_lib.OxqError, match="exceeds the built-in scratch") as e:
        _lib.call("oxq_awq_gemm_noalloc", one, _lib.OXQ_BF16, one, one, one, _lib.OXQ_F16, None, 0, one, _lib.OXQ_BF16,
                  64, k, 256, 128, None)
    assert e.value.status == -5

"""The scratch-free total-attention entry point against the regular one.

``b200attn_total_attention_static`` exists for callers that have no device memory to lend the
library: a process whose memory pool took the whole budget up front, or glue code that only ever
sees input and output buffers. It keeps its per-query statistics in an array compiled into the
library instead of a caller workspace. Both entry points run the same kernels, so the results must
be identical; two calls in a row (the second on a smaller, differently shaped problem) check that
whatever the first call left in the shared array does not leak into the second.
"""
import math

import pytest
import torch

from flagattention_b200 import _lib

pytestmark = pytest.mark.gpu


def _total(entry, q, k, lse, causal, workspace):
    lib = _lib.load()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    tot = torch.full((B, Hq, N), float("nan"), dtype=torch.float32, device=q.device)
    status = torch.zeros(1, dtype=torch.int32, device=q.device)
    p = _lib.TotalParams(_lib.tensor4(q), _lib.tensor4(k), lse.data_ptr(), tot.data_ptr(),
                         workspace.data_ptr() if workspace is not None else None,
                         B, Hq, Hk, M, N, D, _lib.dtype_code(q.dtype), int(causal), 1.0 / math.sqrt(D),
                         status.data_ptr())
    _lib.check(getattr(lib, entry)(p, torch.cuda.current_stream().cuda_stream), entry)
    torch.cuda.synchronize()
    assert status.item() == 0
    return tot


def _case(B, Hq, Hk, M, N, D, dtype, causal, seed):
    from flagattention_b200 import flash_attention
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, Hq, M, D, device="cuda", dtype=dtype, generator=g)
    k = torch.randn(B, Hk, N, D, device="cuda", dtype=dtype, generator=g)
    v = torch.randn(B, Hk, N, D, device="cuda", dtype=dtype, generator=g)
    _, lse, _, _, _ = flash_attention(q, k, v, causal, return_log_normalizer=True)
    return q, k, lse


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    lib = _lib.load()
    for (B, Hq, Hk, M, N, D, dtype, causal) in [(2, 8, 2, 1000, 1300, 128, torch.bfloat16, True),
                                                (1, 4, 4, 300, 200, 64, torch.float16, False)]:
        q, k, lse = _case(B, Hq, Hk, M, N, D, dtype, causal, seed=M)
        ws = torch.empty(lib.b200attn_total_workspace_bytes(B, Hq, M) // 4, dtype=torch.float32, device="cuda")
        want = _total("b200attn_total_attention", q, k, lse, causal, ws)
        got = _total("b200attn_total_attention_static", q, k, lse, causal, None)
        assert not torch.isnan(got).any()
        # identical kernels on identical statistics: same tolerance as the aux-output tests would
        # allow, in practice bit-equal
        torch.testing.assert_close(got, want, atol=1e-5, rtol=0)


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.load()
    q = torch.zeros(1, 1, 16, 64, dtype=torch.float16, device="cuda")
    p = _lib.TotalParams(_lib.tensor4(q), _lib.tensor4(q), q.data_ptr(), q.data_ptr(), None,
                         64, 64, 64, 4096, 128, 64, _lib.F16, 0, 0.125, None)
    assert lib.b200attn_total_attention_static(p, None) == -2
    assert b"exceeds the built-in scratch" in lib.b200attn_last_error()

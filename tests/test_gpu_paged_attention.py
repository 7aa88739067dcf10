"""GPU parity of paged_attention against the oracle and the reference's fixtures, on the shapes and the
tolerance of the reference's own tests (tests/flag_attn/test_paged_attention.py:24-160)."""
import pytest
import torch

from conftest import PAGED_GOLDENS, load_paged_golden
from flagattention_b200 import check_device_status, paged_attention
from gpu_util import device
from oracle.paged import paged_attention as oracle_paged

pytestmark = pytest.mark.gpu

NUM_BLOCKS = 1000


def _case(num_seqs, num_query_heads, query_group_size, head_size, block_size, max_seq_len, dtype, seed=0):
    g = torch.Generator(device=device()).manual_seed(seed)
    num_kv_heads = num_query_heads // query_group_size
    context_lens = torch.randint(1, max(2, max_seq_len), [num_seqs], dtype=torch.int32, device=device(), generator=g)
    context_lens[0] = max_seq_len
    max_context_len = int(context_lens.max().item())
    per_seq = (max_context_len + block_size - 1) // block_size
    scale = head_size ** -0.5
    q = torch.empty(num_seqs, num_query_heads, head_size, dtype=dtype, device=device()).uniform_(-scale, scale, generator=g)
    k_cache = torch.empty(NUM_BLOCKS, num_kv_heads, block_size, head_size, dtype=dtype,
                          device=device()).uniform_(-scale, scale, generator=g)
    v_cache = torch.empty_like(k_cache).uniform_(-scale, scale, generator=g)
    block_tables = torch.randint(0, NUM_BLOCKS, (num_seqs, per_seq), device=device(), generator=g)
    return q, k_cache, v_cache, context_lens, block_tables, scale, max_context_len


def _check(q, k_cache, v_cache, context_lens, block_tables, scale, max_context_len, num_splits=0):
    out = paged_attention(q, k_cache, v_cache, context_lens, block_tables, scale, max_context_len, num_splits)
    ref = oracle_paged(q, k_cache, v_cache, block_tables, context_lens, scale)
    check_device_status()
    assert out.shape == q.shape and out.dtype == q.dtype
    # the reference's acceptance test (test_paged_attention.py:74)
    assert torch.allclose(out.float(), ref.float(), atol=2e-3, rtol=1e-5), (out.float() - ref.float()).abs().max()


@pytest.mark.parametrize("num_seqs", [1, 32])
@pytest.mark.parametrize("query_group_size", [1, 8])
@pytest.mark.parametrize("head_size", [64, 128])
@pytest.mark.parametrize("block_size", [16, 128, 256])
@pytest.mark.parametrize("max_seq_len", [512, 4096])
def test_paged_attention_default(num_seqs, query_group_size, head_size, block_size, max_seq_len):
    _check(*_case(num_seqs, 64, query_group_size, head_size, block_size, max_seq_len, torch.float16))


@pytest.mark.parametrize("num_seqs", [1, 16])
@pytest.mark.parametrize("query_group_size", [1, 8])
@pytest.mark.parametrize("head_size", [32, 64])
@pytest.mark.parametrize("num_splits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_paged_attention_by_num_splits(num_seqs, query_group_size, head_size, num_splits):
    _check(*_case(num_seqs, 64, query_group_size, head_size, 16, 2048, torch.float16), num_splits=num_splits)


@pytest.mark.parametrize("num_seqs,heads,group,head_size,block_size,max_seq_len,num_splits,dtype", [
    (1, 12, 1, 64, 16, 2, 0, torch.float16),
    (16, 64, 8, 32, 16, 2048, 2, torch.float16),
    (16, 64, 1, 64, 16, 2048, 6, torch.float16),
    (3, 8, 2, 128, 32, 1000, 0, torch.bfloat16),      # two heads per KV head: streaming kernel, 2 rows
    (5, 24, 3, 64, 8, 777, 0, torch.bfloat16),        # smallest block the tensor-core path takes
    (4, 32, 16, 128, 64, 3000, 5, torch.bfloat16),    # odd split count: single-stream packed tile
    (2, 16, 4, 16, 16, 300, 0, torch.float16),
    (7, 8, 1, 32, 4, 129, 0, torch.float16),          # tiny blocks, streaming kernel
])
def test_paged_attention_more_shapes(num_seqs, heads, group, head_size, block_size, max_seq_len, num_splits, dtype):
    _check(*_case(num_seqs, heads, group, head_size, block_size, max_seq_len, dtype, seed=3), num_splits=num_splits)


@pytest.mark.parametrize("name", PAGED_GOLDENS)
def test_paged_attention_against_reference_fixture(name):
    g = load_paged_golden(name)
    q, kc, vc = (g[k].to(device()) for k in ("q", "key_cache", "value_cache"))
    out = paged_attention(q, kc, vc, g["context_lens"].to(device()), g["block_tables"].to(device()), g["scale"],
                          int(g["context_lens"].max()))
    check_device_status()
    err = (out.float().cpu() - g["out_fp32"]).abs().max().item()
    ref_err = (g["out"].float() - g["out_fp32"]).abs().max().item()
    assert err <= 2 * ref_err + 1e-5, (err, ref_err)


@pytest.mark.parametrize("group,head_size,block_size", [(1, 64, 16), (2, 128, 32), (8, 128, 16), (8, 64, 256),
                                                       (4, 32, 128)])
def test_unused_cache_rows_may_hold_anything(group, head_size, block_size):
    """Rows past a sequence's context length (and blocks no sequence uses) are never part of the
    result, even when they hold NaN: the reference masks them at load time (paged.py:246-262)."""
    q, kc, vc, lens, tables, scale, mx = _case(6, 16, group, head_size, block_size, 1000, torch.float16, seed=9)
    valid = torch.zeros(NUM_BLOCKS, block_size, dtype=torch.bool, device=device())
    for s_, n in enumerate(lens.tolist()):
        for i in range((n + block_size - 1) // block_size):
            valid[tables[s_, i], : min(block_size, n - i * block_size)] = True
    ref = oracle_paged(q, kc, vc, tables, lens, scale)
    hole = ~valid[:, None, :, None].expand_as(kc)
    kc = kc.masked_fill(hole, float("nan"))
    vc = vc.masked_fill(hole, float("nan"))
    out = paged_attention(q, kc, vc, lens, tables, scale, mx)
    check_device_status()
    assert not torch.isnan(out).any()
    assert torch.allclose(out.float(), ref.float(), atol=2e-3, rtol=1e-5)


def test_paged_attention_rejects_unsupported_blocks():
    q, kc, vc, lens, tables, scale, mx = _case(2, 8, 1, 64, 16, 100, torch.float16)
    kc24 = torch.zeros(10, 8, 24, 64, dtype=torch.float16, device=device())
    with pytest.raises(RuntimeError, match="power of two"):
        paged_attention(q, kc24, kc24.clone(), lens, tables, scale, mx)

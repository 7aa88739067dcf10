"""Decode attention over a paged K/V cache: the reference's ``flag_attn.paged_attention``
(``paged.py:20-170``) on this library's decode kernels.

Same arguments and result as the reference operator. One query token per sequence attends to the
``context_lens[s]`` keys of its sequence, which live in cache blocks of ``block_size`` keys addressed
through ``block_tables``. With one or two query heads per KV head the work is a pure stream over the
cache and runs in the register-resident streaming kernel; with more, all query heads of a KV head share
one tensor-core tile, whose K/V tiles the TMA producer gathers block by block.
"""
from __future__ import annotations

import torch

from . import _lib
from .flash import _SPLIT_COUNTS, _sm_count, _status_word, _tma_ready

_SUPPORTED_HEAD_SIZES = (16, 32, 64, 128)


def _as4(x: torch.Tensor) -> _lib.Tensor4:
    """[num_seqs, heads, D] described as [num_seqs, heads, 1, D]."""
    return _lib.Tensor4(x.data_ptr(), (_lib.c_int64 * 4)(x.stride(0), x.stride(1), x.shape[2], x.stride(2)))


def paged_attention(query, key_cache, value_cache, context_lens, block_tables, attn_scale, max_context_len,
                    num_splits=0):
    """
    Arguments (as ``paged.py:20-29``):
        query: ``[num_seqs, num_kv_heads * query_group_size, head_size]`` fp16/bf16.
        key_cache, value_cache: ``[num_blocks, num_kv_heads, kv_block_size, head_size]``.
        context_lens: ``[num_seqs]`` integer tensor.
        block_tables: ``[num_seqs, max_num_blocks_per_seq]`` integer tensor.
        attn_scale: softmax scale.
        max_context_len: largest entry of ``context_lens`` (sizes the key partition).
        num_splits: 0 = chosen by the library; a positive value is used as given (the result does not
            depend on it beyond fp32 rounding).
    Returns ``[num_seqs, num_query_heads, head_size]`` in ``query.dtype``.
    """
    if not (query.is_cuda and key_cache.is_cuda and value_cache.is_cuda):
        raise RuntimeError("paged_attention runs on CUDA tensors only (no CPU fallback)")
    if query.dim() != 3 or key_cache.dim() != 4 or value_cache.shape != key_cache.shape:
        raise ValueError("expected query [seqs, heads, D] and key/value caches [blocks, kv_heads, block, D]")
    num_seqs, Hq, D = query.shape
    num_blocks, Hkv, block_size, head_size = key_cache.shape
    assert head_size == D and D in _SUPPORTED_HEAD_SIZES, f"head_size={head_size}"
    assert Hq % Hkv == 0, "number of query heads must be a multiple of the number of KV heads"
    if not (query.dtype == key_cache.dtype == value_cache.dtype) or query.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("query and caches must share dtype float16 or bfloat16")
    max_context_len = int(max_context_len)
    assert max_context_len >= 1
    device = query.device

    query, key_cache, value_cache = _tma_ready(query), _tma_ready(key_cache), _tma_ready(value_cache)
    if context_lens.dtype != torch.int32 or context_lens.device != device or not context_lens.is_contiguous():
        context_lens = context_lens.to(device=device, dtype=torch.int32).contiguous()
    if block_tables.dtype != torch.int32 or block_tables.device != device or block_tables.stride(-1) != 1:
        block_tables = block_tables.to(device=device, dtype=torch.int32).contiguous()
    lib = _lib.load()
    out = torch.empty((num_seqs, Hq, D), dtype=query.dtype, device=device)
    num_sms = _sm_count(device)
    if num_splits and num_splits > 0:
        S = int(num_splits)
    else:
        key = (num_seqs, Hq, Hkv, 1, max_context_len, D, num_sms)
        S = _SPLIT_COUNTS.get(key)
        if S is None:
            S = _SPLIT_COUNTS[key] = int(lib.b200attn_splitkv_num_splits(num_seqs, Hq, Hkv, 1, max_context_len, D, num_sms))
    rows = num_seqs * Hq

    def launch():
        buf = torch.empty(rows * (S * D + S + 1), dtype=torch.float32, device=device)
        part_o = buf.data_ptr()
        part_l = part_o + 4 * rows * S * D
        lse = part_l + 4 * rows * S
        p = _lib.PagedParams(
            _as4(query), _lib.tensor4(key_cache), _lib.tensor4(value_cache), _as4(out),
            block_tables.data_ptr(), block_tables.stride(0), context_lens.data_ptr(),
            lse, part_o, part_l, num_seqs, Hq, Hkv, D, block_size, num_blocks, max_context_len, S,
            _lib.dtype_code(query.dtype), float(attn_scale), _status_word(device).data_ptr())
        _lib.check(lib.b200attn_paged_attention(p, _lib.current_stream_ptr(device)), "b200attn_paged_attention")

    if device.index == torch.cuda.current_device():
        launch()
    else:
        with torch.cuda.device(device):
            launch()
    return out

"""CPU/GPU restatement of the reference's PyTorch paged attention. TEST INFRASTRUCTURE ONLY: imported
by tests/, never by the product.

Follows ``src/flag_attn/testing/paged.py:19-66``: per sequence, gather the first ``context_len`` keys
and values through the block table (key ``j`` = row ``j % block`` of block ``table[j // block]``),
repeat them over the query heads of each KV head, ``softmax(q K^T * scale)`` in fp32 and ``P V`` in
fp32, result cast to the value dtype. Pinned by ``tests/golden/paged_*.npz``, which hold the
reference function's own outputs (``tests/test_oracle_golden.py``).
"""
from __future__ import annotations

import torch


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, scale):
    """query [S, Hq, D]; caches [blocks, Hkv, block, D]; returns [S, Hq, D] in the cache dtype."""
    num_seqs, Hq, D = query.shape
    _, Hkv, block, _ = value_cache.shape
    group = Hq // Hkv
    out = torch.empty_like(query, dtype=value_cache.dtype)
    tables = block_tables.to("cpu").tolist()
    lens = context_lens.to("cpu").tolist()
    for s in range(num_seqs):
        n = int(lens[s])
        pos = torch.arange(n, device=query.device)
        blk = torch.tensor(tables[s], device=query.device, dtype=torch.long)[pos // block]
        keys = key_cache[blk, :, pos % block, :]      # [n, Hkv, D]
        values = value_cache[blk, :, pos % block, :]
        if group > 1:
            keys = keys.repeat_interleave(group, dim=1)
            values = values.repeat_interleave(group, dim=1)
        scores = torch.einsum("hd,nhd->hn", query[s].float(), keys.float()) * scale
        probs = torch.softmax(scores, dim=-1)
        out[s] = torch.einsum("hn,nhd->hd", probs, values.float()).to(value_cache.dtype)
    return out

"""Multi-GPU partitioning of ``flash_attention`` without any collective.

The operator is independent per (batch, KV head): all query heads that share a KV head stay on one
rank, so dK/dV need no cross-rank reduction. ``unit_range`` assigns each rank a contiguous range
of the ``B * Hkv`` units; ``shard`` returns the matching views of q, k, v (and anything shaped
like q), one piece per batch the range touches. One process per GPU runs its pieces through the
ordinary ``flash_attention``; results are bit-identical to the corresponding slices of a
single-GPU run.
"""
from __future__ import annotations

from typing import Iterator

import torch


def unit_range(num_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split: the first ``num_units % world`` ranks get one extra unit."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(num_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def pieces(B: int, Hkv: int, rank: int, world: int) -> Iterator[tuple[int, int, int]]:
    """Yields ``(batch, kv_head_begin, kv_head_end)`` covering this rank's units."""
    lo, hi = unit_range(B * Hkv, rank, world)
    while lo < hi:
        b, h0 = divmod(lo, Hkv)
        h1 = min(Hkv, h0 + (hi - lo))
        yield b, h0, h1
        lo += h1 - h0


def shard(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int, *like_q: torch.Tensor):
    """List of ``(q_piece, k_piece, v_piece, *like_q_pieces)`` views owned by ``rank``."""
    B, Hq = q.shape[:2]
    Hkv = k.shape[1]
    groups = Hq // Hkv
    out = []
    for b, h0, h1 in pieces(B, Hkv, rank, world):
        qs = slice(h0 * groups, h1 * groups)
        out.append((q[b:b + 1, qs], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1], *(t[b:b + 1, qs] for t in like_q)))
    return out

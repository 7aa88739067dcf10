"""Split-KV dispatch rule of the reference (``split_kv.py:245-278``, used at ``flash.py:73-75``).

``flash_attention`` switches to a split-KV forward when the plain grid would leave most SMs idle
(decode-like shapes). The rule is evaluated with the reference's split-KV tile (16 query rows x
128 keys) so that the same calls take the same branch, including the branch's "no dropout"
restriction.
"""
from __future__ import annotations

import math

SPLIT_BLOCK_M = 16
SPLIT_BLOCK_N = 128
MAX_SPLITS = 128


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


def choose_num_splits(B: int, H: int, M: int, N: int, num_sms: int,
                      block_m: int = SPLIT_BLOCK_M, block_n: int = SPLIT_BLOCK_N,
                      max_splits: int = MAX_SPLITS) -> int:
    """Number of KV splits (1 = no split): the smallest admissible split count whose wave
    efficiency reaches 85 % of the best one, when fewer than 0.8 x num_sms CTAs exist unsplit."""
    ctas = B * H * _cdiv(M, block_m)
    if ctas >= 0.8 * num_sms:
        return 1
    n_blocks = _cdiv(N, block_n)
    limit = min(num_sms, n_blocks, max_splits)
    candidates = []
    best = 0.0
    for s in range(1, limit + 1):
        per_split = _cdiv(n_blocks, s)
        if s != 1 and per_split * s - n_blocks >= per_split:
            continue  # some split would be empty
        waves = ctas * s / num_sms
        eff = waves / math.ceil(waves)
        candidates.append((s, eff))
        best = max(best, eff)
    for s, eff in candidates:
        if eff >= 0.85 * best:
            return s
    return 1

"""numpy restatement of the dropout keep-mask the reference draws with Triton's Philox.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Algorithm (published Philox-4x32 of Salmon et al., as parameterised by Triton's
``triton/language/random.py``; the reference calls it at ``flash.py:474-477`` and
``testing/dropout.py:19-30``):

* key = (seed low 32 bits, seed high 32 bits); counter = (c0, c1, 0, 0) where (c0, c1) are the low
  / high words of ``offset + linear_index``; 6 rounds with multipliers 0xD2511F53 / 0xCD9E8D57 and
  key increments 0x9E3779B9 / 0xBB67AE85; only output word 0 is used.
* the word is read as int32 ``x``, folded to ``x if x >= 0 else -x - 1``, scaled by
  4.6566127342e-10 in fp32, and the element is kept iff that uniform is ``> dropout_p``.
* Triton types a kernel argument that fits in int32 as i32: when ``offset < 2**31`` the counter
  arithmetic is 32-bit and the high counter word is 0; otherwise it is 64-bit.
"""
from __future__ import annotations

import numpy as np

_ROUND_A = np.uint64(0xD2511F53)
_ROUND_B = np.uint64(0xCD9E8D57)
_KEY_A = 0x9E3779B9
_KEY_B = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)
_SHIFT32 = np.uint64(32)


def philox6_word0(seed: int, counter: np.ndarray, wide: bool) -> np.ndarray:
    """Output word 0 of 6-round Philox-4x32 for every 64-bit ``counter`` (uint64 array)."""
    seed &= 0xFFFFFFFFFFFFFFFF
    k0, k1 = seed & 0xFFFFFFFF, seed >> 32
    counter = np.asarray(counter, dtype=np.uint64)
    c0 = counter & _MASK32
    c1 = (counter >> _SHIFT32) if wide else np.zeros_like(counter)
    c2 = np.zeros_like(counter)
    c3 = np.zeros_like(counter)
    for _ in range(6):
        prod_a = _ROUND_A * c0            # < 2**64, exact in uint64
        prod_b = _ROUND_B * c2
        n0 = (prod_b >> _SHIFT32) ^ c1 ^ np.uint64(k0)
        n2 = (prod_a >> _SHIFT32) ^ c3 ^ np.uint64(k1)
        c1 = prod_b & _MASK32
        c3 = prod_a & _MASK32
        c0, c2 = n0, n2
        k0 = (k0 + _KEY_A) & 0xFFFFFFFF
        k1 = (k1 + _KEY_B) & 0xFFFFFFFF
    return c0.astype(np.uint32)


def uniform_from_word(word: np.ndarray) -> np.ndarray:
    x = word.astype(np.uint32).view(np.int32).astype(np.int64)
    folded = np.where(x < 0, -x - 1, x)
    return folded.astype(np.float32) * np.float32(4.6566127342e-10)


def dropout_keep_mask(B: int, H: int, M: int, N: int, dropout_p: float, seed: int, offset: int) -> np.ndarray:
    """Boolean ``[B, H, M, N]`` keep-mask for the given Philox ``(seed, offset)``."""
    total = B * H * M * N
    if dropout_p == 0:
        return np.ones((B, H, M, N), dtype=bool)
    wide = offset >= 2**31
    out = np.empty(total, dtype=bool)
    step = 1 << 22
    for lo in range(0, total, step):
        idx = np.arange(lo, min(total, lo + step), dtype=np.uint64)
        ctr = idx + np.uint64(offset & 0xFFFFFFFFFFFFFFFF)   # wraps modulo 2**64 like the kernel
        u = uniform_from_word(philox6_word0(seed, ctr, wide))
        out[lo:lo + len(idx)] = u > np.float32(dropout_p)
    return out.reshape(B, H, M, N)

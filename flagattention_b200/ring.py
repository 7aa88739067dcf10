"""Ring-KV sequence-parallel forward for long causal contexts (one process per GPU).

The sequence is cut into ``2 * P`` chunks; rank ``r`` owns chunks ``r`` and ``2P-1-r`` of q, k and v
("zig-zag"), which gives every rank the same amount of causal work. K/V shards travel around the
ring with ``torch.distributed`` point-to-point transfers (NCCL over NVLink on GPUs), landing in a
local double buffer while the current step computes, so the kernels only ever read local memory. Each
ring step produces a partial result (O normalised over the keys of that step, and its
log-normaliser) with the ordinary forward kernel; partials are folded into an fp32 accumulator
with the library's log-sum-exp merge (the algebra of the reference's split-KV combine,
``split_kv.py:199-231``). Steps that causality masks completely are never launched.

The reference has no multi-GPU path; this is the second mode of the 32k-token configuration.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib
from .status import poll as _status_word


LAUNCHES = 0  # kernels launched by this module in this process (read by the benchmark)


def zigzag_chunks(rank: int, world: int) -> tuple[int, int]:
    return rank, 2 * world - 1 - rank


def zigzag_shard(x: torch.Tensor, rank: int, world: int, dim: int = 2) -> torch.Tensor:
    """This rank's two chunks of a full-sequence tensor, concatenated (low chunk first)."""
    chunks = x.chunk(2 * world, dim=dim)
    lo, hi = zigzag_chunks(rank, world)
    return torch.cat([chunks[lo], chunks[hi]], dim=dim).contiguous()


def zigzag_unshard(parts: list[torch.Tensor], dim: int = 2) -> torch.Tensor:
    """Inverse of ``zigzag_shard`` given every rank's local tensor in rank order."""
    world = len(parts)
    chunks: list[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=dim)
        lo, hi = zigzag_chunks(r, world)
        chunks[lo], chunks[hi] = a, b
    return torch.cat(chunks, dim=dim)


def plan_step(rank: int, src: int):
    """Attention calls of one ring step, for local q = [q_lo; q_hi] and the K/V shard of rank
    ``src`` = [kv_lo; kv_hi]. Each entry is ``(q_half, kv_halves, causal)`` with ``q_half`` in
    {"lo", "hi", "both"} and ``kv_halves`` in {"lo", "both"}; causal calls are bottom-right aligned."""
    if src == rank:
        return [("lo", "lo", True), ("hi", "both", True)]
    if src < rank:
        return [("both", "lo", False)]      # both local chunks come after chunk `src`
    return [("hi", "both", False)]          # only the late local chunk sees rank `src`'s chunks


def _cuda_partial(q, k, v, causal, sm_scale):
    """Forward kernel through the C ABI with an fp32 output; returns (o fp32, lse)."""
    lib = _lib.load()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    o = torch.empty((B, Hq, M, D), dtype=torch.float32, device=q.device)
    lse = torch.empty((B, Hq, M), dtype=torch.float32, device=q.device)
    p = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(),
                       B, Hq, Hk, M, N, D, _lib.dtype_code(q.dtype), _lib.F32, int(causal), float(sm_scale),
                       0.0, 0, 0, _status_word(q.device).data_ptr())
    _lib.check(lib.b200attn_fwd(p, _lib.current_stream_ptr(q.device)), "b200attn_fwd")
    global LAUNCHES
    LAUNCHES += 1
    return o, lse


def _cuda_merge(o_acc, lse_acc, acc_row0, o_part, lse_part, part_row0, rows, first):
    """Folds rows [part_row0, part_row0+rows) of a partial into rows [acc_row0, ...) of the
    accumulator, for every (batch, head), with the library's merge kernel."""
    global LAUNCHES
    LAUNCHES += 1
    lib = _lib.load()
    heads = o_acc.shape[0] * o_acc.shape[1]
    _lib.check(lib.b200attn_merge_partial(o_acc.data_ptr(), lse_acc.data_ptr(), o_part.data_ptr(),
                                          lse_part.data_ptr(), heads, rows, o_acc.shape[-1],
                                          o_acc.shape[2], acc_row0, o_part.shape[2], part_row0, int(first),
                                          _lib.current_stream_ptr(o_acc.device)), "b200attn_merge_partial")


def ring_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: Optional[float] = None,
                           group=None, partial_fn: Optional[Callable] = None,
                           merge_fn: Optional[Callable] = None):
    """Causal attention over a zig-zag sharded sequence.

    ``q`` is ``[B, Hq, 2c, D]`` and ``k``/``v`` ``[B, Hkv, 2c, D]``: this rank's two chunks of length
    ``c``. Returns ``(o, lse)`` for the local rows, ``o`` in q's dtype. ``partial_fn(q, k, v, causal,
    sm_scale) -> (o fp32, lse)`` and ``merge_fn(o_acc, lse_acc, acc_row0, o_part, lse_part, part_row0, rows, first)`` default to
    the CUDA library; they exist so the ring logic can be exercised on CPU ranks.
    """
    partial_fn = partial_fn or _cuda_partial
    merge_fn = merge_fn or _cuda_merge
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, Hq, L, D = q.shape
    assert L % 2 == 0 and k.shape[2] == L and v.shape[2] == L
    c = L // 2
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q = q.contiguous()
    o_acc = torch.empty((B, Hq, L, D), dtype=torch.float32, device=q.device)
    lse_acc = torch.empty((B, Hq, L), dtype=torch.float32, device=q.device)
    started = {"lo": False, "hi": False}

    kv_cur = torch.stack([k.contiguous(), v.contiguous()])       # [2, B, Hkv, 2c, D]
    kv_next = torch.empty_like(kv_cur)
    send_to = (rank + 1) % world
    recv_from = (rank - 1) % world

    for step in range(world):
        src = (rank - step) % world
        reqs = []
        if step + 1 < world:
            ops = [dist.P2POp(dist.isend, kv_cur, send_to, group), dist.P2POp(dist.irecv, kv_next, recv_from, group)]
            reqs = dist.batch_isend_irecv(ops)
        k_s, v_s = kv_cur[0], kv_cur[1]
        for q_half, kv_halves, causal in plan_step(rank, src):
            rows = {"lo": slice(0, c), "hi": slice(c, L), "both": slice(0, L)}[q_half]
            keys = slice(0, c) if kv_halves == "lo" else slice(0, L)
            o_p, lse_p = partial_fn(q[:, :, rows], k_s[:, :, keys], v_s[:, :, keys], causal, sm_scale)
            for half in (("lo", "hi") if q_half == "both" else (q_half,)):
                acc_row0 = 0 if half == "lo" else c
                part_row0 = acc_row0 if q_half == "both" else 0
                merge_fn(o_acc, lse_acc, acc_row0, o_p, lse_p, part_row0, c, not started[half])
                started[half] = True
        for r in reqs:
            r.wait()
        if step + 1 < world:
            kv_cur, kv_next = kv_next, kv_cur
    return o_acc.to(q.dtype), lse_acc

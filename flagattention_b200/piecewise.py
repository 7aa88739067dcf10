"""Piecewise attention: the reference's ``flag_attn.piecewise_attention`` (``piecewise.py:39-235``) on
this library's kernels.

``S[m, n] = q2[m]·k2[n]`` where the distance ``m + (N - M) - n`` is at least ``dist_threshold`` and
``q1[m]·k1[n]`` elsewhere; one softmax over the whole row; ``o = P v``. The two regions are disjoint
bands of the distance, so the row's softmax is the normaliser-weighted merge of two band-limited
attentions: the forward runs the forward kernel once per (q, k) pair with the band mask of its region
(``b200attn_fwd`` with ``band``), writing fp32 partial outputs and log-normalisers, and merges them
(``b200attn_merge_partial_store``, the algebra of the split-KV combine, rounding straight into the
output). The backward runs the backward
kernels once per pair with the same bands, both on the merged log-normaliser and on ``delta`` of the
merged output; each call yields its pair's dQ and dK, and the two dV contributions are added.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from .flash import _status_word, _tma_ready

_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128)


def _bands(w: int, causal: bool):
    """(dist_min, dist_max) of the near region (first pair) and of the far region (second pair)."""
    near = (0 if causal else _lib.BAND_OPEN_MIN, w)
    far = (max(w, 0) if causal else w, _lib.BAND_OPEN_MAX)
    return near, far


class PiecewiseAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q1, k1, q2, k2, v, w, causal, sm_scale):
        Dq1, Dk1, Dq2, Dk2, Dv = q1.shape[-1], k1.shape[-1], q2.shape[-1], k2.shape[-1], v.shape[-1]
        assert Dq1 == Dk1 == Dq2 == Dk2 == Dv
        assert Dk1 in _SUPPORTED_HEAD_DIMS
        B, H, M, D = q1.shape
        N = k1.shape[2]
        if not all(t.is_cuda for t in (q1, k1, q2, k2, v)):
            raise RuntimeError("piecewise_attention runs on CUDA tensors only (no CPU fallback)")
        if len({t.dtype for t in (q1, k1, q2, k2, v)}) != 1 or q1.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("q1, k1, q2, k2, v must share dtype float16 or bfloat16")
        if q2.shape != q1.shape or k2.shape != k1.shape or v.shape != k1.shape or k1.shape[:2] != (B, H):
            raise ValueError("expected q1, q2 of shape [B, H, M, D] and k1, k2, v of shape [B, H, N, D]")
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        w = int(w)
        q1, k1, q2, k2, v = (_tma_ready(t) for t in (q1, k1, q2, k2, v))
        lib = _lib.load()
        device = q1.device
        dt = _lib.dtype_code(q1.dtype)
        with torch.cuda.device(device):
            stream = _lib.current_stream_ptr(device)
            status = _status_word(device)
            parts = []
            for (q, k), (dmin, dmax) in zip(((q1, k1), (q2, k2)), _bands(w, bool(causal))):
                o_part = torch.empty((B, H, M, D), dtype=torch.float32, device=device)
                l_part = torch.empty((B, H, M), dtype=torch.float32, device=device)
                fp = _lib.FwdParams(
                    _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o_part), l_part.data_ptr(),
                    B, H, H, M, N, D, dt, _lib.dtype_code(torch.float32), int(bool(causal)), float(sm_scale),
                    0.0, 0, 0, status.data_ptr(), 1, dmin, dmax)
                _lib.check(lib.b200attn_fwd(fp, stream), "b200attn_fwd")
                parts.append((o_part, l_part))
            (o_acc, L), (o_far, l_far) = parts
            o = torch.empty_like(q1)
            _lib.check(lib.b200attn_merge_partial_store(o_acc.data_ptr(), L.data_ptr(), o_far.data_ptr(),
                                                        l_far.data_ptr(), B, H, M, D, _lib.tensor4(o), dt, stream),
                       "b200attn_merge_partial_store")
        ctx.save_for_backward(q1, k1, q2, k2, v, o, L)
        ctx.sm_scale = sm_scale
        ctx.causal = bool(causal)
        ctx.w = w
        return o

    @staticmethod
    def backward(ctx, do):
        q1, k1, q2, k2, v, o, L = ctx.saved_tensors
        B, H, M, D = q1.shape
        N = k1.shape[2]
        do = _tma_ready(do)
        o = _tma_ready(o)
        lib = _lib.load()
        device = q1.device
        dt = _lib.dtype_code(q1.dtype)
        with torch.cuda.device(device):
            stream = _lib.current_stream_ptr(device)
            status = _status_word(device)
            delta = torch.empty_like(L)
            workspace = torch.empty(max(lib.b200attn_bwd_workspace_bytes(B, H, H, M, N, D), 4) // 4,
                                    dtype=torch.float32, device=device)
            unfused = _lib.BWD_STAGE_UNFUSED if torch.are_deterministic_algorithms_enabled() else 0
            grads = []
            stages = _lib.BWD_STAGE_ALL  # the second call reuses the statistics the first one prepared
            dv = torch.empty((B, H, N, D), dtype=v.dtype, device=device)
            for (q, k), (dmin, dmax) in zip(((q1, k1), (q2, k2)), _bands(ctx.w, ctx.causal)):
                dq = torch.empty((B, H, M, D), dtype=q.dtype, device=device)
                dk = torch.empty((B, H, N, D), dtype=k.dtype, device=device)
                bp = _lib.BwdParams(
                    _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), _lib.tensor4(do),
                    _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv),
                    L.data_ptr(), delta.data_ptr(), workspace.data_ptr(),
                    B, H, H, M, N, D, dt, dt, int(ctx.causal), float(ctx.sm_scale), 0.0, 0, 0, status.data_ptr(),
                    1, dmin, dmax, None, int(bool(grads)))   # the far region's dV is added onto the near one's
                _lib.check(lib.b200attn_bwd_stages(bp, stream, stages | unfused), "b200attn_bwd_stages")
                grads.append((dq, dk))
                stages = _lib.BWD_STAGE_KV | _lib.BWD_STAGE_Q
            (dq1, dk1), (dq2, dk2) = grads
        return dq1, dk1, dq2, dk2, dv, None, None, None


def piecewise_attention(q1, k1, q2, k2, v, dist_threshold, causal=False, sm_scale=None):
    """
    Arguments (as ``piecewise.py:183-205``):
        q1, q2: ``(batch, heads, seqlen_q, headdim)``; k1, k2, v: ``(batch, heads, seqlen_k, headdim)``.
        dist_threshold: scores at distance ``m + seqlen_k - seqlen_q - n >= dist_threshold`` come from the
            second (q, k) pair, the others from the first.
        causal: bottom-right aligned causal mask.
        sm_scale: softmax scale, default ``1/sqrt(headdim)``.
    Returns ``(batch, heads, seqlen_q, headdim)``; differentiable in all five tensors.
    """
    return PiecewiseAttentionFunction.apply(q1, k1, q2, k2, v, dist_threshold, causal, sm_scale)

"""CPU/GPU restatement of the reference's PyTorch piecewise attention. TEST INFRASTRUCTURE ONLY:
imported by tests/, never by the product.

Follows ``src/flag_attn/testing/piecewise.py:19-49``: ``S1 = q1 k1^T``, ``S2 = q2 k2^T``, the second where
``m + (N - M) - n >= dist_threshold``, scaled; causal positions filled with the dtype's minimum; fp32
softmax cast to the value dtype and re-masked to zero; ``P v``. Gradients come from autograd through
this function. Pinned by ``tests/golden/piecewise_*.npz`` (outputs and gradients of the reference
function itself).
"""
from __future__ import annotations

import math

import torch


def piecewise_attention(q1, k1, q2, k2, v, dist_threshold, causal=False, sm_scale=None, upcast=False):
    in_dtype = q1.dtype
    if upcast:
        q1, k1, q2, k2, v = (t.float() for t in (q1, k1, q2, k2, v))
    D = q1.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    M, N = q1.shape[-2], k1.shape[-2]
    dist = (torch.arange(M, device=q1.device).unsqueeze(-1) + (N - M)) - torch.arange(N, device=q1.device)
    s1 = torch.matmul(q1, k1.transpose(2, 3))
    s2 = torch.matmul(q2, k2.transpose(2, 3))
    s = torch.where(dist >= dist_threshold, s2, s1) * sm_scale
    if causal:
        s = torch.where(dist >= 0, s, torch.finfo(s.dtype).min)
    p = torch.softmax(s, dim=-1, dtype=torch.float32).to(v.dtype)
    if causal:
        p = torch.where(dist >= 0, p, 0.0)
    return torch.matmul(p, v).to(in_dtype)

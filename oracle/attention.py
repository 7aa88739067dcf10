"""PyTorch restatement of the reference's attention math, forward and backward.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``). Runs on whatever device its inputs are on;
the tests use it on CPU for small cases and on the GPU (as the checker, never as the product) for
the reference's large test shapes.

Forward follows ``src/flag_attn/testing/flash.py:19-84`` step for step: optional fp32 upcast, KV
heads repeated over their query group, ``S = Q K^T * sm_scale``, bottom-right aligned causal mask
``m + (N - M) >= n``, fp32 ``logsumexp`` / softmax, masked probabilities forced to 0 (so rows with
no visible key give 0 instead of NaN), total attention = column sums of P before dropout, then
``O = (dropout(P) -> v.dtype) V / (1 - p)`` cast back to the input dtype.

Backward is the closed form the reference's kernels implement (``flash.py:591-931``):
``dV = Pd^T dO``, ``dP = dO V^T`` (masked and scaled like Pd), ``dS = P * (dP - rowsum(dO*O))``,
``dQ = dS K * sm_scale``, ``dK = dS^T Q * sm_scale``, with dK/dV summed over each KV head's query
group. It is validated against ``torch.autograd`` through the forward in the oracle's own tests.
"""
from __future__ import annotations

import math

import torch


def _visible(M: int, N: int, device) -> torch.Tensor:
    rows = torch.arange(M, device=device).unsqueeze(-1)
    cols = torch.arange(N, device=device)
    return rows + (N - M) >= cols


def attention_forward(q, k, v, causal=False, sm_scale=None, dropout_p=0.0, dropout_mask=None,
                      upcast=False, return_log_normalizer=False, return_total_attention=False):
    """Returns ``o`` or ``(o, log_normalizer|None, total_attention|None)`` like the reference's
    ``flag_attn.testing.flash_attention``."""
    in_dtype = q.dtype
    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    assert Hq % Hk == 0
    groups = Hq // Hk
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    if groups > 1:
        k = k.repeat_interleave(groups, dim=1)
        v = v.repeat_interleave(groups, dim=1)

    scores = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    vis = _visible(M, N, q.device) if causal else None
    if causal:
        scores = torch.where(vis, scores, float("-inf"))
    scores = scores.float()
    lse = torch.logsumexp(scores, dim=-1) if return_log_normalizer else None
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32)
    if causal:
        probs = torch.where(vis, probs, 0.0)
    tot = probs.sum(dim=-2) if return_total_attention else None
    if dropout_mask is not None:
        probs = probs.masked_fill(~dropout_mask, 0.0)
    out = torch.matmul(probs.to(v.dtype), v) * (1.0 / (1.0 - dropout_p))
    out = out.to(in_dtype)
    if return_log_normalizer or return_total_attention:
        return out, lse, tot
    return out


def attention_backward(q, k, v, do, causal=False, sm_scale=None, dropout_p=0.0, dropout_mask=None):
    """fp32 closed-form gradients ``(dq, dk, dv)`` of ``sum(o * do)``; inputs are upcast to fp32."""
    q32, k32, v32, do32 = q.float(), k.float(), v.float(), do.float()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    groups = Hq // Hk
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    kx = k32.repeat_interleave(groups, dim=1) if groups > 1 else k32
    vx = v32.repeat_interleave(groups, dim=1) if groups > 1 else v32
    scores = torch.matmul(q32, kx.transpose(2, 3)) * sm_scale
    if causal:
        vis = _visible(M, N, q.device)
        scores = torch.where(vis, scores, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    if causal:
        probs = torch.where(vis, probs, 0.0)
    probs = torch.nan_to_num(probs, nan=0.0)
    keep_scale = 1.0 / (1.0 - dropout_p)
    if dropout_mask is not None:
        dropped = probs.masked_fill(~dropout_mask, 0.0) * keep_scale
    else:
        dropped = probs * keep_scale
    out = torch.matmul(dropped, vx)
    dv_full = torch.matmul(dropped.transpose(2, 3), do32)
    dp = torch.matmul(do32, vx.transpose(2, 3)) * keep_scale
    if dropout_mask is not None:
        dp = dp.masked_fill(~dropout_mask, 0.0)
    delta = (out * do32).sum(-1, keepdim=True)
    ds = probs * (dp - delta)
    dq = torch.matmul(ds, kx) * sm_scale
    dk_full = torch.matmul(ds.transpose(2, 3), q32) * sm_scale
    dk = dk_full.reshape(B, Hk, groups, N, D).sum(2)
    dv = dv_full.reshape(B, Hk, groups, N, D).sum(2)
    return dq, dk, dv


def autograd_backward(q, k, v, do, causal=False, sm_scale=None, dropout_p=0.0, dropout_mask=None,
                      upcast=True):
    """Gradients through ``attention_forward`` by ``torch.autograd`` (what the reference's tests do,
    ``tests/flag_attn/test_flash_attention.py:206-216``)."""
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = attention_forward(q, k, v, causal, sm_scale, dropout_p, dropout_mask, upcast=upcast)
    return torch.autograd.grad(out, (q, k, v), do)


def max_abs_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.float() - b.float()).abs().max().item()


def within_reference_tolerance(hyp, low_precision, exact, slack=1e-5, factor=2.0):
    """The reference's acceptance rule (``test_flash_attention.py:120-124``): the error of the
    kernel against the fp32 result may be at most ``factor`` x the error of the same math done in
    the input dtype, plus ``slack``. Returns ``(ok, hyp_err, lowp_err)``."""
    hyp_err = max_abs_diff(hyp, exact)
    low_err = max_abs_diff(low_precision, exact)
    return hyp_err <= factor * low_err + slack, hyp_err, low_err

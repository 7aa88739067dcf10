"""Parity at the full sizes of the five benchmark configurations.

The oracle cannot materialise whole score matrices at these sizes, so each configuration is checked
through (a) the oracle on a slice that is independent of the rest (one batch / KV group, or a band
of query rows with the keys it can see) and (b) size-independent properties: rows of P sum to one,
total attention sums to the number of queries, shard-by-head results are bit-identical to the
corresponding slice of the full run, repeated runs are bit-identical."""
import math

import pytest
import torch

from flagattention_b200 import check_device_status, flash_attention
from gpu_util import (assert_2x_rule, attention_backward, attention_forward, clean, device,
                      kernel_dropout_mask, max_abs_diff)

pytestmark = pytest.mark.gpu


def _gen(shape, dtype, seed, uniform=False):
    g = torch.Generator(device=device()).manual_seed(seed)
    if uniform:
        return (torch.rand(shape, device=device(), generator=g) * 2 - 1).to(dtype)
    return torch.randn(shape, device=device(), dtype=dtype, generator=g)


def test_c2_gqa_prefill_train_step():
    B, Hq, Hk, M, N, D = 4, 32, 8, 4096, 4096, 128
    dt = torch.bfloat16
    q, k, v, do = (_gen(s, dt, i) for i, s in enumerate([(B, Hq, M, D), (B, Hk, N, D), (B, Hk, N, D), (B, Hq, M, D)]))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    o, lse, _, _, _ = flash_attention(q, k, v, causal=True, return_log_normalizer=True)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    check_device_status()
    # (a) oracle on three (batch, KV group) units (query heads 4g..4g+3), each an independent unit of the problem
    for b, g in ((1, 3), (0, 0), (3, 7)):
        hs = slice(4 * g, 4 * g + 4)
        qs, ks, vs, dos = q[b:b + 1, hs].detach(), k[b:b + 1, g:g + 1].detach(), v[b:b + 1, g:g + 1].detach(), do[b:b + 1, hs]
        o_ref, l_ref, _ = attention_forward(qs, ks, vs, True, upcast=True, return_log_normalizer=True)
        o_low = attention_forward(qs, ks, vs, True, upcast=False)
        assert_2x_rule("o", o[b:b + 1, hs], o_low, o_ref)
        assert max_abs_diff(lse[b:b + 1, hs], l_ref) <= 1e-4
        rdq, rdk, rdv = attention_backward(qs, ks, vs, dos, True)
        qa, ka, va = (t.clone().requires_grad_(True) for t in (qs, ks, vs))
        g_low = torch.autograd.grad(attention_forward(qa, ka, va, True, upcast=False), (qa, ka, va), dos)
        assert_2x_rule("dq", dq[b:b + 1, hs], g_low[0], rdq)
        assert_2x_rule("dk", dk[b:b + 1, g:g + 1], g_low[1], rdk)
        assert_2x_rule("dv", dv[b:b + 1, g:g + 1], g_low[2], rdv)
    b, g = 3, 7
    # (b) sharding by (batch, KV group) reproduces the full run bit for bit
    q2, k2, v2 = (t.detach()[b:b + 1, sl].clone().requires_grad_(True)
                  for t, sl in ((q, slice(4 * g, 4 * g + 4)), (k, slice(g, g + 1)), (v, slice(g, g + 1))))
    o2, lse2, _, _, _ = flash_attention(q2, k2, v2, causal=True, return_log_normalizer=True)
    g2 = torch.autograd.grad(o2, (q2, k2, v2), dos.clone(), retain_graph=True)
    assert torch.equal(o2, o[b:b + 1, 4 * g:4 * g + 4]) and torch.equal(lse2, lse[b:b + 1, 4 * g:4 * g + 4])
    assert torch.equal(g2[1], dk[b:b + 1, g:g + 1]) and torch.equal(g2[2], dv[b:b + 1, g:g + 1])
    # dQ at D = 128 and 64 is summed over the key blocks by fp32 reductions whose order is not fixed: equal up
    # to that, and bit for bit when PyTorch's deterministic mode selects the two separate kernels.
    torch.testing.assert_close(g2[0].float(), dq[b:b + 1, 4 * g:4 * g + 4].float(), atol=2e-3, rtol=2e-2)
    torch.use_deterministic_algorithms(True)
    try:
        d_full = torch.autograd.grad(o, (q, k, v), do)
        d_part = torch.autograd.grad(o2, (q2, k2, v2), dos.clone())
    finally:
        torch.use_deterministic_algorithms(False)
    assert torch.equal(d_part[0], d_full[0][b:b + 1, 4 * g:4 * g + 4])
    assert torch.equal(d_full[1], dk) and torch.equal(d_full[2], dv)
    assert_2x_rule("dq (separate kernels)", d_full[0][b:b + 1, 4 * g:4 * g + 4], g_low[0], rdq)


def test_c3_d64_dropout_with_aux_outputs():
    B, H, M, N, D = 16, 16, 2048, 2048, 64
    dt = torch.float16
    q, k, v, do = (_gen((B, H, M, D), dt, 10 + i) for i in range(4))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

    def run():
        torch.cuda.manual_seed(20260)
        out = flash_attention(q, k, v, causal=False, dropout_p=0.1, return_log_normalizer=True,
                              return_total_attention=True, return_seed_offset=True)
        grads = torch.autograd.grad(out[0], (q, k, v), do)
        return out, grads

    (o, lse, tot, seed, offset), (dq, dk, dv) = run()
    check_device_status()
    # rows of P sum to one, so total attention sums to M for every (batch, head)
    torch.testing.assert_close(tot.sum(-1), torch.full((B, H), float(M), device=device()), atol=0.5, rtol=0)
    # oracle on batch 5, heads 2..3 with the mask rebuilt from (seed, offset)
    b, hs = 5, slice(2, 4)
    mask = kernel_dropout_mask(B, H, M, N, 0.1, seed, offset)[b:b + 1, hs]
    assert abs(1.0 - mask.float().mean().item() - 0.1) < 2e-3
    qs, ks, vs, dos = (t.detach()[b:b + 1, hs] for t in (q, k, v, do))
    o_ref, l_ref, t_ref = attention_forward(qs, ks, vs, False, dropout_p=0.1, dropout_mask=mask, upcast=True,
                                            return_log_normalizer=True, return_total_attention=True)
    o_low = attention_forward(qs, ks, vs, False, dropout_p=0.1, dropout_mask=mask, upcast=False)
    assert_2x_rule("o", o[b:b + 1, hs], o_low, o_ref)
    assert max_abs_diff(lse[b:b + 1, hs], l_ref) <= 1e-4
    assert max_abs_diff(tot[b:b + 1, hs], t_ref) <= 2e-3 * t_ref.max().item()
    rdq, rdk, rdv = attention_backward(qs, ks, vs, dos, False, dropout_p=0.1, dropout_mask=mask)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (qs, ks, vs))
    g_low = torch.autograd.grad(attention_forward(qa, ka, va, False, dropout_p=0.1, dropout_mask=mask, upcast=False),
                                (qa, ka, va), dos)
    assert_2x_rule("dq", dq[b:b + 1, hs], g_low[0], rdq)
    assert_2x_rule("dk", dk[b:b + 1, hs], g_low[1], rdk)
    assert_2x_rule("dv", dv[b:b + 1, hs], g_low[2], rdv)
    # same generator state -> bit-identical results (exact mask); dQ, which the fused pass sums by
    # fp32 reductions in no fixed order, only up to that order...
    (o2, lse2, tot2, seed2, offset2), (dq2, dk2, dv2) = run()
    assert (seed2, offset2) == (seed, offset)
    for a, b_ in ((o, o2), (lse, lse2), (tot, tot2), (dk, dk2), (dv, dv2)):
        assert torch.equal(a, b_)
    torch.testing.assert_close(dq2.float(), dq.float(), atol=1e-3, rtol=2e-2)
    # ... and bit for bit with the two separate kernels of PyTorch's deterministic mode
    torch.use_deterministic_algorithms(True)
    try:
        (_, (dq3, dk3, dv3)), (_, (dq4, dk4, dv4)) = run(), run()
    finally:
        torch.use_deterministic_algorithms(False)
    assert torch.equal(dq3, dq4) and torch.equal(dk3, dk) and torch.equal(dv3, dv) and torch.equal(dk4, dk)
    assert_2x_rule("dq (separate kernels)", dq3[b:b + 1, hs], g_low[0], rdq)


def test_c4_mqa_cross_attention_forward():
    B, Hq, Hk, M, N, D = 8, 16, 1, 512, 8192, 128
    dt = torch.bfloat16
    q = _gen((B, Hq, M, D), dt, 30)
    k = _gen((B, Hk, N, D), dt, 31)
    v = _gen((B, Hk, N, D), dt, 32, uniform=True)
    o = flash_attention(q, k, v, causal=False)
    check_device_status()
    b = 6
    o_ref = attention_forward(q[b:b + 1], k[b:b + 1], v[b:b + 1], False, upcast=True)
    o_low = attention_forward(q[b:b + 1], k[b:b + 1], v[b:b + 1], False, upcast=False)
    assert_2x_rule("o", o[b:b + 1], o_low, o_ref)
    # V = 1 -> every output element is sum_n P = 1
    ones = torch.ones_like(v)
    o1 = flash_attention(q, k, ones, causal=False)
    assert max_abs_diff(o1, torch.ones_like(o1)) <= 2 ** -7


def test_c5_long_context_causal_forward():
    B, Hq, Hk, M, N, D = 1, 64, 8, 32768, 32768, 128
    dt = torch.bfloat16
    q = _gen((B, Hq, M, D), dt, 40)
    k = _gen((B, Hk, N, D), dt, 41)
    v = _gen((B, Hk, N, D), dt, 42)
    o, lse, _, _, _ = flash_attention(q, k, v, causal=True, return_log_normalizer=True)
    check_device_status()
    r = 384
    # last r queries of head 63 see all keys: causal with M=r, N=32768 is the same alignment
    h, hk = 63, 7
    o_ref, l_ref, _ = attention_forward(q[:, h:h + 1, -r:], k[:, hk:hk + 1], v[:, hk:hk + 1], True, upcast=True,
                                        return_log_normalizer=True)
    o_low = attention_forward(q[:, h:h + 1, -r:], k[:, hk:hk + 1], v[:, hk:hk + 1], True, upcast=False)
    assert_2x_rule("o tail", o[:, h:h + 1, -r:], o_low, o_ref)
    assert max_abs_diff(lse[:, h:h + 1, -r:], l_ref) <= 2e-4
    # first r queries of head 9 only see the first r keys
    h, hk = 9, 1
    o_ref, l_ref, _ = attention_forward(q[:, h:h + 1, :r], k[:, hk:hk + 1, :r], v[:, hk:hk + 1, :r], True,
                                        upcast=True, return_log_normalizer=True)
    o_low = attention_forward(q[:, h:h + 1, :r], k[:, hk:hk + 1, :r], v[:, hk:hk + 1, :r], True, upcast=False)
    assert_2x_rule("o head", o[:, h:h + 1, :r], o_low, o_ref)
    assert max_abs_diff(lse[:, h:h + 1, :r], l_ref) <= 2e-4
    # a band in the middle of head 30: rows [m0, m0+r) see keys [0, m0+r)
    h, hk, m0 = 30, 3, 16000
    sl = slice(m0, m0 + r)
    o_ref = attention_forward(q[:, h:h + 1, sl], k[:, hk:hk + 1, :m0 + r], v[:, hk:hk + 1, :m0 + r], True, upcast=True)
    o_low = attention_forward(q[:, h:h + 1, sl], k[:, hk:hk + 1, :m0 + r], v[:, hk:hk + 1, :m0 + r], True, upcast=False)
    assert_2x_rule("o middle", o[:, h:h + 1, sl], o_low, o_ref)
    # one more head of every KV group, each on its own band of 256 rows
    for hk in range(8):
        h, m0 = hk * 8 + (3 * hk + 1) % 8, 2048 + 3800 * hk
        sl = slice(m0, m0 + 256)
        o_ref, l_ref, _ = attention_forward(q[:, h:h + 1, sl], k[:, hk:hk + 1, :m0 + 256], v[:, hk:hk + 1, :m0 + 256], True,
                                            upcast=True, return_log_normalizer=True)
        o_low = attention_forward(q[:, h:h + 1, sl], k[:, hk:hk + 1, :m0 + 256], v[:, hk:hk + 1, :m0 + 256], True, upcast=False)
        assert_2x_rule(f"o head {h}", o[:, h:h + 1, sl], o_low, o_ref)
        assert max_abs_diff(lse[:, h:h + 1, sl], l_ref) <= 2e-4
    # V = 1 -> O = 1 everywhere
    o1 = flash_attention(q, k, torch.ones_like(v), causal=True)
    assert max_abs_diff(o1, torch.ones_like(o1)) <= 2 ** -7


def test_c1_plumbing_config_matches_cpu_oracle():
    # B=1 Hq=Hkv=4 M=N=128 D=64 fp16, q/k/v ~ N(0,1) from seed 0, checked against the fp32 CPU oracle.
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 4, 128, 64, generator=g).to(torch.float16) for _ in range(3))
    o = flash_attention(q.cuda(), k.cuda(), v.cuda(), causal=False, sm_scale=1.0 / math.sqrt(64))
    o_ref = attention_forward(q, k, v, False, upcast=True)
    o_low = attention_forward(q, k, v, False, upcast=False)
    assert max_abs_diff(o.cpu(), o_ref) <= 2 * max_abs_diff(o_low, o_ref) + 1e-5

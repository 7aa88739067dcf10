"""Seeded random shapes through every operator (ragged sizes, odd head groupings, random thresholds
and cache block sizes) against the oracles, with the reference's acceptance rule. Complements the fixed
shape lists taken from the reference's tests."""
import random

import pytest
import torch

from flagattention_b200 import (check_device_status, flash_attention, flash_attention_split_kv, paged_attention,
                                piecewise_attention)
from gpu_util import assert_2x_rule, attention_forward, device, kernel_dropout_mask
from oracle.paged import paged_attention as oracle_paged
from oracle.piecewise import piecewise_attention as oracle_piecewise

pytestmark = pytest.mark.gpu


def _setup(seed):
    rnd = random.Random(seed)
    g = torch.Generator(device=device()).manual_seed(seed)
    D = rnd.choice([16, 32, 64, 128])
    dtype = rnd.choice([torch.float16, torch.bfloat16])
    return rnd, g, D, dtype


def _randn(g, dtype, *shape, grad=False):
    return torch.randn(*shape, device=device(), dtype=dtype, generator=g, requires_grad=grad)


@pytest.mark.parametrize("seed", range(16))
def test_flash_attention_random(seed):
    rnd, g, D, dtype = _setup(seed)
    B, Hk, G = rnd.randint(1, 3), rnd.choice([1, 2, 3]), rnd.choice([1, 2, 4])
    Hq = Hk * G
    M, N, causal = rnd.randint(1, 700), rnd.randint(1, 900), rnd.random() < 0.5
    # stay out of the split-KV branch, which has no backward
    M = max(M, 16 * -(-119 // (B * Hq)))
    q, k, v = _randn(g, dtype, B, Hq, M, D, grad=True), _randn(g, dtype, B, Hk, N, D, grad=True), _randn(g, dtype, B, Hk, N, D, grad=True)
    do = _randn(g, dtype, B, Hq, M, D)
    o = flash_attention(q, k, v, causal)
    grads = torch.autograd.grad(o, (q, k, v), do)
    o_ref = attention_forward(q, k, v, causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_low = attention_forward(q, k, v, causal, upcast=False)
    g_low = torch.autograd.grad(o_low, (q, k, v), do)
    check_device_status()
    assert_2x_rule("o", o, o_low, o_ref)
    for name, a, b_, c in zip(("dq", "dk", "dv"), grads, g_low, g_ref):
        assert_2x_rule(name, a, b_, c)


@pytest.mark.parametrize("seed", range(200, 212))
def test_flash_attention_random_many_items(seed):
    """Shapes with a few hundred 256-row work items (more than the GPU has SMs), so forward CTAs walk
    several items each; grouped heads, both layouts, causal or not, dropout in a quarter of the cases."""
    rnd, g, D, dtype = _setup(seed)
    Hk, G = rnd.choice([2, 4, 8, 12]), rnd.choice([1, 2, 4])
    Hq = Hk * G
    M, N, causal = rnd.randint(200, 1500), rnd.randint(1, 3000), rnd.random() < 0.6
    B = max(2, min(12, (300 * 256) // (Hq * M) + 1))
    while B > 1 and B * Hq * M * N * 4 > 4e9:
        B -= 1
    p = rnd.choice([0.0, 0.0, 0.0, 0.25])
    transposed = rnd.random() < 0.5

    def mk(H, T):
        t = _randn(g, dtype, B, T, H, D).transpose(1, 2) if transposed else _randn(g, dtype, B, H, T, D)
        return t.requires_grad_(True)

    q, k, v = mk(Hq, M), mk(Hk, N), mk(Hk, N)
    do = _randn(g, dtype, B, Hq, M, D)
    kw = {}
    if p > 0:
        o, _, _, rng_seed, rng_offset = flash_attention(q, k, v, causal, dropout_p=p, return_seed_offset=True)
        kw = dict(dropout_p=p, dropout_mask=kernel_dropout_mask(B, Hq, M, N, p, int(rng_seed), int(rng_offset)))
    else:
        o = flash_attention(q, k, v, causal)
    grads = torch.autograd.grad(o, (q, k, v), do)
    o_ref = attention_forward(q, k, v, causal, upcast=True, **kw)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    o_low = attention_forward(q, k, v, causal, upcast=False, **kw)
    g_low = torch.autograd.grad(o_low, (q, k, v), do)
    check_device_status()
    assert_2x_rule("o", o, o_low, o_ref)
    for name, a, b_, c in zip(("dq", "dk", "dv"), grads, g_low, g_ref):
        assert_2x_rule(name, a, b_, c)


@pytest.mark.parametrize("seed", range(100, 116))
def test_split_kv_random(seed):
    rnd, g, D, dtype = _setup(seed)
    B, Hk, G = rnd.randint(1, 3), rnd.choice([1, 2, 4]), rnd.choice([1, 2, 3, 8, 16, 32])
    M, N, causal = rnd.choice([1, 1, 2, 3, 5, 17]), rnd.randint(1, 20000), rnd.random() < 0.5
    q, k, v = _randn(g, dtype, B, Hk * G, M, D) * 2, _randn(g, dtype, B, Hk, N, D) * 2, _randn(g, dtype, B, Hk, N, D)
    o = flash_attention_split_kv(q, k, v, causal)
    check_device_status()
    assert_2x_rule("o", o, attention_forward(q, k, v, causal, upcast=False), attention_forward(q, k, v, causal, upcast=True))


@pytest.mark.parametrize("seed", range(200, 216))
def test_paged_attention_random(seed):
    rnd, g, D, dtype = _setup(seed)
    S, Hk, G = rnd.randint(1, 9), rnd.choice([1, 2, 4]), rnd.choice([1, 2, 3, 8, 16])
    block, longest, blocks = rnd.choice([8, 16, 32, 64, 128, 256]), rnd.randint(1, 5000), rnd.randint(50, 300)
    lens = torch.randint(1, longest + 1, (S,), device=device(), dtype=torch.int32, generator=g)
    lens[0] = longest
    q = _randn(g, dtype, S, Hk * G, D)
    kc, vc = _randn(g, dtype, blocks, Hk, block, D), _randn(g, dtype, blocks, Hk, block, D)
    tables = torch.randint(0, blocks, (S, -(-longest // block)), device=device(), generator=g)
    o = paged_attention(q, kc, vc, lens, tables, D ** -0.5, longest)
    check_device_status()
    assert_2x_rule("o", o, oracle_paged(q, kc, vc, tables, lens, D ** -0.5),
                   oracle_paged(q.float(), kc.float(), vc.float(), tables, lens, D ** -0.5))


@pytest.mark.parametrize("seed", range(300, 316))
def test_piecewise_attention_random(seed):
    rnd, g, D, dtype = _setup(seed)
    B, H, M, N = rnd.randint(1, 2), rnd.choice([1, 2, 3]), rnd.randint(1, 600), rnd.randint(1, 800)
    causal, w = rnd.random() < 0.5, rnd.randint(-50, max(M, N) + 50)
    leaves = tuple(_randn(g, dtype, B, H, T, D, grad=True) for T in (M, N, M, N, N))
    do = _randn(g, dtype, B, H, M, D)
    o = piecewise_attention(*leaves, w, causal)
    grads = torch.autograd.grad(o, leaves, do)
    o_ref = oracle_piecewise(*leaves, w, causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, leaves, do)
    o_low = oracle_piecewise(*leaves, w, causal)
    g_low = torch.autograd.grad(o_low, leaves, do)
    check_device_status()
    assert_2x_rule("o", o, o_low, o_ref)
    for name, a, b_, c in zip(("dq1", "dk1", "dq2", "dk2", "dv"), grads, g_low, g_ref):
        assert_2x_rule(name, a, b_, c)

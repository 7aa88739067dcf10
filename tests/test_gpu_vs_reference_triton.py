"""Same-GPU A/B against the reference's own Triton ``flash_attention``.

The unmodified reference is installed under ``baseline/_ref`` (git-ignored) with
``python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <writable copy of the reference checkout>``.
On identical seeded inputs, and with the default CUDA generator put in the same state before each call
(so both draw the same Philox ``(seed, offset)`` and hence the same dropout decisions), every result of
this library must lie within

    err(ours) <= 2 * err(reference Triton kernel) + 1e-5        (max-abs error against the fp32 oracle)

for O, the log-normaliser, total attention, dQ, dK and dV. This is the stated acceptance tolerance of
the project; the in-tree rule of the reference's tests (2 x the native-dtype PyTorch error,
``tests/flag_attn/test_flash_attention.py:116-124``) is enforced by the other test files.

The five benchmark configurations run at full size: the Triton kernel and ours see the whole problem,
the fp32 oracle is evaluated on (batch, KV-group) units and query-row bands of it (its score matrix
would not fit otherwise), and the errors of both kernels are taken on exactly those slices.
"""
import importlib
import math

import pytest
import torch

from flagattention_b200 import flash_attention
from gpu_util import attention_forward, clean, device, kernel_dropout_mask, make_qkv, max_abs_diff

pytestmark = pytest.mark.gpu


def _reference():
    try:
        return importlib.import_module("flag_attn")
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference install baseline/_ref not importable ({exc!r}); install it with pip --target baseline/_ref")


def _err(x, ref):
    return max_abs_diff(clean(x), clean(ref))


def _check(name, ours, theirs, exact):
    e_o, e_t = _err(ours, exact), _err(theirs, exact)
    assert e_o <= 2 * e_t + 1e-5, f"{name}: ours {e_o:.3e} > 2 x reference Triton {e_t:.3e}"
    return e_o, e_t


def _set_rng(seed):
    torch.cuda.manual_seed(seed)


def _run_both(fa, q, k, v, do, causal, p, aux, seed=1234):
    outs = []
    for fn in (flash_attention, fa.flash_attention):
        _set_rng(seed)
        res = fn(q, k, v, causal, dropout_p=p, return_log_normalizer=True, return_total_attention=aux,
                 return_seed_offset=True)
        o, lse, tot, s, off = res
        grads = torch.autograd.grad(o, (q, k, v), do) if do is not None else (None, None, None)
        outs.append((o, lse, tot, s, off, *grads))
    return outs


SHAPES = [
    # (B, Hq, Hk, M, N, D, causal, dtype, dropout, aux) -- the reference's shapes incl. its dropout and aux ones
    (2, 4, 4, 512, 612, 128, False, torch.float16, 0.0, True),
    (2, 4, 2, 512, 612, 128, True, torch.bfloat16, 0.0, False),
    (2, 4, 4, 1024, 1034, 64, False, torch.bfloat16, 0.0, True),
    (2, 4, 1, 1024, 1034, 64, True, torch.float16, 0.0, False),
    (2, 4, 4, 2048, 2048, 32, True, torch.float16, 0.0, False),
    (2, 4, 4, 2048, 2048, 32, False, torch.bfloat16, 0.5, False),
    (2, 4, 4, 4096, 4096, 16, False, torch.float16, 0.0, True),
    (2, 4, 4, 4001, 4001, 32, True, torch.bfloat16, 0.0, False),
    (2, 4, 4, 4001, 4096, 64, True, torch.float16, 0.8, False),
    (2, 4, 4, 4001, 4096, 64, False, torch.bfloat16, 0.0, True),
    (2, 4, 4, 4096, 4001, 128, False, torch.float16, 0.0, True),
    (2, 4, 4, 4096, 4000, 128, True, torch.bfloat16, 0.5, False),
    (2, 4, 2, 4096, 4001, 128, True, torch.float16, 0.0, False),
    (1, 2, 2, 8192, 8202, 16, False, torch.bfloat16, 0.0, True),
    (1, 2, 1, 8192, 8192, 32, True, torch.float16, 0.0, False),
    (2, 4, 4, 10006, 10, 128, True, torch.float16, 0.0, False),
]


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,p,aux", SHAPES,
                         ids=lambda x: str(x).replace("torch.", "") if not isinstance(x, bool) else ("T" if x else "F"))
@pytest.mark.parametrize("layout", ["BHTD", "BTHD"])
def test_all_outputs_within_twice_the_triton_error(B, Hq, Hk, M, N, D, causal, dtype, p, aux, layout):
    fa = _reference()
    if p > 0 and Hq != Hk:
        pytest.skip("the reference's dropout tests are MHA only")
    q, k, v, do = make_qkv(B, Hq, Hk, M, N, D, dtype, layout, 1.0, seed=2026, requires_grad=True)
    ours, theirs = _run_both(fa, q, k, v, do, causal, p, aux)
    mask = None
    if p > 0:
        assert ours[3:5] == theirs[3:5], "both calls must have drawn the same Philox (seed, offset)"
        mask = kernel_dropout_mask(B, Hq, M, N, p, ours[3], ours[4])
        ref_mask = fa.testing.recompute_mask(B, Hq, M, N, p, theirs[3], theirs[4], q.device)
        assert torch.equal(mask, ref_mask), "dropout decisions differ from the reference's compiled tl.rand"
    res = attention_forward(q, k, v, causal, dropout_p=p, dropout_mask=mask, upcast=True,
                            return_log_normalizer=True, return_total_attention=aux)
    o_ref, l_ref = res[0], res[1]
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    _check("o", ours[0], theirs[0], o_ref)
    fin = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(ours[1]), fin)
    _check("log_normalizer", ours[1][fin], theirs[1][fin], l_ref[fin])
    if aux:
        _check("total_attention", ours[2], theirs[2], res[2])
    for name, a, b_, c in zip(("dq", "dk", "dv"), ours[5:], theirs[5:], g_ref):
        _check(name, a, b_, c)


def test_ten_key_case_where_the_in_tree_rule_is_decided_by_one_rounding():
    """B2 Hq4 Hk2 M=10006 N=10 D128 bf16, causal, [B,T,H,D] layout, inputs of seed 10086: the one input
    of the reference's test grid on which `err <= 2 x err(native-dtype PyTorch)` does not hold for dQ --
    for the reference's Triton kernel (1.95e-2 against 2 x 7.8e-3) exactly as for this library. Against
    the Triton kernel's own error, the acceptance rule of this project, it passes."""
    fa = _reference()
    q, k, v, do = make_qkv(2, 4, 2, 10006, 10, 128, torch.bfloat16, "BTHD", 1.0, seed=10086, requires_grad=True)
    ours, theirs = _run_both(fa, q, k, v, do, True, 0.0, False)
    o_ref = attention_forward(q, k, v, True, upcast=True)
    g_ref = torch.autograd.grad(o_ref, (q, k, v), do)
    _check("o", ours[0], theirs[0], o_ref)
    for name, a, b_, c in zip(("dq", "dk", "dv"), ours[5:], theirs[5:], g_ref):
        _check(name, a, b_, c)


# ------------------------------------------------------------------ the five benchmark configurations
def _oracle_slices(q, k, v, do, causal, p, full_mask, units, bands, want_tot):
    """fp32 oracle on chosen (batch, kv head) units and, within them, query-row bands [r0, r1).
    Yields (b, hk, r0, r1, o, lse, tot-or-None, (dq, dk, dv)-or-None); gradients only for whole units."""
    G = q.shape[1] // k.shape[1]
    M, N = q.shape[2], k.shape[2]
    for b, hk in units:
        for r0, r1 in bands:
            qs = q[b:b + 1, hk * G:(hk + 1) * G, r0:r1].detach().requires_grad_(True)
            # bottom-right aligned causal mask: a row band [r0, r1) of the full problem sees keys up to
            # r1 - 1 + (N - M), which is itself a bottom-right aligned problem over keys [0, r1 + N - M)
            n_hi = min(N, r1 + N - M) if causal else N
            if n_hi <= 0:
                continue
            ks = k[b:b + 1, hk:hk + 1, :n_hi].detach().requires_grad_(True)
            vs = v[b:b + 1, hk:hk + 1, :n_hi].detach().requires_grad_(True)
            mask = full_mask[b:b + 1, hk * G:(hk + 1) * G, r0:r1, :n_hi] if full_mask is not None else None
            o, lse, tot = attention_forward(qs, ks, vs, causal, dropout_p=p, dropout_mask=mask, upcast=True,
                                            return_log_normalizer=True, return_total_attention=True)
            grads = None
            if do is not None and (r0, r1) == (0, M):
                grads = torch.autograd.grad(o, (qs, ks, vs), do[b:b + 1, hk * G:(hk + 1) * G])
            yield b, hk, r0, r1, n_hi, o.detach(), lse.detach(), (tot.detach() if want_tot else None), grads


CONFIGS = {
    # name: B, Hq, Hk, M, N, D, dtype, causal, p, bwd, aux, k/v distribution, units, row bands
    "c1": (1, 4, 4, 128, 128, 64, torch.float16, False, 0.0, False, False, [(0, 0), (0, 3)], None),
    "c2": (4, 32, 8, 4096, 4096, 128, torch.bfloat16, True, 0.0, True, False, [(0, 0), (3, 7)], None),
    "c3": (16, 16, 16, 2048, 2048, 64, torch.float16, False, 0.1, True, True, [(0, 0), (15, 9)], None),
    "c4": (8, 16, 1, 512, 8192, 128, torch.bfloat16, False, 0.0, False, False, [(0, 0), (7, 0)], None),
    "c5": (1, 64, 8, 32768, 32768, 128, torch.bfloat16, True, 0.0, False, False, [(0, 2)],
           [(0, 512), (16384, 16896), (32256, 32768)]),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_benchmark_configs_within_twice_the_triton_error(name):
    fa = _reference()
    B, Hq, Hk, M, N, D, dtype, causal, p, bwd, aux, units, bands = CONFIGS[name]
    dev = device()
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, Hq, M, D, device=dev, dtype=dtype, generator=g).requires_grad_(bwd)
    k = torch.randn(B, Hk, N, D, device=dev, dtype=dtype, generator=g).requires_grad_(bwd)
    if name == "c4":
        v = (torch.rand(B, Hk, N, D, device=dev, generator=g) * 2 - 1).to(dtype).requires_grad_(bwd)
    else:
        v = torch.randn(B, Hk, N, D, device=dev, dtype=dtype, generator=g).requires_grad_(bwd)
    do = torch.randn(B, Hq, M, D, device=dev, dtype=dtype, generator=g) if bwd else None
    ours, theirs = _run_both(fa, q, k, v, do, causal, p, aux)
    if p > 0:
        assert ours[3:5] == theirs[3:5]
    G = Hq // Hk
    bands = bands or [(0, M)]
    full_mask = kernel_dropout_mask(B, Hq, M, N, p, ours[3], ours[4]) if p > 0 else None
    worst = {}
    for b, hk, r0, r1, n_hi, o, lse, tot, grads in _oracle_slices(q, k, v, do, causal, p, full_mask, units, bands, aux):
        hs = slice(hk * G, (hk + 1) * G)
        worst["o"] = _check("o", ours[0][b:b + 1, hs, r0:r1], theirs[0][b:b + 1, hs, r0:r1], o)
        _check("log_normalizer", ours[1][b:b + 1, hs, r0:r1], theirs[1][b:b + 1, hs, r0:r1], lse)
        if tot is not None:
            _check("total_attention", ours[2][b:b + 1, hs], theirs[2][b:b + 1, hs], tot)
        if grads is not None:
            _check("dq", ours[5][b:b + 1, hs], theirs[5][b:b + 1, hs], grads[0])
            _check("dk", ours[6][b:b + 1, hk:hk + 1], theirs[6][b:b + 1, hk:hk + 1], grads[1])
            _check("dv", ours[7][b:b + 1, hk:hk + 1], theirs[7][b:b + 1, hk:hk + 1], grads[2])
    assert worst, "no slice was checked"

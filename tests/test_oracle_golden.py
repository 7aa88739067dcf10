"""The CPU oracle against fixtures produced by the reference's own code (tests/golden)."""
import json

import numpy as np
import pytest
import torch

from conftest import ATTENTION_GOLDENS, GOLDEN, TRITON_GOLDENS, load_golden
from oracle.attention import attention_backward, attention_forward, autograd_backward, max_abs_diff
from oracle.philox import dropout_keep_mask


def _finite_close(a, b, atol, rtol=0.0):
    a, b = a.float(), b.float()
    inf = torch.isinf(b)
    assert torch.equal(torch.isinf(a), inf)
    assert torch.equal(a[inf], b[inf])
    torch.testing.assert_close(a[~inf], b[~inf], atol=atol, rtol=rtol)


@pytest.mark.parametrize("name", ATTENTION_GOLDENS)
def test_forward_matches_reference_pytorch(name):
    g = load_golden(name)
    m = g["meta"]
    for tag, up in (("ref32", True), ("lowp", False)):
        o, lse, tot = attention_forward(g["q"], g["k"], g["v"], m["causal"], dropout_p=m["dropout_p"],
                                        dropout_mask=g["mask"], upcast=up, return_log_normalizer=True,
                                        return_total_attention=True)
        # Same formulae, same library; tolerances only absorb a different CPU's matmul blocking.
        assert max_abs_diff(torch.nan_to_num(o), torch.nan_to_num(g[f"o_{tag}"])) <= (4e-3 if up else 4e-2)
        if up:
            _finite_close(lse, g["lse_ref32"], atol=1e-4)
            torch.testing.assert_close(tot, g["tot_ref32"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("name", ATTENTION_GOLDENS)
def test_backward_matches_reference_autograd(name):
    g = load_golden(name)
    m = g["meta"]
    grads = attention_backward(g["q"], g["k"], g["v"], g["do"], m["causal"], dropout_p=m["dropout_p"],
                               dropout_mask=g["mask"])
    auto = autograd_backward(g["q"], g["k"], g["v"], g["do"], m["causal"], dropout_p=m["dropout_p"],
                             dropout_mask=g["mask"])
    tol = 2e-2 if m["dtype"] == "bfloat16" else 4e-3
    scale = 1.0 / (1.0 - m["dropout_p"])
    for mine, ag, key in zip(grads, auto, ("dq_ref32", "dk_ref32", "dv_ref32")):
        ref = torch.nan_to_num(g[key].float())
        bound = tol * scale * max(1.0, ref.abs().max().item())
        assert max_abs_diff(mine, ref) <= bound, key
        assert max_abs_diff(torch.nan_to_num(ag.float()), ref) <= bound, key


@pytest.mark.parametrize("name", TRITON_GOLDENS)
def test_oracle_matches_reference_triton_kernels(name):
    """The reference's Triton kernels (run by the Triton interpreter when the fixture was made)
    agree with the oracle to fp16 rounding, including -inf log-normalisers and dropout."""
    g = load_golden(name)
    m = g["meta"]
    mask = None
    if m["dropout_p"] > 0:
        mask = torch.from_numpy(dropout_keep_mask(m["B"], m["Hq"], m["M"], m["N"], m["dropout_p"],
                                                  m["rng_seed"], m["rng_offset"]))
    o, lse, tot = attention_forward(g["q"], g["k"], g["v"], m["causal"], dropout_p=m["dropout_p"],
                                    dropout_mask=mask, upcast=True, return_log_normalizer=True,
                                    return_total_attention=True)
    assert max_abs_diff(o, g["o"]) <= 4e-3
    _finite_close(lse, g["lse"], atol=1e-4)
    torch.testing.assert_close(tot, g["tot"], atol=2e-3, rtol=2e-3)
    dq, dk, dv = attention_backward(g["q"], g["k"], g["v"], g["do"], m["causal"],
                                    dropout_p=m["dropout_p"], dropout_mask=mask)
    assert max_abs_diff(dq, g["dq"]) <= 1e-2
    assert max_abs_diff(dk, g["dk"]) <= 2e-2
    assert max_abs_diff(dv, g["dv"]) <= 2e-2
    delta = (o.float() * g["do"].float()).sum(-1)
    assert max_abs_diff(delta, g["delta"]) <= 2e-2


def test_philox_mask_bit_exact_with_reference_kernel():
    z = np.load(GOLDEN / "dropout_masks.npz")
    B, H, M, N = (int(x) for x in z["shape"])
    for i, (seed, offset, p) in enumerate(json.loads(str(z["cases"]))):
        want = np.unpackbits(z[f"mask{i}"])[: B * H * M * N].reshape(B, H, M, N).astype(bool)
        got = dropout_keep_mask(B, H, M, N, p, seed, offset)
        assert np.array_equal(got, want), (seed, offset, p)


def test_philox_mask_statistics():
    # Same check as the reference's tests/flag_attn/test_dropout.py:24-48 (drop rate within 1 %).
    for p in (0.5, 0.8):
        mask = dropout_keep_mask(1, 2, 512, 612, p, 123456789, 123456789123456789)
        rate = 1.0 - mask.mean()
        assert abs(rate - p) / p < 0.01


from conftest import PAGED_GOLDENS, load_paged_golden  # noqa: E402


@pytest.mark.parametrize("name", PAGED_GOLDENS)
def test_paged_oracle_matches_reference_fixture(name):
    """oracle/paged.py against outputs of the reference's testing/paged.py (native dtype and fp32)."""
    from oracle.paged import paged_attention
    g = load_paged_golden(name)
    got = paged_attention(g["q"], g["key_cache"], g["value_cache"], g["block_tables"], g["context_lens"], g["scale"])
    assert got.dtype == g["out"].dtype
    torch.testing.assert_close(got.float(), g["out"].float(), atol=2e-3, rtol=1e-2)
    got32 = paged_attention(g["q"].float(), g["key_cache"].float(), g["value_cache"].float(), g["block_tables"],
                            g["context_lens"], g["scale"])
    torch.testing.assert_close(got32, g["out_fp32"], atol=1e-5, rtol=1e-5)


from conftest import PIECEWISE_GOLDENS  # noqa: E402


@pytest.mark.parametrize("name", PIECEWISE_GOLDENS)
def test_piecewise_oracle_matches_reference_fixture(name):
    """oracle/piecewise.py against outputs and autograd gradients of the reference's
    testing/piecewise.py: same formula on the same CPU, so bit for bit."""
    from oracle.piecewise import piecewise_attention
    g = load_golden(name)
    meta = g["meta"]
    for mode, upcast in (("upcast", True), ("native", False)):
        leaves = [g[k].clone().requires_grad_(True) for k in ("q1", "k1", "q2", "k2", "v")]
        o = piecewise_attention(*leaves, meta["w"], meta["causal"], upcast=upcast)
        assert torch.equal(o, g[f"o_{mode}"])
        grads = torch.autograd.grad(o, leaves, g["do"])
        for nm, got in zip(("dq1", "dk1", "dq2", "dk2", "dv"), grads):
            assert torch.equal(got, g[f"{nm}_{mode}"]), (name, mode, nm)

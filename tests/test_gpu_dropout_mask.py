"""Dropout keep-masks: bit-exact against the numpy oracle, the reference fixtures and, when
Triton is importable, the compiled `tl.rand(seed, offs, n_rounds=6)` the reference uses."""
import json

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from gpu_util import kernel_dropout_mask
from oracle.philox import dropout_keep_mask

pytestmark = pytest.mark.gpu

CASES = [(123456789, 0, 0.3), (123456789, 123456789123456789, 0.5), ((1 << 40) + 7, 12, 0.8),
         (5, (1 << 31) - 100, 0.1), (77, (1 << 32) - 1000, 0.5), (2 ** 63 + 5, 4, 0.5)]


@pytest.mark.parametrize("seed,offset,p", CASES)
def test_mask_matches_oracle(seed, offset, p):
    B, H, M, N = 2, 3, 37, 1001
    got = kernel_dropout_mask(B, H, M, N, p, seed, offset).cpu().numpy()
    want = dropout_keep_mask(B, H, M, N, p, seed, offset)
    assert np.array_equal(got, want)


def test_mask_matches_reference_fixture():
    z = np.load(GOLDEN / "dropout_masks.npz")
    B, H, M, N = (int(x) for x in z["shape"])
    for i, (seed, offset, p) in enumerate(json.loads(str(z["cases"]))):
        want = np.unpackbits(z[f"mask{i}"])[: B * H * M * N].reshape(B, H, M, N).astype(bool)
        got = kernel_dropout_mask(B, H, M, N, p, seed, offset).cpu().numpy()
        assert np.array_equal(got, want), (seed, offset, p)


@pytest.mark.parametrize("seed,offset,p", CASES[:5])
def test_mask_matches_compiled_triton(seed, offset, p):
    triton = pytest.importorskip("triton")
    import triton.language as tl

    @triton.jit
    def _mask(mask, total, dropout_p, seed, offset, BLOCK: tl.constexpr):
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        keep = tl.rand(seed, offset + offs, n_rounds=6) > dropout_p
        tl.store(mask + offs, keep, mask=offs < total)

    B, H, M, N = 1, 2, 37, 1500
    total = B * H * M * N
    ref = torch.zeros(total, dtype=torch.bool, device="cuda")
    _mask[(triton.cdiv(total, 1024),)](ref, total, p, seed, offset, BLOCK=1024)
    got = kernel_dropout_mask(B, H, M, N, p, seed, offset).reshape(-1)
    assert torch.equal(got, ref)


@pytest.mark.parametrize("p", [0.5, 0.8])
@pytest.mark.parametrize("B,H,M,N", [(2, 4, 512, 612), (2, 4, 1024, 1034), (2, 4, 2048, 2048), (2, 4, 4096, 4096),
                                     (2, 4, 4001, 4001), (2, 4, 4001, 4096), (2, 4, 4096, 4001),
                                     (1, 2, 8192, 8202), (1, 2, 8192, 8192)])
def test_drop_rate(B, H, M, N, p):
    # tests/flag_attn/test_dropout.py:24-48 of the reference: empirical drop rate within 1 %.
    mask = kernel_dropout_mask(B, H, M, N, p, 123456789, 123456789123456789)
    rate = 1.0 - mask.float().mean().item()
    assert abs(rate - p) / p < 0.01

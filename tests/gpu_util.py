"""Helpers shared by the GPU parity tests."""
import math

import torch

from flagattention_b200 import _lib
from oracle.attention import attention_backward, attention_forward, max_abs_diff  # noqa: F401


def device():
    return torch.device("cuda", 0)


def make_qkv(B, Hq, Hk, M, N, D, dtype, layout="BHTD", std=1.0, seed=0, requires_grad=False):
    """Seeded inputs in the two layouts the reference's tests use: contiguous [B,H,T,D] or a
    transposed view of [B,T,H,D] (tests/flag_attn/test_flash_attention.py:107-114)."""
    g = torch.Generator(device=device()).manual_seed(seed)

    def mk(H, T):
        if layout == "BHTD":
            t = torch.empty(B, H, T, D, dtype=dtype, device=device()).normal_(0.0, std, generator=g)
        else:
            t = torch.empty(B, T, H, D, dtype=dtype, device=device()).normal_(0.0, std, generator=g).transpose(1, 2)
        return t.requires_grad_(requires_grad)

    q, k, v = mk(Hq, M), mk(Hk, N), mk(Hk, N)
    if layout == "BHTD":
        do = torch.randn(B, Hq, M, D, dtype=dtype, device=device(), generator=g)
    else:
        do = torch.randn(B, M, Hq, D, dtype=dtype, device=device(), generator=g).transpose(1, 2)
    return q, k, v, do


def kernel_dropout_mask(B, H, M, N, p, seed, offset):
    """Keep-mask for (seed, offset) materialised by the library's mask kernel (bool [B,H,M,N])."""
    lib = _lib.load()
    m = torch.empty(B, H, M, N, dtype=torch.uint8, device=device())
    _lib.check(lib.b200attn_dropout_mask(m.data_ptr(), B, H, M, N, float(p), seed & (2 ** 64 - 1),
                                         offset & (2 ** 64 - 1), torch.cuda.current_stream().cuda_stream),
               "b200attn_dropout_mask")
    return m.bool()


def clean(x):
    return torch.nan_to_num(x.float(), nan=0.0, posinf=0.0, neginf=0.0)


def assert_2x_rule(name, hyp, lowp, exact, slack=1e-5):
    """err(hyp) <= 2 * err(same math in the input dtype) + slack, the reference's acceptance rule
    (tests/flag_attn/test_flash_attention.py:116-124)."""
    e_h = max_abs_diff(clean(hyp), clean(exact))
    e_l = max_abs_diff(clean(lowp), clean(exact))
    assert e_h <= 2 * e_l + slack, f"{name}: kernel err {e_h:.3e} > 2 x {e_l:.3e}"
    return e_h, e_l

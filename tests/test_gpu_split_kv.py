"""GPU parity of flash_attention_split_kv (the reference's flash-decoding operator,
split_kv.py:282-347) and of the kernels behind it: the register-resident streaming kernel for up to
two query rows per KV head, the head-packed tensor-core tile for grouped heads, and the plain
tile pair. Cases follow tests/flag_attn/test_flash_attention.py:38-76,127-172."""
import pytest
import torch

from flagattention_b200 import _lib, check_device_status, flash_attention, flash_attention_split_kv
from gpu_util import assert_2x_rule, attention_forward, device, make_qkv, max_abs_diff

pytestmark = pytest.mark.gpu

OPERATORS = {"flash_attention": flash_attention, "flash_attention_split_kv": flash_attention_split_kv}


@pytest.mark.parametrize("seed", [17, 35, 36, 68, 77])
@pytest.mark.parametrize("operator", list(OPERATORS))
def test_splitkv_large_logits(seed, operator):
    g = torch.Generator(device=device()).manual_seed(seed)
    q = torch.randn((1, 2, 4, 16), generator=g, device=device(), dtype=torch.float16) * 10
    k = torch.randn((1, 1, 8202, 16), generator=g, device=device(), dtype=torch.float16) * 10
    v = torch.randn(k.shape, generator=g, device=device(), dtype=torch.float16) * 10
    expected = attention_forward(q, k, v, False, upcast=True)
    baseline = attention_forward(q, k, v, False, upcast=False)
    actual = OPERATORS[operator](q, k, v)
    assert actual.dtype == q.dtype
    assert max_abs_diff(actual, expected) <= 2 * max_abs_diff(baseline, expected) + 1e-5
    check_device_status()


def test_splitkv_single_split_preserves_dtype():
    g = torch.Generator(device=device()).manual_seed(2026)
    q, k, v = [torch.randn((1, 1, 16, 16), generator=g, device=device(), dtype=torch.bfloat16)
               for _ in range(3)]
    actual = flash_attention_split_kv(q, k, v)
    expected = attention_forward(q, k, v, False, upcast=True)
    assert actual.dtype == q.dtype
    torch.testing.assert_close(actual.float(), expected.float(), atol=2e-2, rtol=2e-2)
    check_device_status()


@pytest.mark.parametrize("operator", list(OPERATORS))
def test_splitkv_independent_kv_strides(operator):
    g = torch.Generator(device=device()).manual_seed(2026)
    q = torch.randn((2, 4, 1, 32), generator=g, device=device(), dtype=torch.float16)
    k = torch.randn((2, 2, 257, 32), generator=g, device=device(), dtype=torch.float16)
    v = torch.randn((2, 257, 2, 32), generator=g, device=device(), dtype=torch.float16).transpose(1, 2)
    assert k.stride() != v.stride()
    actual = OPERATORS[operator](q, k, v)
    expected = attention_forward(q, k, v, False, upcast=True)
    baseline = attention_forward(q, k, v, False, upcast=False)
    assert max_abs_diff(actual, expected) <= 2 * max_abs_diff(baseline, expected) + 1e-5
    check_device_status()


# (B, Hq, Hk, M, N, D): rows per KV head = Hq/Hk * M selects the kernel.
DECODE_SHAPES = [
    # 1..4 rows per KV head: streaming kernel up to 2 rows, head-packed tile above (grouped heads)
    (2, 4, 4, 1, 1, 128), (2, 4, 4, 1, 127, 64), (2, 16, 16, 1, 4099, 128), (3, 8, 8, 1, 33000, 64),
    (2, 4, 4, 1, 8202, 32), (1, 2, 2, 1, 8202, 16), (2, 8, 4, 1, 5000, 128), (2, 4, 4, 2, 4000, 64),
    (1, 6, 2, 1, 2049, 32), (2, 8, 2, 1, 9000, 128), (1, 4, 2, 2, 3001, 16), (1, 2, 2, 4, 8202, 64),
    # head-packed tensor-core tile: 8..128 rows per KV head
    (2, 16, 2, 1, 5000, 128), (1, 32, 4, 1, 8202, 64), (2, 8, 1, 3, 4001, 32), (1, 16, 2, 8, 3000, 16),
    (1, 8, 1, 16, 6000, 128), (2, 6, 2, 5, 2500, 64),
    # plain tile pair: more than 128 rows per KV head, or ungrouped with M > 4
    (1, 16, 1, 9, 5000, 128), (1, 2, 2, 8, 8202, 64), (1, 4, 4, 33, 4000, 32),
]


def _decode_params():
    out, i = [], 0
    for shape in DECODE_SHAPES:
        for causal in (False, True):
            dtype = (torch.float16, torch.bfloat16)[i % 2]
            layout = ("BHTD", "BTHD")[(i // 2) % 2]
            i += 1
            out.append(pytest.param(*shape, causal, dtype, layout,
                                    id=f"{'x'.join(map(str, shape))}-{'c' if causal else 'n'}-"
                                       f"{str(dtype)[6:]}-{layout}"))
    return out


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,layout", _decode_params())
def test_split_kv_operator(B, Hq, Hk, M, N, D, causal, dtype, layout):
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, layout, 3.0, seed=4242)
    o_ref = attention_forward(q, k, v, causal, upcast=True)
    o_low = attention_forward(q, k, v, causal, upcast=False)
    o = flash_attention_split_kv(q, k, v, causal)
    assert o.dtype == q.dtype and o.shape == q.shape
    assert_2x_rule("o", o, o_low, o_ref)
    check_device_status()


@pytest.mark.parametrize("Hq,Hk,M", [(4, 4, 1), (8, 4, 2), (16, 2, 3), (4, 4, 9)])
@pytest.mark.parametrize("num_splits", [1, 2, 7, 40])
def test_split_count_does_not_change_result(Hq, Hk, M, num_splits):
    """Through the C ABI with an explicit split count (more splits than 128-key tiles included):
    output and log-normaliser agree with the oracle for every count."""
    B, N, D, dtype = 2, 3000, 64, torch.float16
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "BHTD", 2.0, seed=7)
    lib = _lib.load()
    o = torch.empty_like(q)
    lse = torch.empty((B, Hq, M), dtype=torch.float32, device=device())
    part_o = torch.empty((B, Hq, num_splits, M, D), dtype=torch.float32, device=device())
    part_l = torch.empty((B, Hq, num_splits, M), dtype=torch.float32, device=device())
    status = torch.zeros(1, dtype=torch.int32, device=device())
    sp = _lib.SplitKVParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o),
                            lse.data_ptr(), part_o.data_ptr(), part_l.data_ptr(), B, Hq, Hk, M, N, D,
                            num_splits, _lib.dtype_code(dtype), 1, 0.125, status.data_ptr())
    _lib.check(lib.b200attn_fwd_splitkv(sp, torch.cuda.current_stream().cuda_stream), "fwd_splitkv")
    o_ref, lse_ref = attention_forward(q, k, v, True, 0.125, upcast=True, return_log_normalizer=True)[:2]
    o_low = attention_forward(q, k, v, True, 0.125, upcast=False)
    assert int(status.item()) == 0
    assert_2x_rule("o", o, o_low, o_ref)
    torch.testing.assert_close(lse, lse_ref.float(), atol=2e-3, rtol=1e-4)


def test_suggested_split_count_is_admissible():
    lib = _lib.load()
    for (B, Hq, Hk, M, N, D) in DECODE_SHAPES + [(2, 32, 32, 1, 2 ** 19, 64), (1, 1, 1, 1, 100, 16)]:
        s = lib.b200attn_splitkv_num_splits(B, Hq, Hk, M, N, D, 0)
        tiles = -(-N // 128)
        rows = Hq // Hk * M
        if 2 < rows <= 128 and Hq > Hk and s % 2 == 0:
            s //= 2  # head-packed tiles: two partials per CTA
        assert 1 <= s <= max(1, tiles)
        per = -(-tiles // s)
        assert per * (s - 1) < tiles  # no CTA without keys

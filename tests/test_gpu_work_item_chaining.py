"""Forward launches with more work items (256 query rows of one head) than the GPU has SMs: every CTA
then walks several items, carrying its barrier phases, K/V ring position and output staging buffers
from one to the next. Shapes are ragged on purpose (partial and empty second query tiles, M != N,
grouped heads, bands, dropout, transposed layouts) and every head dimension is covered; results are
checked against the oracle with the reference's acceptance rule
(tests/flag_attn/test_flash_attention.py:116-124), and against a launch of one CTA per item where
the two must agree bit for bit."""
import pytest
import torch

from flagattention_b200 import _lib, check_device_status, flash_attention
from gpu_util import assert_2x_rule, attention_forward, device, kernel_dropout_mask, make_qkv

pytestmark = pytest.mark.gpu

# (B, Hq, Hk, M, N, D): B * Hq * ceil(M / 256) is 2 to 6 times the SM count
SHAPES = [
    (8, 16, 16, 700, 700, 128),    # last item of a head: partial first tile, empty second tile
    (4, 32, 8, 1000, 1000, 64),    # grouped heads, partial second tile
    (6, 24, 4, 520, 333, 32),      # M > N
    (16, 12, 12, 300, 1500, 16),   # M < N: every query sees the N - M prefix
    (3, 40, 10, 1025, 257, 128),   # one row in the last item
    (5, 36, 36, 384, 4000, 64),    # exactly one full tile in the last item
]


def _params():
    out, i = [], 0
    for shape in SHAPES:
        for causal in (False, True):
            dtype = (torch.bfloat16, torch.float16)[i % 2]
            layout = ("BHTD", "BTHD")[(i // 2) % 2]
            i += 1
            out.append(pytest.param(*shape, causal, dtype, layout,
                                    id=f"{'x'.join(map(str, shape))}-{'c' if causal else 'n'}-{str(dtype)[6:]}-{layout}"))
    return out


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,dtype,layout", _params())
def test_forward_many_items(B, Hq, Hk, M, N, D, causal, dtype, layout):
    sms = torch.cuda.get_device_properties(device()).multi_processor_count
    assert B * Hq * -(-M // 256) > sms
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, layout, 1.0, seed=99)
    o, lse = flash_attention(q, k, v, causal, return_log_normalizer=True)[:2]
    check_device_status()
    o_ref, lse_ref = attention_forward(q, k, v, causal, upcast=True, return_log_normalizer=True)[:2]
    o_low = attention_forward(q, k, v, causal, upcast=False)
    assert_2x_rule("o", o, o_low, o_ref)
    finite = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), finite)
    torch.testing.assert_close(lse[finite], lse_ref.float()[finite], atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("D", [64, 128])
def test_forward_many_items_dropout(D):
    B, Hq, Hk, M, N = 4, 48, 12, 600, 777
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, torch.float16, "BHTD", 1.0, seed=5)
    torch.manual_seed(1234)
    o, _, _, seed, offset = flash_attention(q, k, v, True, dropout_p=0.3, return_seed_offset=True)
    check_device_status()
    mask = kernel_dropout_mask(B, Hq, M, N, 0.3, int(seed), int(offset))
    o_ref = attention_forward(q, k, v, True, dropout_p=0.3, dropout_mask=mask, upcast=True)
    o_low = attention_forward(q, k, v, True, dropout_p=0.3, dropout_mask=mask, upcast=False)
    assert_2x_rule("o", o, o_low, o_ref)


@pytest.mark.parametrize("dist_min,dist_max", [(0, 200), (-50, 300), (100, 1 << 30)])
@pytest.mark.parametrize("D", [64, 128])
def test_forward_many_items_band(dist_min, dist_max, D):
    """A visibility band through the C entry point: items whose first K/V tile is not tile 0 (D = 128 takes
    the 64-key softmax pipeline, D = 64 the 128-key one)."""
    B, Hq, Hk, M, N, dtype = 4, 40, 8, 900, 1100, torch.bfloat16
    q, k, v, _ = make_qkv(B, Hq, Hk, M, N, D, dtype, "BHTD", 1.0, seed=8)
    lib = _lib.load()
    o = torch.empty_like(q)
    lse = torch.empty((B, Hq, M), dtype=torch.float32, device=device())
    status = torch.zeros(1, dtype=torch.int32, device=device())
    fp = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(),
                        B, Hq, Hk, M, N, D, _lib.dtype_code(dtype), _lib.dtype_code(dtype), 0, D ** -0.5, 0.0, 0, 0,
                        status.data_ptr(), 1, dist_min, dist_max, None)
    _lib.check(lib.b200attn_fwd(fp, torch.cuda.current_stream().cuda_stream), "fwd")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    dist = (torch.arange(M, device=device()).unsqueeze(-1) + (N - M)) - torch.arange(N, device=device())
    visible = (dist >= dist_min) & (dist < dist_max)
    groups = Hq // Hk

    def formula(upcast):
        qq, kk, vv = (q.float(), k.float(), v.float()) if upcast else (q, k, v)
        s = (qq @ kk.repeat_interleave(groups, 1).transpose(2, 3)) * D ** -0.5
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s.float(), -1)
        p = torch.nan_to_num(p, nan=0.0)  # rows that see no key
        return p.to(vv.dtype) @ vv.repeat_interleave(groups, 1)

    assert_2x_rule("o", o, formula(False), formula(True))


@pytest.mark.parametrize("B,Hq,Hk,M,N,D,causal,p", [
    (8, 16, 16, 700, 700, 128, True, 0.0), (4, 32, 8, 1000, 1000, 64, False, 0.0),
    (4, 48, 12, 600, 777, 64, True, 0.2), (16, 12, 12, 300, 1500, 16, True, 0.0),
    (6, 32, 8, 900, 1300, 128, False, 0.0)])
def test_chained_items_match_one_cta_per_item(B, Hq, Hk, M, N, D, causal, p):
    """A launch over the whole batch has more work items than SMs, so every CTA walks several of them; a
    launch over one batch element has fewer and runs one CTA per item. Both must give identical bits: the
    per-item arithmetic does not depend on which CTA runs the item or on what that CTA ran before."""
    sms = torch.cuda.get_device_properties(device()).multi_processor_count
    per_batch = Hq * -(-M // 256)
    assert B * per_batch > sms >= per_batch
    g = torch.Generator(device=device()).manual_seed(3)
    q = torch.randn(B, Hq, M, D, device=device(), dtype=torch.bfloat16, generator=g)
    k = torch.randn(B, Hk, N, D, device=device(), dtype=torch.bfloat16, generator=g)
    v = torch.randn(B, Hk, N, D, device=device(), dtype=torch.bfloat16, generator=g)
    torch.cuda.manual_seed(77)
    o, lse, _, seed, offset = flash_attention(q, k, v, causal, dropout_p=p, return_log_normalizer=True,
                                              return_seed_offset=True)
    for b in (0, B - 1):
        if p > 0:
            # element (b, h, m, n) of the whole problem draws counter offset + ((b*Hq + h)*M + m)*N + n:
            # put the generator where the slice's own numbering reproduces those counters
            st = torch.cuda.default_generators[device().index].get_state()
            st.view(torch.int64)[0] = seed
            st.view(torch.int64)[1] = offset + b * Hq * M * N
            torch.cuda.default_generators[device().index].set_state(st)
        o1, lse1 = flash_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], causal, dropout_p=p,
                                   return_log_normalizer=True)[:2]
        assert torch.equal(o1, o[b:b + 1]) and torch.equal(lse1, lse[b:b + 1])
    check_device_status()

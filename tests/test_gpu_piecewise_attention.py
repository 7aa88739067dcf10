"""GPU parity of piecewise_attention against the oracle, on the shapes and the acceptance rule of the
reference's tests (tests/flag_attn/test_piecewise_attention.py:27-160), plus the visibility band of the
C ABI that it is built on."""
import itertools
import math

import pytest
import torch

from conftest import PIECEWISE_GOLDENS, load_golden
from flagattention_b200 import _lib, check_device_status
from flagattention_b200.piecewise import piecewise_attention
from gpu_util import assert_2x_rule, device, max_abs_diff
from oracle.piecewise import piecewise_attention as oracle_piecewise

pytestmark = pytest.mark.gpu

SHAPES = [(2, 4, 512, 612, 128), (2, 4, 1024, 1034, 64), (2, 4, 2048, 2048, 32), (2, 4, 4096, 4096, 16),
          (2, 4, 4096, 4001, 16), (1, 2, 8192, 8192, 16), (1, 2, 8192, 8192, 32), (1, 2, 8192, 3867, 32)]
_cycle = itertools.cycle(itertools.product(["BHTD", "BTHD"], [1.0, 2.0, 3.0, 4.0]))


def _params():
    out = []
    for shape in SHAPES:
        for causal in (True, False):
            for dtype in (torch.float16, torch.bfloat16):
                layout, scale = next(_cycle)
                out.append(pytest.param(*shape, causal, dtype, layout, scale,
                                        id=f"{'x'.join(map(str, shape))}-{'c' if causal else 'n'}-"
                                           f"{str(dtype)[6:]}-{layout}-s{scale:g}"))
    return out


def _inputs(B, H, M, N, D, dtype, layout, scale, requires_grad):
    g = torch.Generator(device=device()).manual_seed(10086)

    def mk(T):
        if layout == "BHTD":
            t = torch.empty(B, H, T, D, dtype=dtype, device=device()).normal_(0.0, scale, generator=g)
        else:
            t = torch.empty(B, T, H, D, dtype=dtype, device=device()).normal_(0.0, scale, generator=g).transpose(1, 2)
        return t.requires_grad_(requires_grad)

    q1, q2 = mk(M), mk(M)
    k1, k2, v = mk(N), mk(N), mk(N)
    do = mk(M).detach()
    return q1, k1, q2, k2, v, do


@pytest.mark.parametrize("B,H,M,N,D,causal,dtype,layout,scale", _params())
def test_attention_fwd(B, H, M, N, D, causal, dtype, layout, scale):
    q1, k1, q2, k2, v, _ = _inputs(B, H, M, N, D, dtype, layout, scale, False)
    w = (M // 2) if M < N else (M - N // 2)
    o_ref = oracle_piecewise(q1, k1, q2, k2, v, w, causal=causal, upcast=True)
    o_low = oracle_piecewise(q1, k1, q2, k2, v, w, causal=causal)
    o = piecewise_attention(q1, k1, q2, k2, v, w, causal=causal)
    check_device_status()
    assert o.dtype == q1.dtype and o.shape == q1.shape
    assert_2x_rule("o", o, o_low, o_ref)


@pytest.mark.parametrize("B,H,M,N,D,causal,dtype,layout,scale", _params())
def test_attention_bwd(B, H, M, N, D, causal, dtype, layout, scale):
    q1, k1, q2, k2, v, do = _inputs(B, H, M, N, D, dtype, layout, scale, True)
    leaves = (q1, k1, q2, k2, v)
    w = (M // 2) if M < N else (M - N // 2)
    o_ref = oracle_piecewise(*leaves, w, causal=causal, upcast=True)
    g_ref = torch.autograd.grad(o_ref, leaves, do)
    o_low = oracle_piecewise(*leaves, w, causal=causal)
    g_low = torch.autograd.grad(o_low, leaves, do)
    o = piecewise_attention(*leaves, w, causal=causal)
    g = torch.autograd.grad(o, leaves, do)
    check_device_status()
    assert_2x_rule("o", o, o_low, o_ref)
    for name, a, b_, c in zip(("dq1", "dk1", "dq2", "dk2", "dv"), g, g_low, g_ref):
        assert a.shape == c.shape and a.dtype == c.dtype
        assert_2x_rule(name, a, b_, c)


@pytest.mark.parametrize("name", PIECEWISE_GOLDENS)
def test_against_reference_fixture(name):
    g = load_golden(name)
    meta = g["meta"]
    leaves = [g[k].to(device()).requires_grad_(True) for k in ("q1", "k1", "q2", "k2", "v")]
    o = piecewise_attention(*leaves, meta["w"], causal=meta["causal"])
    grads = torch.autograd.grad(o, leaves, g["do"].to(device()))
    check_device_status()
    assert_2x_rule("o", o.cpu(), g["o_native"], g["o_upcast"])
    for nm, got in zip(("dq1", "dk1", "dq2", "dk2", "dv"), grads):
        assert_2x_rule(nm, got.cpu(), g[f"{nm}_native"], g[f"{nm}_upcast"])


@pytest.mark.parametrize("w", [-5, 0, 1, 100, 10 ** 6])
def test_degenerate_thresholds(w):
    """Thresholds that empty one of the regions: everything from the second pair (w <= 0 under the
    causal mask) or from the first (w beyond every distance)."""
    q1, k1, q2, k2, v, _ = _inputs(1, 2, 200, 333, 64, torch.float16, "BHTD", 1.0, False)
    for causal in (True, False):
        o = piecewise_attention(q1, k1, q2, k2, v, w, causal=causal)
        check_device_status()
        assert_2x_rule("o", o, oracle_piecewise(q1, k1, q2, k2, v, w, causal=causal),
                       oracle_piecewise(q1, k1, q2, k2, v, w, causal=causal, upcast=True))


@pytest.mark.parametrize("dmin,dmax", [(0, 100), (-64, 64), (37, 300), (None, 129), (200, None), (500, 600)])
@pytest.mark.parametrize("D", [64, 128])
def test_band_mask_through_the_c_abi(dmin, dmax, D):
    """b200attn_fwd / b200attn_bwd with a visibility band (a sliding window) against masked dense math."""
    B, H, M, N = 1, 2, 400, 520
    dtype = torch.bfloat16
    g = torch.Generator(device=device()).manual_seed(5)
    q, do = (torch.randn(B, H, M, D, device=device(), dtype=dtype, generator=g) for _ in range(2))
    k, v = (torch.randn(B, H, N, D, device=device(), dtype=dtype, generator=g) for _ in range(2))
    lo = _lib.BAND_OPEN_MIN if dmin is None else dmin
    hi = _lib.BAND_OPEN_MAX if dmax is None else dmax
    dist = (torch.arange(M, device=device()).unsqueeze(-1) + (N - M)) - torch.arange(N, device=device())
    vis = (dist >= lo) & (dist < hi)

    def dense(upcast):
        leaves = [t.detach().clone().float().requires_grad_(True) if upcast else t.detach().clone().requires_grad_(True)
                  for t in (q, k, v)]
        s = (leaves[0] @ leaves[1].transpose(2, 3)) / math.sqrt(D)
        s = torch.where(vis, s, float("-inf")).float()
        p = torch.nan_to_num(torch.softmax(s, -1), nan=0.0)
        o = (p.to(leaves[2].dtype) @ leaves[2])
        grads = torch.autograd.grad(o, leaves, do.to(o.dtype))
        return o, torch.logsumexp(s, -1), grads

    o_ref, lse_ref, g_ref = dense(True)
    o_low, _, g_low = dense(False)
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=device())
    o = torch.empty_like(q)
    lse = torch.empty(B, H, M, dtype=torch.float32, device=device())
    dt = _lib.dtype_code(dtype)
    fp = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(), B, H, H, M, N,
                        D, dt, dt, 0, 1 / math.sqrt(D), 0.0, 0, 0, status.data_ptr(), 1, lo, hi)
    _lib.check(lib.b200attn_fwd(fp, st), "fwd")
    assert_2x_rule("o", o, o_low, o_ref)
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), fin)
    assert max_abs_diff(lse[fin], lse_ref[fin]) <= 1e-3
    for stages in (_lib.BWD_STAGE_ALL, _lib.BWD_STAGE_ALL | _lib.BWD_STAGE_UNFUSED):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty_like(lse)
        ws = torch.empty(lib.b200attn_bwd_workspace_bytes(B, H, H, M, N, D) // 4, dtype=torch.float32, device=device())
        bp = _lib.BwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), _lib.tensor4(do),
                            _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv), lse.data_ptr(), delta.data_ptr(),
                            ws.data_ptr(), B, H, H, M, N, D, dt, dt, 0, 1 / math.sqrt(D), 0.0, 0, 0, status.data_ptr(),
                            1, lo, hi)
        _lib.check(lib.b200attn_bwd_stages(bp, st, stages), "bwd")
        for name, a, b_, c in zip(("dq", "dk", "dv"), (dq, dk, dv), g_low, g_ref):
            assert_2x_rule(name, a, b_, c)
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [16, 128])
def test_merge_partial_store_equals_merge_then_round(D, dtype):
    """The merge that rounds straight into a 16-bit tensor (transposed layout here) gives the bits of
    the in-place fp32 merge followed by a cast, and the same log-normaliser; rows that one or both
    partials leave empty (log-normaliser -inf) included."""
    B, H, M = 2, 3, 77
    g = torch.Generator(device=device()).manual_seed(5)
    o_a = torch.randn(B, H, M, D, device=device(), generator=g)
    o_b = torch.randn(B, H, M, D, device=device(), generator=g)
    l_a = torch.randn(B, H, M, device=device(), generator=g) * 3
    l_b = torch.randn(B, H, M, device=device(), generator=g) * 3
    l_a[0, 0, :5] = float("-inf")
    l_b[0, 0, 3:9] = float("-inf")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    ref_o, ref_l = o_a.clone(), l_a.clone()
    _lib.check(lib.b200attn_merge_partial(ref_o.data_ptr(), ref_l.data_ptr(), o_b.data_ptr(), l_b.data_ptr(),
                                          B * H, M, D, M, 0, M, 0, 0, st), "merge_partial")
    out = torch.empty(B, M, H, D, dtype=dtype, device=device()).transpose(1, 2)
    got_l = l_a.clone()
    _lib.check(lib.b200attn_merge_partial_store(o_a.data_ptr(), got_l.data_ptr(), o_b.data_ptr(), l_b.data_ptr(),
                                                B, H, M, D, _lib.tensor4(out), _lib.dtype_code(dtype), st),
               "merge_partial_store")
    torch.cuda.synchronize()
    assert torch.equal(out, ref_o.to(dtype))
    assert torch.equal(got_l, ref_l)


@pytest.mark.parametrize("D,N,out_contig", [(128, 1000, True), (64, 777, True), (32, 300, True), (128, 520, False)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dv_accumulate_adds_in_fp32_and_rounds_once(D, N, out_contig, dtype):
    """`dv_accumulate`: the backward adds its dV onto the 16-bit gradient already in the dv buffer (what the
    second region of piecewise attention does, `piecewise.py:132-180` sums both regions into one dv). The
    result must be round(float(previous) + fp32 dV): compared with a plain call's dV it may differ from
    round(previous + round(dV)) by one rounding of dV only. dQ and dK are untouched by the flag. The last
    case has dv in the transposed layout, which the kernel stores from registers instead of through TMA."""
    B, H, M = 2, 3, 333
    g = torch.Generator(device=device()).manual_seed(11)
    q, do = (torch.randn(B, H, M, D, device=device(), dtype=dtype, generator=g) for _ in range(2))
    k, v = (torch.randn(B, H, N, D, device=device(), dtype=dtype, generator=g) for _ in range(2))
    prev = torch.randn(B, H, N, D, device=device(), dtype=dtype, generator=g)
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    dt = _lib.dtype_code(dtype)
    status = torch.zeros(1, dtype=torch.int32, device=device())
    o = torch.empty_like(q)
    lse = torch.empty(B, H, M, dtype=torch.float32, device=device())
    fp = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(), B, H, H, M, N, D,
                        dt, dt, 1, 1 / math.sqrt(D), 0.0, 0, 0, status.data_ptr())
    _lib.check(lib.b200attn_fwd(fp, st), "fwd")
    results = []
    for accumulate in (0, 1):
        dq, dk = torch.empty_like(q), torch.empty_like(k)
        dv = (prev.clone() if out_contig else prev.transpose(1, 2).contiguous().transpose(1, 2)) if accumulate \
            else torch.empty_like(v)
        delta = torch.empty_like(lse)
        ws = torch.empty(max(lib.b200attn_bwd_workspace_bytes(B, H, H, M, N, D), 4) // 4, dtype=torch.float32,
                         device=device())
        bp = _lib.BwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), _lib.tensor4(do),
                            _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv), lse.data_ptr(), delta.data_ptr(),
                            ws.data_ptr(), B, H, H, M, N, D, dt, dt, 1, 1 / math.sqrt(D), 0.0, 0, 0, status.data_ptr(),
                            0, 0, 0, None, accumulate)
        _lib.check(lib.b200attn_bwd_stages(bp, st, _lib.BWD_STAGE_ALL | _lib.BWD_STAGE_UNFUSED), "bwd")
        results.append((dq, dk, dv))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    (dq0, dk0, dv0), (dq1, dk1, dv1) = results
    assert torch.equal(dq0, dq1) and torch.equal(dk0, dk1)
    want = prev.float() + dv0.float()            # dv0 = round(fp32 dV): within half an ulp of dV
    ulp = torch.finfo(dtype).eps
    tol = (dv0.float().abs() * ulp / 2 + want.abs() * ulp / 2 + 1e-6)
    assert bool(((dv1.float() - want).abs() <= tol * 1.01).all())
    assert not torch.equal(dv1, prev)

"""Pins the tcgen05 operand layouts the kernels rely on, one 128 x N tile product at a time."""
import pytest
import torch

from flagattention_b200 import _lib

pytestmark = pytest.mark.gpu

SW = {128: (2, 3), 64: (4, 2), 32: (6, 1)}  # row bytes -> (descriptor swizzle code, TMA swizzle enum)


def desc_hi(lbo, sbo, swz):
    return ((lbo >> 4) & 0x3fff) << 16 | ((sbo >> 4) & 0x3fff) << 32 | (1 << 46) | (swz & 7) << 61


def idesc(bf16, m, n, a_mn, b_mn):
    f = 1 if bf16 else 0
    return (1 << 4) | (f << 7) | (f << 10) | (int(a_mn) << 15) | (int(b_mn) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24)


def run(a, b, ref, **kw):
    dev = a.device
    d = torch.full((128, kw["n"]), float("nan"), device=dev, dtype=torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = _lib.SelftestParams()
    p.a, p.b, p.d = a.data_ptr(), b.data_ptr(), d.data_ptr()
    p.a_cols, p.b_rows, p.b_cols = a.shape[1], b.shape[0], b.shape[1]
    p.bf16 = int(a.dtype == torch.bfloat16)
    p.status = status.data_ptr()
    for key, val in kw.items():
        setattr(p, key, val)
    lib = _lib.load()
    _lib.check(lib.b200attn_umma_selftest(p, torch.cuda.current_stream().cuda_stream), "selftest")
    torch.cuda.synchronize()
    assert status.item() == 0
    torch.testing.assert_close(d, ref, atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols,row_bytes", [(64, 128), (32, 64), (16, 32)])
def test_kmajor_operands(dtype, cols, row_bytes):
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    a = torch.randn(128, cols, device=dev, dtype=dtype)
    b = torch.randn(128, cols, device=dev, dtype=dtype)
    us, ts = SW[row_bytes]
    run(a, b, a.float() @ b.float().T, box_cols=cols, swizzle=ts, a_in_tmem=0, n=128, k_steps=cols // 16,
        idesc=idesc(bf, 128, 128, 0, 0), a_desc_hi=desc_hi(16, 8 * row_bytes, us),
        b_desc_hi=desc_hi(16, 8 * row_bytes, us), a_step_bytes=32, b_step_bytes=32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kmajor_two_chunks(dtype):
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    a = torch.randn(128, 128, device=dev, dtype=dtype)
    b = torch.randn(128, 128, device=dev, dtype=dtype)
    run(a, b, a.float() @ b.float().T, box_cols=64, swizzle=3, a_in_tmem=0, n=128, k_steps=8,
        idesc=idesc(bf, 128, 128, 0, 0), a_desc_hi=desc_hi(16, 1024, 2), b_desc_hi=desc_hi(16, 1024, 2),
        a_step_bytes=32, b_step_bytes=32, a_chunk_steps=4, b_chunk_steps=4, a_chunk_bytes=16384,
        b_chunk_bytes=16384)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dcols,row_bytes", [(128, 128), (64, 128), (32, 64), (16, 32)])
def test_tmem_a_times_mnmajor_b(dtype, dcols, row_bytes):
    """P (packed 16-bit pairs in TMEM) x V (rows = contraction index, read MN-major)."""
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    a = torch.randn(128, 128, device=dev, dtype=dtype)
    v = torch.randn(128, dcols, device=dev, dtype=dtype)
    us, ts = SW[row_bytes]
    run(a, v, a.float() @ v.float(), box_cols=min(dcols, 64), swizzle=ts, a_in_tmem=1, n=dcols, k_steps=8,
        idesc=idesc(bf, 128, dcols, 0, 1), a_desc_hi=0, b_desc_hi=desc_hi(128 * row_bytes, 8 * row_bytes, us),
        a_step_bytes=0, b_step_bytes=16 * row_bytes)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_mnmajor_a(dtype):
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    am = torch.randn(128, 128, device=dev, dtype=dtype)
    b = torch.randn(128, 128, device=dev, dtype=dtype)
    run(am, b, am.float().T @ b.float().T, box_cols=64, swizzle=3, a_in_tmem=0, n=128, k_steps=8,
        idesc=idesc(bf, 128, 128, 1, 0), a_desc_hi=desc_hi(16384, 1024, 2), b_desc_hi=desc_hi(16, 1024, 2),
        a_step_bytes=2048, b_step_bytes=32, b_chunk_steps=4, b_chunk_bytes=16384)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_mnmajor_a_times_mnmajor_b_n64(dtype):
    """dQ^T = K^T dS^T of the fused backward: both operands stored with the contraction index as
    the row (K as two 64-column chunks, dS^T as one 128-byte-row tile), N = 64."""
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    am = torch.randn(128, 128, device=dev, dtype=dtype)
    bm = torch.randn(128, 64, device=dev, dtype=dtype)
    run(am, bm, am.float().T @ bm.float(), box_cols=64, swizzle=3, a_in_tmem=0, n=64, k_steps=8,
        idesc=idesc(bf, 128, 64, 1, 1), a_desc_hi=desc_hi(16384, 1024, 2), b_desc_hi=desc_hi(16384, 1024, 2),
        a_step_bytes=2048, b_step_bytes=2048)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols,row_bytes", [(128, 128), (64, 128), (32, 64), (16, 32)])
def test_tmem_a_filled_by_tcgen05_cp(dtype, cols, row_bytes):
    """A operand staged by TMA in shared memory, moved to TMEM one K=16 slice at a time with
    tcgen05.cp (same descriptors as the shared-memory A operand), consumed from TMEM."""
    dev = torch.device("cuda", 0)
    bf = dtype == torch.bfloat16
    a = torch.randn(128, cols, device=dev, dtype=dtype)
    b = torch.randn(128, cols, device=dev, dtype=dtype)
    us, ts = SW[row_bytes]
    box = min(cols, 64)
    run(a, b, a.float() @ b.float().T, box_cols=box, swizzle=ts, a_in_tmem=2, n=128, k_steps=cols // 16,
        idesc=idesc(bf, 128, 128, 0, 0), a_desc_hi=desc_hi(16, 8 * row_bytes, us),
        b_desc_hi=desc_hi(16, 8 * row_bytes, us), a_step_bytes=32, b_step_bytes=32,
        a_chunk_steps=box // 16, b_chunk_steps=box // 16, a_chunk_bytes=128 * row_bytes,
        b_chunk_bytes=128 * row_bytes)

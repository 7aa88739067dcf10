"""Generates the golden fixtures in this directory from the REFERENCE's own code.

Run where the reference checkout is available (read-only), with ``FLAG_ATTN_REF`` pointing at it:
``FLAG_ATTN_REF=<checkout> python tests/golden/make_golden.py``. It needs no GPU:

* ``attention_*.npz``: inputs and outputs of the reference's PyTorch attention
  (``flag_attn.testing.flash_attention``, fp32-upcast and native-dtype), and gradients through it.
* ``triton_interp_*.npz``: outputs of the reference's Triton kernels (``_fwd_kernel``,
  ``_total_attention_kernel``, ``_bwd_preprocess``, ``_bwd_kv_kernel``, ``_bwd_q_kernel``,
  ``recompute_mask_kernel``) executed by the Triton interpreter on CPU tensors.
* ``dropout_masks.npz``: keep-masks from the reference's ``recompute_mask_kernel`` (interpreter).
* ``split_heuristic.json``: ``num_splits_herustic`` evaluated on a grid of shapes.
* ``paged_*.npz``: inputs and output of the reference's PyTorch paged attention
  (``flag_attn.testing.paged_attention``, ``testing/paged.py:19-66``).

* ``piecewise_*.npz``: inputs, outputs and autograd gradients of the reference's PyTorch piecewise
  attention (``flag_attn.testing.piecewise_attention``, ``testing/piecewise.py:19-49``).

``python tests/golden/make_golden.py paged`` (or any of ``split masks attention triton paged piecewise``)
regenerates only the named groups.

The fixtures travel with the repository; the tests never read the reference checkout.
"""
import json
import math
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
REF = os.environ.get("FLAG_ATTN_REF")
if not REF or not os.path.isdir(os.path.join(REF, "src", "flag_attn")):
    raise SystemExit("set FLAG_ATTN_REF to a checkout of the reference (the directory that holds src/flag_attn)")
sys.path.insert(0, os.path.join(REF, "src"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    """16-bit tensors are stored as their raw uint16 bit patterns."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def make_inputs(seed, B, Hq, Hk, M, N, D, dtype, std=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, Hq, M, D, generator=g) * std).to(dtype)
    k = (torch.randn(B, Hk, N, D, generator=g) * std).to(dtype)
    v = (torch.randn(B, Hk, N, D, generator=g) * std).to(dtype)
    do = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    return q, k, v, do


# The dropout cases keep B * Hq * ceil(M / 16) >= 0.8 * 148 so that flash_attention does not take
# its split-KV branch, which refuses dropout (flash.py:107).
ATTENTION_CASES = [
    # name, seed, B, Hq, Hk, M, N, D, dtype, causal, dropout_p, std
    ("c1_plumbing", 0, 1, 4, 4, 128, 128, 64, torch.float16, False, 0.0, 1.0),
    ("gqa_causal_bf16", 1, 1, 4, 2, 136, 200, 128, torch.bfloat16, True, 0.0, 1.0),
    ("mqa_ragged_fp16", 2, 1, 4, 1, 129, 257, 32, torch.float16, False, 0.0, 2.0),
    ("larger_m_causal", 3, 1, 2, 2, 300, 40, 16, torch.bfloat16, True, 0.0, 1.0),
    ("dropout_fp16", 4, 2, 4, 4, 240, 192, 32, torch.float16, True, 0.5, 1.0),
    ("dropout_bf16_gqa", 5, 2, 4, 2, 240, 130, 64, torch.bfloat16, False, 0.8, 1.0),
]


def gen_attention():
    from flag_attn.testing import flash_attention as ref_attention
    from flag_attn.testing.dropout import recompute_mask_kernel
    for (name, seed, B, Hq, Hk, M, N, D, dtype, causal, p, std) in ATTENTION_CASES:
        q, k, v, do = make_inputs(seed, B, Hq, Hk, M, N, D, dtype, std)
        mask = None
        rng_seed, rng_offset = 1234567 + seed, 9876 * (seed + 1)
        if p > 0:
            mask = torch.full((B, Hq, M, N), True, dtype=torch.bool)
            recompute_mask_kernel[(M, B, Hq)](mask, B, Hq, M, N, p, rng_seed, rng_offset)
        out = {}
        for tag, up in (("ref32", True), ("lowp", False)):
            o, lse, tot = ref_attention(q, k, v, causal, dropout_p=p, dropout_mask=mask,
                                        return_log_normalizer=True, return_total_attention=True,
                                        upcast=up)
            out[f"o_{tag}"] = bits(o)
            out[f"lse_{tag}"] = bits(lse)
            out[f"tot_{tag}"] = bits(tot)
            if not up:
                continue  # native-dtype run: only O is kept (it sets the error budget)
            qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            og = ref_attention(qg, kg, vg, causal, dropout_p=p, dropout_mask=mask, upcast=up)
            dq, dk, dv = torch.autograd.grad(og, (qg, kg, vg), do)
            out[f"dq_{tag}"], out[f"dk_{tag}"], out[f"dv_{tag}"] = bits(dq), bits(dk), bits(dv)
        meta = dict(name=name, seed=seed, B=B, Hq=Hq, Hk=Hk, M=M, N=N, D=D,
                    dtype=str(dtype).split(".")[1], causal=causal, dropout_p=p,
                    rng_seed=rng_seed, rng_offset=rng_offset)
        np.savez_compressed(HERE / f"attention_{name}.npz", q=bits(q), k=bits(k), v=bits(v), do=bits(do),
                            mask=(np.packbits(mask.numpy()) if mask is not None else np.zeros(0, np.uint8)),
                            meta=json.dumps(meta), **out)
        print("wrote", name)


def gen_triton_interp():
    """The reference's Triton kernels themselves, on one tiny GQA case, via the interpreter."""
    import triton
    from flag_attn import flash as F
    from flag_attn.total import _total_attention_kernel
    B, Hq, Hk, M, N, D = 1, 4, 2, 48, 80, 32
    dtype = torch.float16
    BM, BN = 32, 32
    for causal in (False, True):
        for p in (0.0, 0.3):
            q, k, v, do = make_inputs(11, B, Hq, Hk, M, N, D, dtype)
            sm_scale = 1.0 / math.sqrt(D)
            seed, offset = 4242, 1000
            groups = Hq // Hk
            o = torch.empty_like(q)
            L = torch.empty((B, Hq, M), dtype=torch.float32)
            F._fwd_kernel[(triton.cdiv(M, BM), Hq, B)](
                q, k, v, sm_scale, p, seed, offset, L, o,
                *q.stride(), *k.stride(), *v.stride(), *o.stride(),
                B, Hq, M, N, N - M, groups,
                BLOCK_M=BM, BLOCK_N=BN, BLOCK_DMODEL=D, IS_CAUSAL=causal, IS_DROPOUT=p > 0,
                LARGER_M=M > N, DIVISIBLE_M=M % BM == 0, DIVISIBLE_N=N % BN == 0)
            tot = torch.empty((B, Hq, N), dtype=torch.float32)
            _total_attention_kernel[(triton.cdiv(N, BN), Hq, B)](
                q, k, L, tot, sm_scale, *q.stride(), *k.stride(),
                B, Hq, M, N, N - M, groups,
                BLOCK_M=BM, BLOCK_DMODEL=D, BLOCK_N=BN, CAUSAL=causal,
                DIVISIBLE_M=M % BM == 0, DIVISIBLE_N=N % BN == 0)
            delta = torch.empty_like(L)
            F._bwd_preprocess[(triton.cdiv(M, BM), Hq, B)](
                o, do, delta, *o.stride(), *do.stride(), *delta.stride(), M,
                BLOCK_M=BM, D_HEAD=D, DIVISIBLE_M=M % BM == 0)
            dk = torch.empty((B, Hq, N, D), dtype=dtype)
            dv = torch.empty((B, Hq, N, D), dtype=dtype)
            F._bwd_kv_kernel[(triton.cdiv(N, BN), Hq, B)](
                q, k, v, sm_scale, do, dk, dv, L, delta, p, seed, offset,
                *q.stride(), *k.stride(), *v.stride(), *do.stride(), *dk.stride(), *dv.stride(),
                B, Hq, M, N, N - M, groups,
                BLOCK_M=BM, BLOCK_DMODEL=D, BLOCK_N=BN, CAUSAL=causal, IS_DROPOUT=p > 0,
                DIVISIBLE_M=M % BM == 0, DIVISIBLE_N=N % BN == 0)
            dq = torch.zeros_like(q)
            F._bwd_q_kernel[(triton.cdiv(M, BM), Hq, B)](
                q, k, v, sm_scale, do, dq, L, delta, p, seed, offset,
                *q.stride(), *k.stride(), *v.stride(), *do.stride(), *dq.stride(),
                B, Hq, M, N, N - M, groups,
                BLOCK_M=BM, BLOCK_DMODEL=D, BLOCK_N=BN, CAUSAL=causal, IS_DROPOUT=p > 0,
                LARGER_M=M > N, DIVISIBLE_M=M % BM == 0, DIVISIBLE_N=N % BN == 0)
            dk = dk.reshape(B, Hk, groups, N, D).sum(2)
            dv = dv.reshape(B, Hk, groups, N, D).sum(2)
            meta = dict(B=B, Hq=Hq, Hk=Hk, M=M, N=N, D=D, dtype="float16", causal=causal, dropout_p=p,
                        rng_seed=seed, rng_offset=offset, input_seed=11)
            name = f"triton_interp_causal{int(causal)}_p{int(p * 10)}"
            np.savez_compressed(HERE / f"{name}.npz", q=bits(q), k=bits(k), v=bits(v), do=bits(do),
                                o=bits(o), lse=bits(L), tot=bits(tot), delta=bits(delta),
                                dq=bits(dq), dk=bits(dk), dv=bits(dv), meta=json.dumps(meta))
            print("wrote", name)


def gen_masks():
    from flag_attn.testing.dropout import recompute_mask_kernel
    cases = [(123456789, 0, 0.3), (123456789, 123456789123456789, 0.5), ((1 << 40) + 7, 12, 0.8),
             (5, (1 << 31) - 100, 0.1), (77, (1 << 32) - 1000, 0.5)]
    B, H, M, N = 1, 2, 5, 1500
    out = {}
    for i, (seed, offset, p) in enumerate(cases):
        mask = torch.full((B, H, M, N), True, dtype=torch.bool)
        recompute_mask_kernel[(M, B, H)](mask, B, H, M, N, p, seed, offset)
        out[f"mask{i}"] = np.packbits(mask.numpy())
    np.savez_compressed(HERE / "dropout_masks.npz", shape=np.array([B, H, M, N]),
                        cases=json.dumps(cases), **out)
    print("wrote dropout_masks")


def gen_split_table():
    from flag_attn.split_kv import num_splits_herustic
    rows = []
    for num_sms in (108, 132, 148):
        for B in (1, 2, 8):
            for H in (1, 2, 4, 16, 32):
                for M in (1, 2, 4, 16, 128, 512, 4096):
                    for N in (10, 128, 257, 4000, 8202, 32768, 524288):
                        rows.append([B, H, M, N, num_sms, num_splits_herustic(B, H, M, N, 16, 128, num_sms, 128)])
    (HERE / "split_heuristic.json").write_text(json.dumps(rows))
    print("wrote split_heuristic", len(rows))


PAGED_CASES = [
    # name, seed, num_seqs, Hq, group, D, block, num_blocks, max_len, dtype
    ("paged_mha_fp16", 11, 3, 2, 1, 64, 16, 12, 100, torch.float16),
    ("paged_gqa8_fp16", 12, 2, 8, 8, 32, 16, 12, 70, torch.float16),
    ("paged_gqa4_bf16", 13, 2, 4, 4, 128, 128, 5, 300, torch.bfloat16),
]


def gen_paged():
    from flag_attn.testing.paged import attention as ref_paged
    for name, seed, num_seqs, Hq, group, D, block, num_blocks, max_len, dtype in PAGED_CASES:
        g = torch.Generator().manual_seed(seed)
        Hkv = Hq // group
        scale = D ** -0.5
        q = ((torch.rand(num_seqs, Hq, D, generator=g) * 2 - 1) * scale * 8).to(dtype)
        kc = ((torch.rand(num_blocks, Hkv, block, D, generator=g) * 2 - 1) * scale * 8).to(dtype)
        vc = ((torch.rand(num_blocks, Hkv, block, D, generator=g) * 2 - 1)).to(dtype)
        lens = torch.randint(1, max_len, (num_seqs,), generator=g, dtype=torch.int32)
        lens[0] = max_len
        per_seq = (max_len + block - 1) // block
        tables = torch.randint(0, num_blocks, (num_seqs, per_seq), generator=g, dtype=torch.int32)
        out = ref_paged(q, kc, vc, tables, lens, scale)
        out32 = ref_paged(q.float(), kc.float(), vc.float(), tables, lens, scale)
        np.savez_compressed(HERE / f"{name}.npz", q=bits(q), key_cache=bits(kc), value_cache=bits(vc),
                            context_lens=lens.numpy(), block_tables=tables.numpy(), out=bits(out),
                            out_fp32=out32.numpy(), scale=np.float32(scale),
                            dtype=np.array(str(dtype)))
        print("wrote", name)


PIECEWISE_CASES = [
    # name, seed, B, H, M, N, D, dtype, causal, w
    ("piecewise_causal_fp16", 21, 1, 2, 136, 200, 32, torch.float16, True, 68),
    ("piecewise_full_bf16", 22, 1, 2, 300, 180, 64, torch.bfloat16, False, 210),
    ("piecewise_causal_larger_m", 23, 1, 1, 260, 129, 16, torch.bfloat16, True, 195),
]


def gen_piecewise():
    from flag_attn.testing.piecewise import attention as ref_piecewise
    for name, seed, B, H, M, N, D, dtype, causal, w in PIECEWISE_CASES:
        g = torch.Generator().manual_seed(seed)
        q1, q2, do = (torch.randn(B, H, M, D, generator=g).to(dtype) for _ in range(3))
        k1, k2, v = (torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(3))
        leaves = [t.clone().requires_grad_(True) for t in (q1, k1, q2, k2, v)]
        o32 = ref_piecewise(*leaves, w, causal, upcast=True)
        g32 = torch.autograd.grad(o32, leaves, do)
        leaves_low = [t.clone().requires_grad_(True) for t in (q1, k1, q2, k2, v)]
        o_low = ref_piecewise(*leaves_low, w, causal, upcast=False)
        g_low = torch.autograd.grad(o_low, leaves_low, do)
        arrays = dict(q1=bits(q1), k1=bits(k1), q2=bits(q2), k2=bits(k2), v=bits(v), do=bits(do),
                      o_upcast=bits(o32.detach()), o_native=bits(o_low.detach()),
                      meta=np.array(json.dumps(dict(B=B, H=H, M=M, N=N, D=D, dtype=str(dtype)[6:], causal=causal, w=w))))
        for nm, a, b_ in zip(("dq1", "dk1", "dq2", "dk2", "dv"), g32, g_low):
            arrays[nm + "_upcast"] = bits(a)
            arrays[nm + "_native"] = bits(b_)
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        print("wrote", name)


if __name__ == "__main__":
    torch.set_num_threads(8)
    groups = {"split": gen_split_table, "masks": gen_masks, "attention": gen_attention,
              "triton": gen_triton_interp, "paged": gen_paged, "piecewise": gen_piecewise}
    for key in (sys.argv[1:] or list(groups)):
        groups[key]()

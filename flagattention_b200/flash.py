"""Host side of ``flash_attention``: the same call contract as ``flag_attn.flash.attention``
(``flash.py:275-306`` of the reference; autograd function ``flash.py:37-272``), dispatching to the
sm_100a kernels in ``libb200attn.so``.

Everything here is shape bookkeeping, allocation and the autograd contract; all arithmetic runs in
the CUDA library. There is no fallback path: a missing library or an unsupported device raises.
"""
from __future__ import annotations

import math
import os

import torch

from . import _lib
from . import status as _status
from .rng_state import as_u64, reserve_philox_stream
from .split_kv import choose_num_splits
from .status import check_device_status

__all__ = ["flash_attention", "FlashAttentionFunction", "check_device_status", "get_fwd_config",
           "get_bwd_config"]

_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128)
# Largest dropout keep-decision cache (bytes, one bit per attention score) handed from forward to backward.
_KEEP_MASK_LIMIT = 1 << 30


def _status_word(device: torch.device) -> torch.Tensor:
    """The device's status word, after a non-blocking look at what earlier launches reported
    (``status.poll``): a kernel that gave up on a bounded wait makes one of the next calls raise."""
    return _status.poll(device)


def get_fwd_config(B, H, M, N, D, causal):
    """Counterpart of the reference's tile-configuration hook (``flash.py:311-342``): returns
    ``(BLOCK_M, BLOCK_N, num_stages, num_warps)`` of the forward kernel that would run. The reference
    documents its hook as replaceable at run time (``examples/use_cutom_config_func.py:18-23`` assigns
    ``flag_attn.flash.get_fwd_config``). Here tile shapes are template parameters of the CUDA kernels,
    so the function reports them and assigning another one is accepted and has no effect."""
    stages = 2 if D == 128 else (3 if D == 64 else 4)
    return (256, 128, stages, 12)   # two 128-row query tiles per CTA, 128-key K/V tiles, 384 threads


def get_bwd_config(B, H, M, N, D, causal):
    """Counterpart of the reference's backward hook (``flash.py:514-539``); see ``get_fwd_config``.
    The backward keeps 128 rows resident per CTA and streams 64 columns per step."""
    fused = D in (64, 128)
    return (128, 64, 3 if D == 128 else 4, 14 if fused else 10)


def _tma_ready(x: torch.Tensor) -> torch.Tensor:
    """Returns ``x`` or a contiguous copy that satisfies what TMA needs: unit feature stride,
    16-byte aligned base and strides. The reference only copies when the feature stride is not 1
    (``flash.py:28-31``); the extra cases cannot be expressed as a tensor map."""
    strides = x.stride()
    ok = strides[-1] == 1 and x.data_ptr() % 16 == 0
    if ok:
        esize = x.element_size()
        for size, stride in zip(x.shape[:-1], strides[:-1]):
            if size > 1 and (stride <= 0 or (stride * esize) % 16 != 0):
                ok = False
                break
    return x if ok else x.contiguous()


_SM_COUNT = {}
_SPLIT_COUNTS = {}  # (B, H, Hk, M, N, D, SMs) -> tuned split count (a pure function of the key)


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _SM_COUNT.get(idx)
    if n is None:
        n = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def _split_kv_forward(lib, q, k, v, causal, sm_scale, num_sms, stream, status):
    """Split-KV forward on TMA-ready q, k, v: returns (o in q.dtype, log-normaliser [B, H, M])."""
    B, H, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    device = q.device
    key = (B, H, Hk, M, N, D, num_sms)
    S = _SPLIT_COUNTS.get(key)
    if S is None:
        if len(_SPLIT_COUNTS) > 4096:
            _SPLIT_COUNTS.clear()
        S = _SPLIT_COUNTS[key] = int(lib.b200attn_splitkv_num_splits(B, H, Hk, M, N, D, num_sms))
    o = torch.empty((B, H, M, D), dtype=q.dtype, device=device)
    rows = B * H * M
    if S > 1:
        # one fp32 scratch allocation: per-split outputs (16-byte aligned rows) | per-split
        # normalisers. The log-normaliser is a tensor of its own: autograd saves it and callers may
        # keep it, which must not keep the partial outputs alive (the reference frees its partials
        # right after the combine).
        buf = torch.empty(rows * (S * D + S), dtype=torch.float32, device=device)
        part_o_ptr = buf.data_ptr()
        part_l_ptr = part_o_ptr + 4 * rows * S * D
        L = torch.empty((B, H, M), device=device, dtype=torch.float32)
    elif (H // Hk) * M <= 2:
        L = torch.empty((B, H, M), device=device, dtype=torch.float32)
        part_o_ptr = part_l_ptr = L.data_ptr()  # unused by the single-split streaming kernel
    else:
        L = torch.empty((B, H, M), device=device, dtype=torch.float32)
        fp = _lib.FwdParams(
            _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), L.data_ptr(),
            B, H, Hk, M, N, D, _lib.dtype_code(q.dtype), _lib.dtype_code(q.dtype),
            int(causal), sm_scale, 0.0, 0, 0, status.data_ptr())
        _lib.check(lib.b200attn_fwd(fp, stream), "b200attn_fwd")
        return o, L
    sp = _lib.SplitKVParams(
        _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o),
        L.data_ptr(), part_o_ptr, part_l_ptr,
        B, H, Hk, M, N, D, S, _lib.dtype_code(q.dtype), int(causal), sm_scale, status.data_ptr())
    _lib.check(lib.b200attn_fwd_splitkv(sp, stream), "b200attn_fwd_splitkv")
    return o, L


def flash_attention_split_kv(q, k, v, causal=False, sm_scale=None):
    """Forward-only attention over split keys/values ("flash decoding"): same arguments, checks and
    result as the reference operator (``split_kv.py:282-347``); the result has ``q``'s dtype
    whatever the split count. Not differentiable, like the reference's."""
    Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Dq == Dk == Dv
    assert Dk in _SUPPORTED_HEAD_DIMS
    B, H, M, D = q.shape
    Hk, Hv = k.shape[1], v.shape[1]
    assert Hk == Hv, "num of heads in k and v should be equal"
    assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("flash_attention_split_kv runs on CUDA tensors only (no CPU fallback)")
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("q, k, v must share dtype float16 or bfloat16")
    if not (q.device == k.device == v.device):
        raise ValueError("q, k, v must live on the same device")
    if k.shape[0] != B or v.shape[0] != B or v.shape[2] != k.shape[2]:
        raise ValueError("batch / sequence sizes of q, k, v are inconsistent")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    lib = _lib.load()
    device = q.device
    # (nothing below is recorded by autograd: the result is a fresh tensor filled by the library)
    if device.index == torch.cuda.current_device():
        o, _ = _split_kv_forward(lib, q, k, v, bool(causal), float(sm_scale), _sm_count(device),
                                 _lib.current_stream_ptr(device), _status_word(device))
    else:
        with torch.cuda.device(device):
            o, _ = _split_kv_forward(lib, q, k, v, bool(causal), float(sm_scale), _sm_count(device),
                                     _lib.current_stream_ptr(device), _status_word(device))
    return o


class FlashAttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, dropout_p, return_log_normalizer,
                return_total_attention, return_seed_offset):
        Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
        assert Dq == Dk == Dv, "feature size of q, k, v should be equal"
        assert Dk in _SUPPORTED_HEAD_DIMS
        B, H, M, D = q.shape
        N = k.shape[2]
        Hk, Hv = k.shape[1], v.shape[1]
        assert Hk == Hv, "num of heads in k and v should be equal"
        assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"
        if not (q.is_cuda and k.is_cuda and v.is_cuda):
            raise RuntimeError("flash_attention runs on CUDA tensors only (no CPU fallback)")
        if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("q, k, v must share dtype float16 or bfloat16")
        if not (q.device == k.device == v.device):
            raise ValueError("q, k, v must live on the same device")
        if k.shape[0] != B or v.shape[0] != B or v.shape[2] != N:
            raise ValueError("batch / sequence sizes of q, k, v are inconsistent")

        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        dropout_p = float(dropout_p)
        is_dropout = dropout_p > 0

        q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
        lib = _lib.load()
        device = q.device
        with torch.cuda.device(device):
            if is_dropout:
                seed, offset = reserve_philox_stream(B * H * M * N, device)
            else:
                seed, offset = 0, 0
            num_sms = _sm_count(device)
            # The reference's rule decides WHETHER the call takes the split-KV branch (and with it
            # the branch's no-dropout restriction, flash.py:73-77); how many splits this library
            # then uses is its own tuning and does not change the result.
            num_splits = choose_num_splits(B, H, M, N, num_sms)
            stream = _lib.current_stream_ptr(device)
            status = _status_word(device)
            keep_mask = None
            if num_splits > 1:
                assert not is_dropout, "Cannot apply dropout with splitkv."
                o, L = _split_kv_forward(lib, q, k, v, bool(causal), float(sm_scale), num_sms, stream,
                                         status)
            else:
                L = torch.empty((B, H, M), device=device, dtype=torch.float32)
                # Backward's row statistic is dot(O, dO): keep the fp32 O for bf16 dropout gradients,
                # as the reference does (flash.py:86-90).
                out_dtype = (torch.float32 if is_dropout and q.dtype == torch.bfloat16
                             and any(ctx.needs_input_grad[:3]) else q.dtype)
                o = torch.empty_like(q, dtype=out_dtype)
                if _tma_ready(o) is not o:
                    o = torch.empty(q.shape, dtype=out_dtype, device=device)
                # With dropout, the keep decisions (one bit per score) are kept for the backward when
                # they fit in _KEEP_MASK_LIMIT bytes: re-evaluating Philox there costs more than the
                # rest of the backward. Larger problems recompute, as the reference always does.
                if is_dropout and any(ctx.needs_input_grad[:3]):
                    mask_bytes = lib.b200attn_keep_mask_bytes(B, H, M, N)
                    if mask_bytes <= _KEEP_MASK_LIMIT:
                        keep_mask = torch.empty(mask_bytes // 4, dtype=torch.int32, device=device)
                fp = _lib.FwdParams(
                    _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), L.data_ptr(),
                    B, H, Hk, M, N, D, _lib.dtype_code(q.dtype), _lib.dtype_code(out_dtype),
                    int(bool(causal)), float(sm_scale), dropout_p, as_u64(seed), as_u64(offset),
                    status.data_ptr(), 0, 0, 0, keep_mask.data_ptr() if keep_mask is not None else None)
                _lib.check(lib.b200attn_fwd(fp, stream), "b200attn_fwd")

            tot_attn = None
            if return_total_attention:
                tot_attn = torch.empty((B, H, N), device=device, dtype=torch.float32)
                ws = torch.empty(lib.b200attn_total_workspace_bytes(B, H, M) // 4, dtype=torch.float32,
                                 device=device)
                tp = _lib.TotalParams(
                    _lib.tensor4(q), _lib.tensor4(k), L.data_ptr(), tot_attn.data_ptr(), ws.data_ptr(),
                    B, H, Hk, M, N, D, _lib.dtype_code(q.dtype), int(bool(causal)), float(sm_scale),
                    status.data_ptr())
                _lib.check(lib.b200attn_total_attention(tp, stream), "b200attn_total_attention")

        ctx.save_for_backward(q, k, v, o, L)
        ctx.keep_mask = keep_mask
        ctx.sm_scale = sm_scale
        ctx.causal = bool(causal)
        ctx.dropout_p = dropout_p
        ctx.seed = seed
        ctx.offset = offset
        o = o.to(q.dtype)

        if return_log_normalizer or return_total_attention or return_seed_offset:
            return (
                o,
                L if return_log_normalizer else None,
                tot_attn if return_total_attention else None,
                seed if is_dropout and return_seed_offset else None,
                offset if is_dropout and return_seed_offset else None,
            )
        return o

    @staticmethod
    def backward(ctx, do, *ignored):
        q, k, v, o, L = ctx.saved_tensors
        B, H, M, D = q.shape
        N = k.shape[2]
        Hk = k.shape[1]
        device = q.device
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        do = _tma_ready(do)
        lib = _lib.load()
        with torch.cuda.device(device):
            stream = _lib.current_stream_ptr(device)
            status = _status_word(device)
            dq = torch.empty_like(q)
            if _tma_ready(dq) is not dq:
                dq = torch.empty(q.shape, dtype=q.dtype, device=device)
            dk = torch.empty((B, Hk, N, D), dtype=k.dtype, device=device)
            dv = torch.empty((B, Hk, N, D), dtype=v.dtype, device=device)
            delta = torch.empty_like(L)
            ws_bytes = lib.b200attn_bwd_workspace_bytes(B, H, Hk, M, N, D)
            workspace = torch.empty(max(ws_bytes, 4) // 4, dtype=torch.float32, device=device)
            bp = _lib.BwdParams(
                _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), _lib.tensor4(do),
                _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv),
                L.data_ptr(), delta.data_ptr(), workspace.data_ptr(),
                B, H, Hk, M, N, D, _lib.dtype_code(q.dtype), _lib.dtype_code(o.dtype),
                int(ctx.causal), float(ctx.sm_scale), float(ctx.dropout_p),
                as_u64(ctx.seed), as_u64(ctx.offset), status.data_ptr(), 0, 0, 0,
                ctx.keep_mask.data_ptr() if ctx.keep_mask is not None else None)
            # At D = 128 and 64 the library produces dQ inside the dK/dV pass, summing the key blocks'
            # contributions by fp32 reductions in global memory: faster, but the summation order (and
            # so the last bit of dQ) can differ between runs. torch.use_deterministic_algorithms(True)
            # selects the two separate kernels, whose results are reproducible bit for bit.
            stages = _lib.BWD_STAGE_ALL
            if torch.are_deterministic_algorithms_enabled():
                stages |= _lib.BWD_STAGE_UNFUSED
            _lib.check(lib.b200attn_bwd_stages(bp, stream, stages), "b200attn_bwd_stages")
        return dq, dk, dv, None, None, None, None, None, None


def flash_attention(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
                    return_log_normalizer=False, return_total_attention=False,
                    return_seed_offset=False):
    """FlashAttention forward (and, through autograd, backward) on B200.

    Arguments:
        q: ``(batch, heads_q, seqlen_q, headdim)`` fp16/bf16 CUDA tensor.
        k, v: ``(batch, heads_k, seqlen_k, headdim)``; ``heads_q`` must be a multiple of ``heads_k``.
        causal: bottom-right aligned causal mask (query ``m`` sees key ``n`` iff
            ``n <= m + seqlen_k - seqlen_q``).
        sm_scale: softmax scale, default ``1/sqrt(headdim)``.
        dropout_p: dropout probability on the attention weights; the Philox stream is taken from
            the default CUDA generator.
        return_log_normalizer / return_total_attention / return_seed_offset: when any is set the
            result is the 5-tuple ``(out, log_normalizer|None, total_attention|None, seed|None,
            offset|None)``; otherwise just ``out``.
    """
    return FlashAttentionFunction.apply(q, k, v, causal, sm_scale, dropout_p, return_log_normalizer,
                                        return_total_attention, return_seed_offset)

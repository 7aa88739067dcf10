"""ctypes binding of ``libb200attn.so`` (declared in ``include/b200attn.h``).

The library is loaded lazily from the package directory (or from ``$B200ATTN_LIB``). There is no
fallback: if the shared object is missing, loading raises, and every operator that needs it fails.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_uint8,
                    c_uint32, c_uint64, c_void_p)
from pathlib import Path

import torch

F16, BF16, F32 = 0, 1, 2
_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

ERROR_NAMES = {0: "OK", -1: "EINVAL", -2: "EUNSUPPORTED", -3: "ECUDA", -4: "ETIMEOUT"}

# Stage bits of b200attn_bwd_stages (include/b200attn.h).
BWD_STAGE_PREP, BWD_STAGE_KV, BWD_STAGE_Q, BWD_STAGE_ALL, BWD_STAGE_UNFUSED, BWD_STAGE_ACC_ZEROED = 1, 2, 4, 7, 8, 16
# Open ends of the visibility band (FwdParams.dist_min / dist_max).
BAND_OPEN_MIN, BAND_OPEN_MAX = -(2 ** 31), 2 ** 31 - 1


class Tensor4(Structure):
    _fields_ = [("ptr", c_void_p), ("stride", c_int64 * 4)]


class FwdParams(Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("lse", c_void_p),
        ("B", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("M", c_int32), ("N", c_int32), ("D", c_int32),
        ("dtype", c_int32), ("o_dtype", c_int32), ("causal", c_int32),
        ("sm_scale", c_float), ("dropout_p", c_float),
        ("seed", c_uint64), ("offset", c_uint64),
        ("status", c_void_p),
        ("band", c_int32), ("dist_min", c_int32), ("dist_max", c_int32),
        ("keep_mask", c_void_p),
    ]


class TotalParams(Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4),
        ("lse", c_void_p), ("tot", c_void_p), ("workspace", c_void_p),
        ("B", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("M", c_int32), ("N", c_int32), ("D", c_int32),
        ("dtype", c_int32), ("causal", c_int32), ("sm_scale", c_float),
        ("status", c_void_p),
    ]


class BwdParams(Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("d_o", Tensor4),
        ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("lse", c_void_p), ("delta", c_void_p), ("workspace", c_void_p),
        ("B", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("M", c_int32), ("N", c_int32), ("D", c_int32),
        ("dtype", c_int32), ("o_dtype", c_int32), ("causal", c_int32),
        ("sm_scale", c_float), ("dropout_p", c_float),
        ("seed", c_uint64), ("offset", c_uint64),
        ("status", c_void_p),
        ("band", c_int32), ("dist_min", c_int32), ("dist_max", c_int32),
        ("keep_mask", c_void_p),
        ("dv_accumulate", c_int32),
    ]


class SplitKVParams(Structure):
    _fields_ = [
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("lse", c_void_p), ("part_o", c_void_p), ("part_lse", c_void_p),
        ("B", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("M", c_int32), ("N", c_int32), ("D", c_int32),
        ("num_splits", c_int32), ("dtype", c_int32), ("causal", c_int32), ("sm_scale", c_float),
        ("status", c_void_p),
    ]


class PagedParams(Structure):
    _fields_ = [
        ("q", Tensor4), ("key_cache", Tensor4), ("value_cache", Tensor4), ("o", Tensor4),
        ("block_table", c_void_p), ("block_table_stride", c_int64), ("context_lens", c_void_p),
        ("lse", c_void_p), ("part_o", c_void_p), ("part_lse", c_void_p),
        ("num_seqs", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("D", c_int32), ("block_size", c_int32),
        ("num_blocks", c_int32), ("max_context_len", c_int32), ("num_splits", c_int32),
        ("dtype", c_int32), ("sm_scale", c_float), ("status", c_void_p),
    ]


class SelftestParams(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("d", c_void_p),
        ("a_cols", c_int32), ("b_rows", c_int32), ("b_cols", c_int32),
        ("box_cols", c_int32), ("swizzle", c_int32), ("bf16", c_int32), ("a_in_tmem", c_int32),
        ("n", c_int32), ("k_steps", c_int32), ("idesc", c_uint32),
        ("a_desc_hi", c_uint64), ("b_desc_hi", c_uint64),
        ("a_step_bytes", c_int32), ("b_step_bytes", c_int32),
        ("a_chunk_steps", c_int32), ("b_chunk_steps", c_int32),
        ("a_chunk_bytes", c_int32), ("b_chunk_bytes", c_int32),
        ("status", c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/b200attn.h declares.
SYMBOLS = {
    "b200attn_fwd": (c_int32, [POINTER(FwdParams), c_void_p]),
    "b200attn_total_workspace_bytes": (c_size_t, [c_int32] * 3),
    "b200attn_total_attention": (c_int32, [POINTER(TotalParams), c_void_p]),
    "b200attn_total_attention_static": (c_int32, [POINTER(TotalParams), c_void_p]),
    "b200attn_bwd_workspace_bytes": (c_size_t, [c_int32] * 6),
    "b200attn_bwd": (c_int32, [POINTER(BwdParams), c_void_p]),
    "b200attn_bwd_stages": (c_int32, [POINTER(BwdParams), c_void_p, c_int32]),
    "b200attn_bwd_delta": (c_int32, [POINTER(Tensor4), c_int32, POINTER(Tensor4), c_int32, c_void_p,
                                     c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "b200attn_dropout_mask": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_float, c_uint64,
                                        c_uint64, c_void_p]),
    "b200attn_keep_mask_bytes": (c_size_t, [c_int32] * 4),
    "b200attn_fwd_splitkv": (c_int32, [POINTER(SplitKVParams), c_void_p]),
    "b200attn_splitkv_num_splits": (c_int32, [c_int32] * 7),
    "b200attn_paged_attention": (c_int32, [POINTER(PagedParams), c_void_p]),
    "b200attn_merge_partial": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                         c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "b200attn_merge_partial_store": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                               c_int32, POINTER(Tensor4), c_int32, c_void_p]),
    "b200attn_abi_version": (c_int32, []),
    "b200attn_last_error": (c_char_p, []),
    "b200attn_umma_selftest": (c_int32, [POINTER(SelftestParams), c_void_p]),
    "b200attn_wait_timeout_selftest": (c_int32, [c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "b200attn_work_order_selftest": (c_int32, [c_int32, c_int32, c_int32]),
}

_LIB = None


def lib_path() -> Path:
    env = os.environ.get("B200ATTN_LIB")
    if env:
        return Path(env)
    return Path(__file__).resolve().parent / "libb200attn.so"


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and sets the prototypes of every exported entry point."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m flagattention_b200.build` "
            "(there is no non-CUDA fallback)")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError here means the .so is stale
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.b200attn_abi_version() != 3:
        raise RuntimeError("libb200attn.so ABI version mismatch; rebuild the library")
    _LIB = lib
    return lib


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}") from None


_Stride4 = c_int64 * 4


def tensor4(t: torch.Tensor) -> Tensor4:
    s0, s1, s2, s3 = t.stride()  # raises unless t has four dimensions
    return Tensor4(t.data_ptr(), _Stride4(s0, s1, s2, s3))


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().b200attn_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed ({ERROR_NAMES.get(rc, rc)}): {msg}")


def current_stream_ptr(device: torch.device) -> int:
    """Raw ``cudaStream_t`` of torch's current stream on ``device``."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None and device.index is not None:
        return raw(device.index)
    return torch.cuda.current_stream(device).cuda_stream

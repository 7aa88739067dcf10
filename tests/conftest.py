import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"

# The unmodified reference, installed into the git-ignored baseline/_ref with
#   python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <writable copy of the reference checkout>
# (it is not product source). Only the same-GPU A/B tests import it; absent, they skip with a reason.
REFERENCE_INSTALL = ROOT / "baseline" / "_ref"
if (REFERENCE_INSTALL / "flag_attn").is_dir() and str(REFERENCE_INSTALL) not in sys.path:
    sys.path.append(str(REFERENCE_INSTALL))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session", autouse=True)
def _exact_fp32_matmul():
    # The fp32 oracle must not run on TF32 tensor cores (the reference's tests do the same,
    # tests/conftest.py:8-16).
    prev = torch.get_float32_matmul_precision()
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.set_float32_matmul_precision(prev)


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no kernel may have given up on a bounded device-side wait. (The kernels
    record a code in a per-device status word and leave instead of spinning; nothing else would
    notice, because the outputs of such a launch are simply incomplete.)"""
    yield
    if request.node.get_closest_marker("gpu") is not None and torch.cuda.is_available():
        from flagattention_b200 import status
        for idx in status.known_devices():
            status.check_device_status(torch.device("cuda", idx))


def _from_bits(arr: np.ndarray, dtype: str) -> torch.Tensor:
    if arr.dtype == np.uint16:
        t = torch.from_numpy(arr.view(np.int16).copy())
        return t.view(torch.float16 if dtype == "float16" else torch.bfloat16)
    return torch.from_numpy(arr.copy())


def load_golden(name: str) -> dict:
    """Loads a fixture written by tests/golden/make_golden.py; 16-bit arrays come back as torch
    tensors of the case's dtype, the dropout mask as a bool tensor (or None)."""
    z = np.load(GOLDEN / f"{name}.npz")
    meta = json.loads(str(z["meta"]))
    out = {"meta": meta}
    for key in z.files:
        if key in ("meta", "mask"):
            continue
        out[key] = _from_bits(z[key], meta["dtype"])
    if "mask" in z.files and z["mask"].size:
        B, H, M, N = meta["B"], meta["Hq"], meta["M"], meta["N"]
        out["mask"] = torch.from_numpy(np.unpackbits(z["mask"])[: B * H * M * N].reshape(B, H, M, N).astype(bool))
    else:
        out["mask"] = None
    return out


ATTENTION_GOLDENS = ["attention_c1_plumbing", "attention_gqa_causal_bf16", "attention_mqa_ragged_fp16",
                     "attention_larger_m_causal", "attention_dropout_fp16", "attention_dropout_bf16_gqa"]
TRITON_GOLDENS = ["triton_interp_causal0_p0", "triton_interp_causal0_p3", "triton_interp_causal1_p0",
                  "triton_interp_causal1_p3"]


PAGED_GOLDENS = ["paged_mha_fp16", "paged_gqa8_fp16", "paged_gqa4_bf16"]


def load_paged_golden(name: str) -> dict:
    """A paged-attention fixture of tests/golden/make_golden.py: q, key_cache, value_cache and out as
    torch tensors of the case's dtype, block_tables / context_lens as int32 tensors, out_fp32, scale."""
    z = np.load(GOLDEN / f"{name}.npz")
    dtype = "bfloat16" if "bfloat16" in str(z["dtype"]) else "float16"
    out = {k: _from_bits(z[k], dtype) for k in ("q", "key_cache", "value_cache", "out")}
    out["block_tables"] = torch.from_numpy(z["block_tables"].copy())
    out["context_lens"] = torch.from_numpy(z["context_lens"].copy())
    out["out_fp32"] = torch.from_numpy(z["out_fp32"].copy())
    out["scale"] = float(z["scale"])
    return out

PIECEWISE_GOLDENS = ["piecewise_causal_fp16", "piecewise_full_bf16", "piecewise_causal_larger_m"]

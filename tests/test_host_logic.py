"""CPU-only checks of the host side: library loading, exported symbols, argument validation,
the split-KV dispatch rule and the wrapper's contract errors. No kernel is launched."""
import ctypes
import json
import re

import pytest
import torch

from conftest import GOLDEN, ROOT
from flagattention_b200 import _lib, flash_attention
from flagattention_b200.split_kv import choose_num_splits


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "b200attn.h").read_text()
    declared = set(re.findall(r"\b(b200attn_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree"
    lib = ctypes.CDLL(str(_lib.lib_path()))
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().b200attn_abi_version() == 3


def test_invalid_arguments_are_rejected_before_any_cuda_call():
    lib = _lib.load()
    assert lib.b200attn_fwd(None, None) == -1
    p = _lib.FwdParams()
    p.B, p.Hq, p.Hkv, p.M, p.N, p.D = 1, 4, 3, 16, 16, 64
    assert lib.b200attn_fwd(p, None) == -1
    assert b"multiple" in lib.b200attn_last_error()
    p.Hkv, p.D = 2, 48
    assert lib.b200attn_fwd(p, None) == -1
    assert b"head dimension" in lib.b200attn_last_error()
    assert lib.b200attn_dropout_mask(None, 1, 1, 1, 1, 0.5, 0, 0, None) == -1
    assert lib.b200attn_bwd(None, None) == -1
    assert lib.b200attn_total_attention(None, None) == -1
    assert lib.b200attn_fwd_splitkv(None, None) == -1


def test_split_rule_matches_reference_table():
    rows = json.loads((GOLDEN / "split_heuristic.json").read_text())
    for B, H, M, N, sms, want in rows:
        assert choose_num_splits(B, H, M, N, sms) == want, (B, H, M, N, sms)


def test_baseline_configs_do_not_split():
    for (B, H, M, N) in [(1, 4, 128, 128), (4, 32, 4096, 4096), (16, 16, 2048, 2048), (8, 16, 512, 8192),
                         (1, 64, 32768, 32768)]:
        assert choose_num_splits(B, H, M, N, 148) == 1


def test_contract_violations_raise_like_the_reference():
    q = torch.zeros(1, 4, 8, 64, dtype=torch.float16)
    with pytest.raises(AssertionError, match="feature size"):
        flash_attention(q, torch.zeros(1, 4, 8, 32, dtype=torch.float16), q)
    with pytest.raises(AssertionError):
        flash_attention(torch.zeros(1, 4, 8, 48), torch.zeros(1, 4, 8, 48), torch.zeros(1, 4, 8, 48))
    with pytest.raises(AssertionError, match="k and v"):
        flash_attention(q, torch.zeros(1, 2, 8, 64, dtype=torch.float16), q)
    with pytest.raises(AssertionError, match="multiple"):
        k = torch.zeros(1, 3, 8, 64, dtype=torch.float16)
        flash_attention(q, k, k)
    with pytest.raises(RuntimeError, match="CUDA"):
        flash_attention(q, q, q)  # CPU tensors: there is no CPU path


def test_bench_flash_record_rows_have_the_reference_recorder_keys(tmp_path, monkeypatch):
    """The sweep's log line carries the row keys of the reference's recorder
    (benchmark/recording.py:36-54) and its FLOP formula (benchmark/flash_benchmark.py:120-128)."""
    import json

    from flagattention_b200 import bench_flash

    assert bench_flash.ROW_KEYS == (
        "case_id", "candidate_source", "legacy_shape", "shape_detail", "latency_base", "latency", "gbps_base",
        "gbps", "speedup", "accuracy", "tflops", "utilization", "compared_speedup", "base_miss_reason", "error_msg")
    # batch 32768 // 4096 = 8, heads 2048 // 128 = 16
    assert bench_flash.flops(4096, 128, False, "fwd") == 4.0 * 8 * 16 * 4096 * 4096 * 128
    assert bench_flash.flops(4096, 128, True, "bwd") == 4.0 * 8 * 16 * 4096 * 4096 * 128 * 2.5 * 0.5
    log = tmp_path / "sub" / "bench.log"
    monkeypatch.setenv(bench_flash.LOG_PATH_ENV, str(log))
    bench_flash.emit({"level": "comprehensive", "op_name": "flash_attention", "dtype": "torch.bfloat16",
                      "mode": "kernel", "result": [dict.fromkeys(bench_flash.ROW_KEYS)]})
    line = log.read_text().strip()
    assert line.startswith("[INFO] ")
    detail = json.loads(line[len("[INFO] "):])
    assert detail["op_name"] == "flash_attention" and set(detail["result"][0]) == set(bench_flash.ROW_KEYS)


def test_tuned_split_count_is_admissible_for_every_kernel_choice():
    """b200attn_splitkv_num_splits is host arithmetic (the SM count is passed in): at least one split,
    no CTA without keys, two partials per CTA for head-packed tiles, one split when the plain grid
    already fills the device."""
    lib = _lib.load()
    for B in (1, 2, 8, 64):
        for Hkv, groups in ((1, 1), (4, 1), (8, 2), (2, 8), (1, 32), (1, 256)):
            for M in (1, 2, 5, 300):
                for N in (1, 100, 4096, 70000, 2 ** 19):
                    s = lib.b200attn_splitkv_num_splits(B, Hkv * groups, Hkv, M, N, 128, 148)
                    tiles = -(-N // 128)
                    rows = groups * M
                    assert s >= 1
                    packed = groups > 1 and 2 < rows <= 128
                    ctas = s // 2 if packed and s % 2 == 0 else s
                    assert 1 <= ctas <= max(1, tiles), (B, Hkv, groups, M, N, s)
                    per = -(-tiles // ctas)
                    assert per * (ctas - 1) < tiles, (B, Hkv, groups, M, N, s)
                    if rows > 128 and B * Hkv * groups * -(-M // 256) >= 0.8 * 148:
                        assert s == 1


def test_prepared_work_item_decode_matches_plain_division():
    """The kernels turn a work-item number into (batch, head) pair and row block with divisions
    prepared on the host (one high multiply and a shift each); the library checks them against plain
    integer division over whole grids, including ragged last chunks and power-of-two sizes."""
    lib = _lib.load()
    for pairs, n_z, chunk in [(128, 16, 192), (128, 16, 128), (1024, 2, 48), (37, 5, 7), (1, 1, 1), (64, 128, 48),
                              (4096, 4, 1), (3, 1000, 2), (255, 17, 256), (2048, 16, 4096)]:
        assert lib.b200attn_work_order_selftest(pairs, n_z, chunk) == 0, (pairs, n_z, chunk)
    assert lib.b200attn_work_order_selftest(0, 1, 1) < 0


def test_tile_config_hooks_exist_and_may_be_assigned():
    """The reference documents `flash.get_fwd_config` / `get_bwd_config` as replaceable at run time
    (`flash.py:309-342`, `:512-539`; `examples/use_cutom_config_func.py:18-23` assigns one). Here they
    report the compiled tile shapes; assigning a replacement must be accepted (and changes nothing)."""
    from flagattention_b200 import flash
    fwd = flash.get_fwd_config(2, 16, 4096, 4096, 128, True)
    bwd = flash.get_bwd_config(2, 16, 4096, 4096, 128, True)
    assert len(fwd) == 4 and len(bwd) == 4 and all(isinstance(x, int) for x in fwd + bwd)
    saved = flash.get_fwd_config, flash.get_bwd_config
    try:
        def get_fwd_config(B, H, M, N, D, causal):
            return (64, 64, 1, 4)
        flash.get_fwd_config = get_fwd_config          # what the reference's example does
        flash.get_bwd_config = lambda *a: (64, 64, 1, 4)
        assert flash.get_fwd_config(2, 16, 4096, 4096, 128, True) == (64, 64, 1, 4)
    finally:
        flash.get_fwd_config, flash.get_bwd_config = saved


def test_wait_timeout_selftest_validates_its_arguments():
    lib = _lib.load()
    assert lib.b200attn_wait_timeout_selftest(100, 1, None, None, None) == -1
    assert b"null" in lib.b200attn_last_error()

"""Flash-decoding benchmark: one query token against a long key/value cache.

Shapes follow the reference's ``benchmark/flash_decoding_benchmark.py`` (batch 2, 2048 / D heads,
one query row, fp16, non-causal, D in {64, 128}, N = 2^9 .. 2^19) plus grouped-head decode shapes
and paged-cache decode (the shapes of ``benchmark/paged_benchmark.py``).
The operation is a pure stream over K and V, so the figure of merit is the rate at which the K/V
bytes are consumed, compared with the measured HBM copy bandwidth of the device.

    python -m flagattention_b200.bench_decoding [--json] [--with-torch] [--graph]

Every timed loop rotates over enough independent K/V copies that the working set exceeds the L2
cache (126 MB), so the rate is an HBM rate at every N. Timing is by CUDA events on the launching
stream around ``iters`` back-to-back calls of the public operator, after warm-up. At short contexts
a call costs more on the host (about 30 us) than on the device; ``--graph`` captures the same calls
into a CUDA graph and times its replay, which is what a serving loop that replays graphs would see.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import torch

from . import _lib, check_device_status, flash_attention_split_kv, paged_attention

L2_BYTES = 126 * 2 ** 20
FALLBACK_HBM_GBS = 6650.0


def _hbm_peak():
    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        peaks = json.loads(path.read_text())
        for key in ("hbm_gbs", "hbm_gb_s", "hbm"):
            if key in peaks:
                return float(peaks[key]), "measured"
    except (OSError, ValueError):
        pass
    return FALLBACK_HBM_GBS, "fallback"


def _time_ms(fn, iters, warmup=5):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(iters):
        fn(i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _torch_attention(q, k, v):
    groups = q.shape[1] // k.shape[1]
    if groups > 1:
        k, v = k.repeat_interleave(groups, 1), v.repeat_interleave(groups, 1)
    p = torch.softmax((q @ k.transpose(2, 3)).float() / math.sqrt(q.shape[-1]), -1)
    return p.to(v.dtype) @ v


def _graph_ms(call, copies, iters):
    """Device time per call when `copies` calls (one per K/V copy) are replayed from a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(copies):
                call(i)
    torch.cuda.current_stream().wait_stream(side)
    replays = max(1, iters // copies)
    return _time_ms(lambda i: graph.replay(), replays, warmup=2) / copies


def run_case(B, Hq, Hk, M, N, D, dtype, iters, with_torch, device, graph=False):
    kv_bytes = 2 * B * Hk * N * D * 2
    copies = max(1, min(16, -(-2 * L2_BYTES // kv_bytes)))
    qs = [torch.randn(B, Hq, M, D, device=device, dtype=dtype) for _ in range(copies)]
    ks = [torch.randn(B, Hk, N, D, device=device, dtype=dtype) for _ in range(copies)]
    vs = [torch.randn(B, Hk, N, D, device=device, dtype=dtype) for _ in range(copies)]
    call = lambda i: flash_attention_split_kv(qs[i % copies], ks[i % copies], vs[i % copies])  # noqa: E731
    ms = _graph_ms(call, copies, iters) if graph else _time_ms(call, iters)
    row = {
        "B": B, "Hq": Hq, "Hkv": Hk, "M": M, "N": N, "D": D, "dtype": str(dtype)[6:],
        "splits": int(_lib.load().b200attn_splitkv_num_splits(B, Hq, Hk, M, N, D, 0)),
        "kv_copies_rotated": copies, "us": round(ms * 1e3, 2), "kv_gbs": round(kv_bytes / ms / 1e6, 1),
        "timed": "cuda graph replay" if graph else "eager calls",
    }
    if with_torch:
        t_ms = _time_ms(lambda i: _torch_attention(qs[i % copies], ks[i % copies], vs[i % copies]),
                        max(3, iters // 4), warmup=2)
        row["torch_us"] = round(t_ms * 1e3, 2)
    return row


def run_paged_case(num_seqs, Hq, group, D, block, context_len, dtype, iters, device):
    """Shapes of the reference's ``benchmark/paged_benchmark.py`` (64 query heads, equal context
    lengths, random block table), but with one distinct cache block per table entry so that the K/V
    working set is what it would be in a real cache (and larger than L2) instead of 1000 shared blocks."""
    Hkv = Hq // group
    per_seq = -(-context_len // block)
    num_blocks = num_seqs * per_seq
    scale = D ** -0.5
    q = torch.empty(num_seqs, Hq, D, dtype=dtype, device=device).uniform_(-scale, scale)
    k_cache = torch.empty(num_blocks, Hkv, block, D, dtype=dtype, device=device).uniform_(-scale, scale)
    v_cache = torch.empty_like(k_cache).uniform_(-scale, scale)
    tables = torch.randperm(num_blocks, device=device).to(torch.int32).view(num_seqs, per_seq)
    lens = torch.full((num_seqs,), context_len, dtype=torch.int32, device=device)
    ms = _time_ms(lambda i: paged_attention(q, k_cache, v_cache, lens, tables, scale, context_len), iters)
    kv_bytes = 2 * num_seqs * Hkv * context_len * D * 2
    return {"num_seqs": num_seqs, "Hq": Hq, "Hkv": Hkv, "D": D, "block_size": block, "context_len": context_len,
            "dtype": str(dtype)[6:], "us": round(ms * 1e3, 2), "kv_gbs": round(kv_bytes / ms / 1e6, 1),
            "splits": int(_lib.load().b200attn_splitkv_num_splits(num_seqs, Hq, Hkv, 1, context_len, D, 0))}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--json", action="store_true", help="one JSON object per line instead of a table")
    ap.add_argument("--with-torch", action="store_true", help="also time the plain PyTorch formula")
    ap.add_argument("--graph", action="store_true",
                    help="time the one-token and grouped-head cases as CUDA graph replays (no host cost per call)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--min-log2-n", type=int, default=9)
    ap.add_argument("--max-log2-n", type=int, default=19)
    ap.add_argument("--head-dim", type=int, default=0, help="restrict the one-token sweep to this D")
    ap.add_argument("--case", default="", help="run only cases whose tag starts with this (profiling runs)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_decoding needs a CUDA device")
    device = torch.device("cuda", 0)
    peak, peak_kind = _hbm_peak()
    cases = []
    for D in (64, 128):
        if args.head_dim and D != args.head_dim:
            continue
        for log2n in range(args.min_log2_n, args.max_log2_n + 1):
            cases.append(("mha", 2, 2048 // D, 2048 // D, 1, 2 ** log2n, D, torch.float16))
    for groups in (2, 4, 8, 16):
        cases.append((f"gqa{groups}", 8, 32, 32 // groups, 1, 32768, 128, torch.bfloat16))
    cases.append(("gqa8", 8, 32, 4, 1, 32768, 64, torch.bfloat16))
    cases.append(("gqa4-4tok", 4, 32, 8, 4, 32768, 128, torch.bfloat16))
    for tag, B, Hq, Hk, M, N, D, dtype in cases:
        if args.case and not tag.startswith(args.case):
            continue
        row = run_case(B, Hq, Hk, M, N, D, dtype, args.iters, args.with_torch, device, args.graph)
        row.update(case=tag, hbm_peak_gbs=peak, hbm_peak_kind=peak_kind, frac=round(row["kv_gbs"] / peak, 3))
        if args.json:
            print(json.dumps(row), flush=True)
        else:
            extra = f"  torch {row['torch_us']:9.1f} us" if args.with_torch else ""
            print(f"{tag:10s} B{B} Hq{Hq} Hkv{Hk} M{M} N{N:7d} D{D:3d} splits {row['splits']:3d}: "
                  f"{row['us']:9.1f} us  {row['kv_gbs']:7.0f} GB/s  {row['frac']:.2f} of {peak_kind} HBM peak"
                  f"{extra}", flush=True)
    for group in (1, 8):
        for block in (16, 128):
            for context_len in (4096, 16384):
                tag = f"paged-g{group}"
                if args.case and not tag.startswith(args.case):
                    continue
                row = run_paged_case(32, 64, group, 128, block, context_len, torch.float16, args.iters, device)
                row.update(case=tag, hbm_peak_gbs=peak, hbm_peak_kind=peak_kind, frac=round(row["kv_gbs"] / peak, 3))
                if args.json:
                    print(json.dumps(row), flush=True)
                else:
                    print(f"{tag:10s} seqs32 Hq64 Hkv{row['Hkv']} ctx{context_len:6d} D128 block{block:4d} splits "
                          f"{row['splits']:3d}: {row['us']:9.1f} us  {row['kv_gbs']:7.0f} GB/s  {row['frac']:.2f} of "
                          f"{peak_kind} HBM peak", flush=True)
    check_device_status(device)


if __name__ == "__main__":
    main()

"""The reference's headline sweep (``benchmark/flash_benchmark.py``) run against this library, with
its result rows in the record format of the reference's recorder (``benchmark/recording.py``).

Shapes: batch ``32768 // N_CTX``, ``2048 // D`` heads, ``N_CTX`` = 2^9 .. 2^15, D in {64, 128},
causal and full, forward and backward, fp16 and bf16 (``flash_benchmark.py:49-73``). TFLOP/s by the
reference's own formula (``:120-128``): forward ``4 B H N^2 D``, backward x2.5, causal x0.5.

Each (dtype) group ends in one line ``[INFO] {json}`` with the keys the reference's recorder emits
(``recording.py:36-54,227-262``): ``level, op_name, dtype, mode, result`` and per row ``shape_detail,
latency, latency_base, speedup, tflops, utilization`` (latencies in ms; ``utilization`` = TFLOP/s over
the 2250 TFLOP/s dense bf16/fp16 peak of a B200), so a report built from the reference's logs shows
this implementation unchanged. When ``FLAG_ATTN_BENCHMARK_LOG_PATH`` is set the lines are appended to
that file instead of stdout, as the reference does.

    python -m flagattention_b200.bench_flash [--no-torch] [--max-log2-n 15] [--quick]

The baseline column is the plain PyTorch formula (the reference's ``torch`` provider); it is skipped
(``latency_base`` null) where its N x N score matrix would not fit comfortably.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch

from . import check_device_status, flash_attention, piecewise_attention

SPEC_PEAK_TFLOPS = 2250.0
LOG_PATH_ENV = "FLAG_ATTN_BENCHMARK_LOG_PATH"
ROW_KEYS = ("case_id", "candidate_source", "legacy_shape", "shape_detail", "latency_base", "latency",
            "gbps_base", "gbps", "speedup", "accuracy", "tflops", "utilization", "compared_speedup",
            "base_miss_reason", "error_msg")


def _time_ms(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _torch_attention(q, k, v, causal):
    s = (q @ k.transpose(2, 3)) * (1.0 / math.sqrt(q.shape[-1]))
    if causal:
        m, n = q.shape[2], k.shape[2]
        keep = torch.ones(m, n, dtype=torch.bool, device=q.device).tril(n - m)
        s = s.masked_fill(~keep, float("-inf"))
    return torch.softmax(s.float(), -1).to(v.dtype) @ v


def flops(n_ctx, head_dim, causal, mode):
    batch, heads = 32768 // n_ctx, 2048 // head_dim
    f = 4.0 * batch * heads * n_ctx * n_ctx * head_dim
    if mode == "bwd":
        f *= 2.5
    return f * (0.5 if causal else 1.0)


def _torch_piecewise(q1, k1, q2, k2, v, w, causal):
    m, n = q1.shape[2], k1.shape[2]
    dist = (torch.arange(m, device=q1.device).unsqueeze(-1) + (n - m)) - torch.arange(n, device=q1.device)
    s = torch.where(dist >= w, q2 @ k2.transpose(2, 3), q1 @ k1.transpose(2, 3)) * (1.0 / math.sqrt(q1.shape[-1]))
    if causal:
        s = s.masked_fill(dist < 0, float("-inf"))
    return torch.softmax(s.float(), -1).to(v.dtype) @ v


def measure(provider, n_ctx, head_dim, causal, mode, dtype, device, warmup, iters, op="flash_attention"):
    batch, heads = 32768 // n_ctx, 2048 // head_dim
    need_grad = mode == "bwd"
    n_inputs = 3 if op == "flash_attention" else 5
    leaves = tuple(torch.randn(batch, heads, n_ctx, head_dim, dtype=dtype, device=device, requires_grad=need_grad)
                   for _ in range(n_inputs))
    if op == "flash_attention":
        q, k, v = leaves
        fn = (lambda: flash_attention(q, k, v, causal=causal)) if provider == "ours" else \
             (lambda: _torch_attention(q, k, v, causal))
    else:
        # the reference's piecewise benchmark: threshold at half the sequence (piecewise_benchmark.py:65)
        q1, k1, q2, k2, v = leaves
        w = n_ctx // 2
        fn = (lambda: piecewise_attention(q1, k1, q2, k2, v, w, causal=causal)) if provider == "ours" else \
             (lambda: _torch_piecewise(q1, k1, q2, k2, v, w, causal))
    if need_grad:
        o = fn()
        do = torch.randn_like(o)
        fn = lambda: torch.autograd.grad(o, leaves, do, retain_graph=True)  # noqa: E731
    return _time_ms(fn, warmup, iters)


def emit(detail):
    line = f"[INFO] {json.dumps(detail, default=str)}"
    path = os.environ.get(LOG_PATH_ENV)
    if path:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with p.open("a", encoding="utf-8") as stream:
            stream.write(line + "\n")
    else:
        print(line, flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--no-torch", action="store_true", help="skip the plain PyTorch baseline column")
    ap.add_argument("--min-log2-n", type=int, default=9)
    ap.add_argument("--max-log2-n", type=int, default=15)
    ap.add_argument("--quick", action="store_true", help="D=128, bf16, causal only")
    ap.add_argument("--op", default="flash_attention", choices=["flash_attention", "piecewise_attention"],
                    help="piecewise_attention: the shapes of benchmark/piecewise_benchmark.py, same FLOP formula")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_flash needs a CUDA device")
    device = torch.device("cuda", 0)
    dtypes = [torch.bfloat16] if args.quick else [torch.float16, torch.bfloat16]
    dims = [128] if args.quick else [64, 128]
    causals = [True] if args.quick else [False, True]
    for dtype in dtypes:
        rows = []
        for mode in ("fwd", "bwd"):
            for causal in causals:
                for head_dim in dims:
                    for log2n in range(args.min_log2_n, args.max_log2_n + 1):
                        n_ctx = 2 ** log2n
                        ms = measure("ours", n_ctx, head_dim, causal, mode, dtype, device, args.warmup, args.iters,
                                     args.op)
                        base = None
                        # scores + probabilities of the plain formula: batch*heads*N^2*(2+4+2) bytes
                        per_score = 8 if args.op == "flash_attention" else 14  # piecewise keeps two score matrices
                        if not args.no_torch and (32768 // n_ctx) * (2048 // head_dim) * n_ctx * n_ctx * per_score <= 40e9:
                            try:
                                base = measure("torch", n_ctx, head_dim, causal, mode, dtype, device, 2,
                                               max(3, args.iters // 4), args.op)
                            except torch.OutOfMemoryError:
                                base = None
                                torch.cuda.empty_cache()
                        tf = flops(n_ctx, head_dim, causal, mode) / ms * 1e-9
                        row = dict.fromkeys(ROW_KEYS)
                        row.update(
                            shape_detail={"D_HEAD": head_dim, "dtype": str(dtype), "mode": mode, "causal": causal,
                                          "N_CTX": n_ctx},
                            latency=ms, latency_base=base, speedup=(base / ms if base else None),
                            tflops=tf, utilization=tf / SPEC_PEAK_TFLOPS)
                        rows.append(row)
                        print(f"{str(dtype)[6:]:8s} {mode} causal={int(causal)} D={head_dim:3d} N_CTX={n_ctx:6d}: "
                              f"{ms:8.3f} ms {tf:7.1f} TFLOP/s"
                              + (f"   torch {base:9.3f} ms  x{base / ms:6.1f}" if base else ""), flush=True)
        emit({"level": "comprehensive", "op_name": args.op, "dtype": str(dtype), "mode": "kernel",
              "result": rows, "baseline": None if args.no_torch else "torch"})
    check_device_status(device)


if __name__ == "__main__":
    main()

"""Benchmark of the flash_attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

One "step" is one forward + backward of the workload over a batch of synthetic, seeded inputs.
The default workload is the Llama-style GQA prefill training step the headline metric is quoted on:
B=4, Hq=32, Hkv=8, M=N=4096, D=128, bf16, causal, log-normaliser returned.

* ``value`` is aggregate algorithmic TFLOPS (reference convention: forward 4*B*Hq*M*N*D, backward
  2.5x that, causal x0.5) over all ranks with inputs resident in HBM; timing is CUDA events around
  exactly K steps, barrier + synchronize on both sides, max over ranks.
* ``e2e`` is the same metric with HOST (pinned) inputs and outputs: every step copies q, k, v, dO to
  the device and o, lse, dq, dk, dv back inside the timed region (copies of neighbouring steps
  overlap the compute on separate streams); it also reports the copy rates per direction.
* ``roofline`` describes the dominant kernel of the step, launched by itself through the C ABI:
  median of >= 20 launches, each between its own pair of CUDA events, over two rotating sets of
  buffers (every launch sees operands that the previous launch did not leave in L2). Because the
  kernel is timed in isolation, ``frac`` divides by the measured BURST bf16 GEMM peak; the fraction of
  the sustained peak and of the 2250 TFLOPS spec peak are printed beside it.
  ``traffic`` (DRAM bytes per launch) is read from the ncu summary under ``profiles/`` that the line
  names, scaled by batch; ``algorithmic_bytes`` are the compulsory bytes of the same launch.
* ``triton_reference`` times the unmodified reference's Triton ``flash_attention`` (installed under
  ``baseline/_ref``) on the same GPU, same inputs: once with the tile configuration the reference
  picks for this GPU and once with its hook overridden by the reference's own sm_80 table entries.
* ``cpu_baseline`` times the CPU oracle (the reference's PyTorch attention restated) on a bounded
  sample of the same workload on this host's cores.
* ``--impl reference`` runs only that CPU path (all host threads) and prints its own line.

N > 1: launched under torchrun, one rank per GPU; every rank runs the full per-GPU workload
(independent (batch x KV-head-group) units, no collective on the data path), so scaling is weak.
After that the ranks also run the 32k-token forward configuration split two ways -- by KV-head groups
(no collective) and as ring-KV sequence parallelism over NCCL -- and report both in ``c5_heads`` and
``c5_ring`` together with rank 0's single-GPU time of the same configuration taken in the same run.
"""
from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import re
import shutil
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    # name: B, Hq, Hkv, M, N, D, dtype, causal, dropout_p, mode
    "c2_gqa_prefill_train": dict(B=4, Hq=32, Hkv=8, M=4096, N=4096, D=128, dtype="bfloat16", causal=True,
                                 dropout_p=0.0, mode="fwd+bwd"),
    "c3_d64_dropout_aux": dict(B=16, Hq=16, Hkv=16, M=2048, N=2048, D=64, dtype="float16", causal=False,
                               dropout_p=0.1, mode="fwd+bwd"),
    "c4_mqa_cross_fwd": dict(B=8, Hq=16, Hkv=1, M=512, N=8192, D=128, dtype="bfloat16", causal=False,
                             dropout_p=0.0, mode="fwd"),
    "c5_long_context_fwd": dict(B=1, Hq=64, Hkv=8, M=32768, N=32768, D=128, dtype="bfloat16", causal=True,
                                dropout_p=0.0, mode="fwd"),
}
DEFAULT_CONFIG = "c2_gqa_prefill_train"
SPEC_PEAK_TFLOPS = 2250.0

FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def fwd_flops(cfg) -> float:
    f = 4.0 * cfg["B"] * cfg["Hq"] * cfg["M"] * cfg["N"] * cfg["D"]
    return f * 0.5 if cfg["causal"] else f


def step_flops(cfg) -> float:
    return fwd_flops(cfg) * (3.5 if cfg["mode"] == "fwd+bwd" else 1.0)


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def ncu_traffic(workload: str, kernel: str, batch: int):
    """DRAM bytes per launch of `kernel` on `workload`, from the ncu summaries under profiles/: lines

        bench-traffic: workload=<w> kernel=<k> batch=<b> dram_read_bytes=<r> dram_write_bytes=<w>

    (one capture each, at a batch small enough to capture; traffic is proportional to batch).
    Returns (bytes scaled to `batch`, file name) or (None, None)."""
    pat = re.compile(r"bench-traffic:\s+workload=(\S+)\s+kernel=(\S+)\s+batch=(\d+)\s+dram_read_bytes=(\d+)\s+"
                     r"dram_write_bytes=(\d+)")
    for path in sorted((ROOT / "profiles").glob("*.md")):
        for m in pat.finditer(path.read_text()):
            if m.group(1) == workload and m.group(2) == kernel:
                per = (int(m.group(4)) + int(m.group(5))) / int(m.group(3))
                return per * batch, f"profiles/{path.name}"
    return None, None


# ------------------------------------------------------------------ clocks sampling
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU every 50 ms; ``stop(t0, t1)`` keeps the
    samples whose time stamp lies inside the timed region [t0, t1] (``datetime`` values of this host)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,timestamp")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.tmp = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = subprocess.Popen(
            [exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
             str(self.gpu_index)], stdout=self.tmp, stderr=subprocess.DEVNULL)

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = []
        for line in Path(self.tmp.name).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                rows.append(parts)
        os.unlink(self.tmp.name)
        if not rows:
            return None
        n_all = len(rows)
        if t0 is not None and t1 is not None:
            def stamp(r):
                try:
                    return datetime.datetime.strptime(r[7], "%Y/%m/%d %H:%M:%S.%f")
                except (ValueError, IndexError):
                    return None
            inside = [r for r in rows if (ts := stamp(r)) is not None and t0 <= ts <= t1]
            if not inside:      # a region shorter than the sampling period: the samples next to it
                near = [r for r in rows if (ts := stamp(r)) is not None
                        and t0 - datetime.timedelta(milliseconds=60) <= ts <= t1 + datetime.timedelta(milliseconds=60)]
                inside = near
            if inside:
                rows = inside
        sm = []
        for r in rows:
            try:
                sm.append(float(r[0]))
            except ValueError:
                pass
        reasons = []
        for idx, name in ((3, "hw_slowdown"), (4, "hw_thermal_slowdown"), (5, "sw_thermal_slowdown"),
                          (6, "sw_power_cap")):
            if any(r[idx].lower().startswith("active") for r in rows):
                reasons.append(name)
        try:
            sm_max = float(rows[0][1])
        except ValueError:
            sm_max = None
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "sm_max_mhz": sm_max, "reasons": reasons, "samples": len(rows), "samples_taken": n_all,
                "note": "samples stamped inside the timed region; the driver's clock reading lags the load by "
                        "about 0.1 s"}


# ------------------------------------------------------------------ workload
def make_inputs(cfg, device, seed):
    dtype = getattr(torch, cfg["dtype"])
    g = torch.Generator(device=device).manual_seed(seed)
    B, Hq, Hkv, M, N, D = (cfg[k] for k in ("B", "Hq", "Hkv", "M", "N", "D"))
    q = torch.randn(B, Hq, M, D, device=device, dtype=dtype, generator=g)
    k = torch.randn(B, Hkv, N, D, device=device, dtype=dtype, generator=g)
    v = torch.randn(B, Hkv, N, D, device=device, dtype=dtype, generator=g)
    do = torch.randn(B, Hq, M, D, device=device, dtype=dtype, generator=g)
    return q, k, v, do


def run_step(cfg, q, k, v, do):
    """One pass of the hot path through the public API; returns every tensor the step produces."""
    from flagattention_b200 import flash_attention
    if cfg["mode"] == "fwd":
        o = flash_attention(q, k, v, causal=cfg["causal"], dropout_p=cfg["dropout_p"])
        return (o,)
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    o, lse, _, _, _ = flash_attention(q, k, v, causal=cfg["causal"], dropout_p=cfg["dropout_p"],
                                      return_log_normalizer=True)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    return o, lse, dq, dk, dv


def kernels_per_step(cfg) -> int:
    # forward: 1 kernel; backward: delta, statistics, then either the dK/dV kernel and the dQ kernel
    # or (D = 128 and 64) the fused dK/dV/dQ kernel and the dQ conversion.
    return 1 + (4 if cfg["mode"] == "fwd+bwd" else 0)


def time_kernels(cfg, inputs, iters=20, n_sets=2):
    """Times the library's kernels one by one through the C ABI: every launch between its own pair of
    CUDA events on the launching stream, `iters` launches per kernel rotating over `n_sets` sets of
    buffers, median. Returns ({name: ms}, {name: algorithmic bytes per launch})."""
    from flagattention_b200 import _lib
    lib = _lib.load()
    q0, k0, v0, do0 = inputs
    dev = q0.device
    B, Hq, Hkv, M, N, D = (cfg[x] for x in ("B", "Hq", "Hkv", "M", "N", "D"))
    dt = _lib.dtype_code(q0.dtype)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sm_scale = 1.0 / math.sqrt(D)
    bwd = cfg["mode"] == "fwd+bwd"
    fused = D in (64, 128)
    sets = []
    for s in range(n_sets):
        q, k, v, do = (q0, k0, v0, do0) if s == 0 else (t.clone() for t in (q0, k0, v0, do0))
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, M, dtype=torch.float32, device=dev)
        # dropout: the forward caches its keep decisions for the backward, as flash_attention does
        keep_mask = None
        if cfg["dropout_p"] > 0 and bwd:
            keep_mask = torch.empty(lib.b200attn_keep_mask_bytes(B, Hq, M, N) // 4, dtype=torch.int32, device=dev)
        mask_ptr = keep_mask.data_ptr() if keep_mask is not None else None
        fp = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(),
                            B, Hq, Hkv, M, N, D, dt, dt, int(cfg["causal"]), sm_scale, float(cfg["dropout_p"]),
                            12345, 0, status.data_ptr(), 0, 0, 0, mask_ptr)
        entry = {"fwd": fp, "keep": (q, k, v, do, o, lse, keep_mask)}
        if bwd:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            delta = torch.empty_like(lse)
            ws = torch.empty(lib.b200attn_bwd_workspace_bytes(B, Hq, Hkv, M, N, D) // 4, dtype=torch.float32,
                             device=dev)
            entry["bwd"] = _lib.BwdParams(
                _lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), _lib.tensor4(do),
                _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv), lse.data_ptr(), delta.data_ptr(),
                ws.data_ptr(), B, Hq, Hkv, M, N, D, dt, dt, int(cfg["causal"]), sm_scale,
                float(cfg["dropout_p"]), 12345, 0, status.data_ptr(), 0, 0, 0, mask_ptr)
            entry["keep"] += (dq, dk, dv, delta, ws)
        sets.append(entry)

    def timed(launch, before=None):
        for e in sets:
            if before:
                before(e)
            launch(e)                                   # warm-up on every set
        torch.cuda.synchronize(dev)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for i, (e0, e1) in enumerate(evs):
            if before:
                before(sets[i % n_sets])                # (outside the event pair)
            e0.record()
            launch(sets[i % n_sets])
            e1.record()
        torch.cuda.synchronize(dev)
        return statistics.median(e0.elapsed_time(e1) for e0, e1 in evs)

    out = {"fwd_kernel": timed(lambda e: _lib.check(lib.b200attn_fwd(e["fwd"], stream), "fwd"))}
    if bwd:
        # D = 128 and 64: one fused pass makes dK, dV and dQ, followed by the conversion of its fp32 dQ
        # accumulator; the accumulator is cleared by the preprocess in the real step and, here, before each
        # timed launch of the fused pass (outside its event pair). Other head dimensions run two separate kernels.
        if fused:
            n_stats = B * Hq * ((M + 127) // 128 * 128) * 2
            out["bwd_prep_kernels"] = timed(lambda e: _lib.check(lib.b200attn_bwd_stages(e["bwd"], stream, 1), "prep"))
            out["bwd_kernel<kv+dq>"] = timed(
                lambda e: _lib.check(lib.b200attn_bwd_stages(e["bwd"], stream, 2 | _lib.BWD_STAGE_ACC_ZEROED), "kv+dq"),
                before=lambda e: e["keep"][-1][n_stats:n_stats + B * Hq * M * D].zero_())
            out["dq_convert_kernel"] = timed(lambda e: _lib.check(lib.b200attn_bwd_stages(e["bwd"], stream, 4), "convert"))
        else:
            for name, mask in (("bwd_prep_kernels", 1), ("bwd_kernel<kv>", 2), ("bwd_kernel<q>", 4)):
                out[name] = timed(lambda e, m=mask: _lib.check(lib.b200attn_bwd_stages(e["bwd"], stream, m), name))
    torch.cuda.synchronize(dev)
    assert status.item() == 0, "a kernel reported a device-side wait timeout"
    # Compulsory bytes per launch (16-bit operands; fp32 statistics): what an ideal kernel moves.
    es = 2
    qb, kb = B * Hq * M * D * es, B * Hkv * N * D * es
    row_stats = B * Hq * M * 4
    alg_bytes = {"fwd_kernel": 2 * qb + 2 * kb + row_stats}
    if bwd:
        alg_bytes["bwd_kernel<kv+dq>"] = 2 * qb + 2 * kb + 2 * kb + qb + 2 * row_stats  # q,dO | k,v | dk,dv | dq
        alg_bytes["bwd_kernel<kv>"] = 2 * qb + 2 * kb + 2 * kb + 2 * row_stats
        alg_bytes["bwd_kernel<q>"] = 2 * qb + 2 * kb + qb + 2 * row_stats
    return out, alg_bytes


# ------------------------------------------------------------------ the reference's Triton kernel
def triton_reference(cfg, q, k, v, do, iters=10):
    """Times the unmodified reference (`flag_attn.flash_attention`, Triton) on the same GPU and inputs,
    as its own benchmark does (`benchmark/flash_benchmark.py:74-83`: forward, then
    `o.backward(do, retain_graph=True)`)."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "flag_attn").is_dir():
        return {"unavailable": "baseline/_ref is not installed (python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <writable copy of the reference checkout>)"}
    if str(ref_dir) not in sys.path:
        sys.path.append(str(ref_dir))
    try:
        import flag_attn
        from flag_attn import flash as ref_flash
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"import failed: {exc!r}"[:300]}
    dev = q.device
    bwd = cfg["mode"] == "fwd+bwd"
    f_fwd = fwd_flops(cfg)

    def median_ms(fn, n):
        fn()
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(n):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(dev)
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    def measure():
        qg, kg, vg = (t.detach().requires_grad_(bwd) for t in (q, k, v))
        call = lambda: flag_attn.flash_attention(qg, kg, vg, causal=cfg["causal"], dropout_p=cfg["dropout_p"])  # noqa: E731
        rec = {"fwd_ms": median_ms(call, iters)}
        rec["fwd_tflops"] = f_fwd / rec["fwd_ms"] * 1e-9
        total = rec["fwd_ms"]
        if bwd:
            o = call()
            rec["bwd_ms"] = median_ms(lambda: o.backward(do, retain_graph=True), max(3, iters // 2))
            rec["bwd_tflops"] = 2.5 * f_fwd / rec["bwd_ms"] * 1e-9
            total += rec["bwd_ms"]
        rec["ms_per_step"] = total
        rec["tflops"] = step_flops(cfg) / total * 1e-9
        return rec

    B, H, M, N, D, causal = cfg["B"], cfg["Hq"], cfg["M"], cfg["N"], cfg["D"], cfg["causal"]
    out = {"source": "baseline/_ref (pip install --no-deps --target of the unmodified reference)"}
    saved = ref_flash.get_fwd_config, ref_flash.get_bwd_config
    try:
        out["default_config"] = {"fwd": list(saved[0](B, H, M, N, D, causal)),
                                 "bwd": list(saved[1](B, H, M, N, D, causal))}
        try:
            out["default"] = measure()
            out.update({k_: out["default"][k_] for k_ in ("ms_per_step", "tflops")})
        except Exception as exc:  # noqa: BLE001
            out["default"] = {"error": repr(exc)[:300]}
        # The reference documents its hook as replaceable (examples/use_cutom_config_func.py:18-23);
        # the replacement used here is the reference's own table for compute capability 8.0
        # (flash.py:312-326, :515-525).
        if causal:
            f_cfg = (128, 64, 4, 4) if D <= 64 else ((128, 32, 2, 4) if M <= 1024 else (128, 128, 3, 8))
            b_cfg = (64, 64, 3 if D <= 64 else 2, 4)
        else:
            f_cfg = (128, 64, 3, 4) if D <= 64 else ((128, 32, 3, 4) if M <= 1024 else (128, 128, 3, 8))
            b_cfg = (128 if D <= 64 else 64, 64, 2, 4)
        ref_flash.get_fwd_config = lambda *a, **kw: f_cfg
        ref_flash.get_bwd_config = lambda *a, **kw: b_cfg
        out["overridden_config"] = {"fwd": list(f_cfg), "bwd": list(b_cfg),
                                    "note": "the reference's own sm_80 table, set through its config hook"}
        try:
            out["overridden"] = measure()
        except Exception as exc:  # noqa: BLE001
            out["overridden"] = {"error": repr(exc)[:300]}
    finally:
        ref_flash.get_fwd_config, ref_flash.get_bwd_config = saved
    return out


# ------------------------------------------------------------------ CPU baseline (oracle)
def cpu_slice_inputs(cfg, seed=0):
    """One (batch, KV-head-group) unit of the workload as CPU tensors."""
    dtype = getattr(torch, cfg["dtype"])
    g = torch.Generator().manual_seed(seed)
    G = cfg["Hq"] // cfg["Hkv"]
    q = torch.randn(1, G, cfg["M"], cfg["D"], generator=g).to(dtype)
    k = torch.randn(1, 1, cfg["N"], cfg["D"], generator=g).to(dtype)
    v = torch.randn(1, 1, cfg["N"], cfg["D"], generator=g).to(dtype)
    do = torch.randn(1, G, cfg["M"], cfg["D"], generator=g).to(dtype)
    return q, k, v, do


def cpu_slice_step(cfg, q, k, v, do):
    from oracle.attention import attention_forward
    if cfg["mode"] == "fwd":
        attention_forward(q, k, v, cfg["causal"], upcast=False)
        return
    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    o = attention_forward(q, k, v, cfg["causal"], upcast=False)
    torch.autograd.grad(o, (q, k, v), do)


def slice_flops(cfg) -> float:
    return step_flops(cfg) / (cfg["B"] * cfg["Hkv"])


def use_all_host_threads() -> int:
    """The CPU legs run on every host core this process may use. (torchrun exports OMP_NUM_THREADS=1
    to its workers, which would otherwise leave the reference arm of a multi-GPU launch on one core.)"""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    if torch.get_num_threads() != n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_baseline(cfg, budget_s=12.0, max_passes=64):
    """Times the oracle (native-dtype path, i.e. the reference's PyTorch CPU attention) on one whole
    (batch, KV-group) unit of the workload, repeated until `budget_s` seconds or `max_passes` passes
    (all units of the workload cost the same, so the rate of one is the rate of all)."""
    threads = use_all_host_threads()
    q, k, v, do = cpu_slice_inputs(cfg)
    # long-context units do not fit the budget: shrink the query rows of the sample and say so
    rows = cfg["M"]
    note = ""
    if cfg["M"] * cfg["N"] > 4096 * 4096 * 4:
        rows = max(128, (4096 * 4096 * 4) // cfg["N"])
        q, do = q[:, :, -rows:], do[:, :, -rows:]
        note = f", last {rows} query rows only (work scaled by rows)"
    frac = rows / cfg["M"]
    n = 0
    t0 = time.perf_counter()
    while n < max_passes and (n == 0 or time.perf_counter() - t0 < budget_s):
        cpu_slice_step(cfg, q, k, v, do)
        n += 1
    dt = time.perf_counter() - t0
    flops = slice_flops(cfg) * frac * n
    if cfg["causal"] and frac < 1.0:
        # the last rows of a causal problem see (almost) every key: x2 relative to the average row
        flops = 4.0 * (cfg["Hq"] // cfg["Hkv"]) * rows * cfg["N"] * cfg["D"] * n * \
            (3.5 if cfg["mode"] == "fwd+bwd" else 1.0)
    return {"value": flops / dt * 1e-12, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"{n} passes over 1 of the workload's {cfg['B'] * cfg['Hkv']} (batch, KV-group) units"
                      f"{note}, {dt:.1f} s, native {cfg['dtype']} math, {os.cpu_count()} logical CPUs"}


# ------------------------------------------------------------------ multi-GPU: the 32k configuration
def c5_sharded_legs(rank, world, device, dist, steps=5):
    """The 32k-token causal forward split over the ranks two ways, plus rank 0's single-GPU time of
    the whole configuration in the same run. Returns (c5_heads, c5_ring) records on rank 0."""
    from flagattention_b200 import flash_attention, ring, sharding, status
    cfg = dict(CONFIGS["c5_long_context_fwd"])
    flops = fwd_flops(cfg)
    q, k, v, _ = make_inputs(cfg, device, seed=5000)

    def timed(fn, n):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize(device)
        t = torch.tensor([e0.elapsed_time(e1) / n], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # rank 0 alone: the whole configuration on one GPU (the others idle at the barrier)
    single_ms = 0.0
    if rank == 0:
        for _ in range(2):
            flash_attention(q, k, v, causal=True)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            flash_attention(q, k, v, causal=True)
        e1.record()
        torch.cuda.synchronize(device)
        single_ms = e0.elapsed_time(e1) / steps
    dist.barrier()

    # by (batch x KV-head-group) units, no collective
    mine = [tuple(t.contiguous() for t in piece) for piece in sharding.shard(q, k, v, rank, world)]
    heads_ms = timed(lambda: [flash_attention(a, b_, c, causal=True) for a, b_, c in mine], steps)
    heads_launches = len(mine)
    del mine

    # ring-KV sequence parallel over NCCL
    ql, kl, vl = (ring.zigzag_shard(t, rank, world) for t in (q, k, v))
    del q, k, v
    ring.LAUNCHES = 0
    ring_ms = timed(lambda: ring.ring_attention_forward(ql, kl, vl), steps)
    ring_launches = ring.LAUNCHES // (steps + 3)
    status.check_device_status(device)
    if rank != 0:
        return None, None
    base = {"config": "c5_long_context_fwd (B1 Hq64 Hkv8 M=N=32768 D128 bf16 causal, forward)", "steps": steps,
            "single_gpu_ms": single_ms, "single_gpu_tflops": flops / single_ms * 1e-9, "scaling": "strong"}
    heads = dict(base, ms_per_step=heads_ms, tflops=flops / heads_ms * 1e-9, speedup_vs_single_gpu=single_ms / heads_ms,
                 launches_per_step_per_rank=heads_launches,
                 sharding="the 8 KV-head groups split over the ranks, no collective")
    ring_rec = dict(base, ms_per_step=ring_ms, tflops=flops / ring_ms * 1e-9, speedup_vs_single_gpu=single_ms / ring_ms,
                    launches_per_step_per_rank=ring_launches,
                    sharding="sequence split zig-zag over the ranks, K/V shards rotated with NCCL send/recv")
    return heads, ring_rec


def bind_to_gpu_numa_node(local_rank: int):
    """Best effort: restrict this process to the CPUs that sysfs lists as local to its GPU before any pinned
    buffer is allocated, so that the host side of the H2D/D2H copies lives on the GPU's own NUMA node (with
    every rank's buffers on one node the copies of an 8-GPU run share that node's memory bandwidth).
    Returns a short description for the record, or the reason nothing was changed."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        addr = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        text = Path(f"/sys/bus/pci/devices/{addr}/local_cpulist").read_text().strip()
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        local = cpus & allowed
        if not local:
            return f"unchanged: none of the GPU-local CPUs ({text}) is in this process's affinity mask"
        if local != allowed:
            os.sched_setaffinity(0, local)
        node = Path(f"/sys/bus/pci/devices/{addr}/numa_node").read_text().strip()
        return f"GPU {addr} numa node {node}: {len(local)} of {len(allowed)} allowed CPUs"
    except Exception as exc:  # noqa: BLE001
        return f"unchanged: {exc!r}"[:160]


# ------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=DEFAULT_CONFIG, choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-triton-reference", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (profiling runs)")
    ap.add_argument("--shard", default="auto", choices=["auto", "replicate", "heads", "ring"],
                    help="N>1: replicate = every rank runs the whole per-GPU workload (weak scaling, "
                         "default for training configs); heads = the workload's (batch x KV-group) units "
                         "are split over the ranks (strong scaling, default for the 32k config); ring = "
                         "ring-KV sequence parallel forward over NCCL (32k config only)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.batch > 0:
        cfg["B"] = args.batch
    warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config_desc = {"workload": args.config, **{k: cfg[k] for k in ("B", "Hq", "Hkv", "M", "N", "D", "dtype",
                                                                  "causal", "dropout_p", "mode")},
                   "sharding": "independent (batch x KV-head-group) units per rank, no collective",
                   "l2_policy": "inputs+outputs per step exceed the 126 MB L2 (no flush needed)"}
    metric = "flash_attention fwd+bwd TFLOPS (bf16 causal D=128)" if args.config == DEFAULT_CONFIG \
        else f"flash_attention {cfg['mode']} TFLOPS ({args.config})"

    shard_mode = args.shard
    if shard_mode == "auto":
        shard_mode = "heads" if (args.config == "c5_long_context_fwd" and world > 1) else "replicate"
    if world == 1:
        shard_mode = "replicate"
    if shard_mode == "ring" and (cfg["mode"] != "fwd" or not cfg["causal"]):
        raise SystemExit("--shard ring is the causal forward-only sequence-parallel mode")
    scaling = "weak" if shard_mode == "replicate" else "strong"
    config_desc["sharding"] = {
        "replicate": "every rank runs the full workload on its own seeded inputs, no collective",
        "heads": "the workload's (batch x KV-head-group) units are split over the ranks, no collective",
        "ring": "sequence split zig-zag over the ranks, K/V shards rotated with NCCL send/recv",
    }[shard_mode]

    if args.impl == "reference":
        # The reference's own CPU implementation of the path (its PyTorch attention, restated in
        # oracle/), all host threads, one (batch, KV-group) unit of the workload per step.
        if rank != 0:
            return
        use_all_host_threads()
        q, k, v, do = cpu_slice_inputs(cfg)
        rows = cfg["M"]
        if cfg["M"] * cfg["N"] > 4096 * 4096 * 4:
            rows = max(128, (4096 * 4096 * 4) // cfg["N"])
            q, do = q[:, :, -rows:], do[:, :, -rows:]
        steps = max(1, min(args.steps, 6))
        for _ in range(min(warmup, 1)):
            cpu_slice_step(cfg, q, k, v, do)
        t0 = time.perf_counter()
        for _ in range(steps):
            cpu_slice_step(cfg, q, k, v, do)
        dt = time.perf_counter() - t0
        per_step = slice_flops(cfg) * rows / cfg["M"]
        if cfg["causal"] and rows < cfg["M"]:
            per_step = 4.0 * (cfg["Hq"] // cfg["Hkv"]) * rows * cfg["N"] * cfg["D"] * \
                (3.5 if cfg["mode"] == "fwd+bwd" else 1.0)
        val = per_step * steps / dt * 1e-12
        sample = (f"each step = 1 of {cfg['B'] * cfg['Hkv']} (batch, KV-group) units"
                  + (f", last {rows} query rows" if rows < cfg["M"] else "") + f"; {steps} steps timed")
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
            "steps": steps, "warmup": min(warmup, 1), "ms_per_step": dt / steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg["dtype"],
            "data": "synthetic", "config": config_desc,
            "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": torch.get_num_threads(),
                             "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)
    from flagattention_b200 import status as status_mod

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    q, k, v, do = make_inputs(cfg, device, seed=1000 + (rank if shard_mode == "replicate" else 0))
    K = args.steps
    total_flops_per_step = step_flops(cfg) * (world if shard_mode == "replicate" else 1)
    ring_step = None
    if shard_mode == "heads":
        from flagattention_b200 import sharding
        my = sharding.shard(q, k, v, rank, world, do)
        if len(my) != 1:
            raise SystemExit("heads sharding expects each rank's units to lie in one batch")
        q, k, v, do = (t.contiguous() for t in my[0])
        cfg = dict(cfg, B=1, Hq=q.shape[1], Hkv=k.shape[1])
    elif shard_mode == "ring":
        from flagattention_b200 import ring
        q, k, v = (ring.zigzag_shard(t, rank, world) for t in (q, k, v))

        def ring_step():
            return ring.ring_attention_forward(q, k, v)

    # ---- device-resident timing --------------------------------------------------------------
    step = (lambda: ring_step()) if ring_step is not None else (lambda: run_step(cfg, q, k, v, do))
    # The clock sampler starts before the warm-up (nvidia-smi takes a few hundred ms to come up) and
    # runs through the timed region; only the samples stamped inside the timed region are reported.
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    for _ in range(warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if ring_step is not None:
        ring.LAUNCHES = 0
    wall0 = datetime.datetime.now()
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    ring_launches = ring.LAUNCHES if ring_step is not None else 0
    barrier()
    wall1 = datetime.datetime.now()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(wall0, wall1) if sampler else None
    status_mod.check_device_status(device)   # no kernel of the timed region gave up on a wait

    # ---- end-to-end timing: host buffers, copies inside the timed region ----------------------
    if args.no_e2e:
        if rank == 0:
            kern_ms, _ = time_kernels(cfg, (q, k, v, do), iters=1, n_sets=1)
            print(json.dumps({"profiling_run": True, "ms_per_step": ms_total / K, "kernels_ms": kern_ms}))
        if dist is not None:
            dist.destroy_process_group()
        return
    full_affinity = os.sched_getaffinity(0)
    numa_note = bind_to_gpu_numa_node(local_rank)
    host_in = [t.cpu().pin_memory() for t in (q, k, v, do)]
    outs = step()
    host_out = [torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory().zero_() for t in outs]
    os.sched_setaffinity(0, full_affinity)   # the pages are placed; the CPU legs below use every core again
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    # Copies and compute are pipelined over three streams with double-buffered device inputs, the
    # way a training input pipeline overlaps transfers with work: step s+1's inputs travel to the
    # device and step s-1's results travel back while step s computes. Every step still moves all
    # of its inputs and outputs inside the timed region.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_cmp = torch.cuda.current_stream(device)
    dev_in = [[torch.empty_like(t) for t in (q, k, v, do)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]     # compute no longer reads dev_in[i]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]      # host_out may be overwritten again

    def e2e_run(n_steps):
        for i in range(2):
            ev_free[i].record(s_cmp)
            ev_out[i].record(s_out)
        for s_idx in range(n_steps):
            i = s_idx & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[i])
                for d, h in zip(dev_in[i], host_in):
                    d.copy_(h, non_blocking=True)
                ev_in[i].record(s_in)
            s_cmp.wait_event(ev_in[i])
            res = ring.ring_attention_forward(*dev_in[i][:3]) if ring_step is not None \
                else run_step(cfg, *dev_in[i])
            ev_free[i].record(s_cmp)
            ev_cmp[i].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[i])
                s_out.wait_event(ev_out[i ^ 1])          # one D2H batch at a time, in order
                for h, d in zip(host_out, res):
                    d.record_stream(s_out)
                    h.copy_(d, non_blocking=True)
                ev_out[i].record(s_out)
        s_cmp.wait_stream(s_out)
        s_cmp.wait_stream(s_in)

    e2e_run(3)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_run(K)
    f1.record()
    barrier()
    ms_e2e_total = f0.elapsed_time(f1)
    status_mod.check_device_status(device)

    # The copies alone, one direction at a time (what the host side of this box can feed one GPU
    # while the other ranks do the same): the ceiling of the end-to-end number.
    def copy_rate(pairs, nbytes, reps=3):
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(reps):
            for dst, src in pairs:
                dst.copy_(src, non_blocking=True)
        c1.record()
        barrier()
        return nbytes * reps / (c0.elapsed_time(c1) * 1e-3) * 1e-9
    h2d_gbs = copy_rate(list(zip(dev_in[0], host_in)), h2d)
    d2h_gbs = copy_rate(list(zip(host_out, outs)), d2h)

    if dist is not None:
        t = torch.tensor([ms_total, ms_e2e_total, -h2d_gbs, -d2h_gbs], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e_total, h2d_gbs, d2h_gbs = t.tolist()
        h2d_gbs, d2h_gbs = -h2d_gbs, -d2h_gbs            # slowest rank

    # ---- per-kernel timing + roofline (rank 0) -------------------------------------------------
    result = None
    if rank == 0:
        peaks, peak_src = load_peaks()
        del dev_in
        kcfg = dict(cfg, M=q.shape[2], N=k.shape[2])   # ring mode: the rank-local problem
        kern_ms, alg_bytes = time_kernels(kcfg, (q, k, v, do))
        f_fwd = fwd_flops(kcfg)
        # Algorithmic FLOPs per launch: forward 2 GEMMs; dK/dV kernel 4 of the backward's 5 GEMMs
        # (S, dP, dV, dK); dQ kernel 1 (its S and dP are recomputation and not counted).
        # The fused pass (D = 128 and 64) performs all 5.
        alg = {"fwd_kernel": f_fwd, "bwd_kernel<kv>": 2.0 * f_fwd, "bwd_kernel<q>": 0.5 * f_fwd,
               "bwd_kernel<kv+dq>": 2.5 * f_fwd}
        dominant = max((n for n in kern_ms if n in alg), key=lambda n: kern_ms[n])
        achieved = alg[dominant] / (kern_ms[dominant] * 1e-3) * 1e-12
        burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        sustained = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        traffic, traffic_src = ncu_traffic(args.config, dominant, cfg["B"])
        value = total_flops_per_step * K / (ms_total * 1e-3) * 1e-12
        e2e_value = total_flops_per_step * K / (ms_e2e_total * 1e-3) * 1e-12
        step_s = ms_total / K * 1e-3
        result = {
            "metric": metric, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16" if cfg["dtype"] == "bfloat16" else "fp16",
            "data": "synthetic", "config": config_desc,
            "per_gpu_tflops": value / world,
            "tokens_per_s": CONFIGS[args.config]["B"] * cfg["M"] * (world if shard_mode == "replicate" else 1) / step_s,
            "frac_of_spec_peak_2250": value / world / SPEC_PEAK_TFLOPS,
            "frac_of_measured_burst_peak": value / world / burst,
            "frac_of_measured_sustained_peak": value / world / sustained,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e_total / K,
                    "h2d_gbs_per_gpu": h2d_gbs, "d2h_gbs_per_gpu": d2h_gbs,
                    "copy_floor_ms_per_step": max(h2d / h2d_gbs, d2h / d2h_gbs) * 1e-6,
                    "host_numa_binding": numa_note,
                    "note": "copy rates are of each direction by itself, slowest rank, all ranks copying at "
                            "once; the step cannot be faster than the slower direction"},
            "gpu_launches": kernels_per_step(cfg) * K if ring_step is None else ring_launches,
            "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": burst,
                         "unit": "TFLOP/s", "frac": achieved / burst,
                         "peak_source": f"{peak_src} burst bf16 GEMM (the kernel is timed in isolation: median of "
                                        "20 launches, one CUDA-event pair each, two rotating buffer sets)",
                         "frac_burst": achieved / burst, "frac_sustained": achieved / sustained,
                         "frac_spec_2250": achieved / SPEC_PEAK_TFLOPS,
                         "algorithmic_flops": alg[dominant], "ms": kern_ms[dominant],
                         "traffic": traffic if args.batch == 0 or traffic is not None else None,
                         "traffic_source": traffic_src, "algorithmic_bytes": alg_bytes.get(dominant)},
            "kernels_ms": kern_ms,
            "kernels_alg_tflops": {n: alg[n] / (kern_ms[n] * 1e-3) * 1e-12 for n in alg if n in kern_ms},
        }
        if world == 1 and not args.no_triton_reference and ring_step is None:
            result["triton_reference"] = triton_reference(cfg, q, k, v, do)
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(cfg)
    if dist is not None and args.config == DEFAULT_CONFIG and args.shard == "auto":
        del q, k, v, do, host_in, host_out, outs
        torch.cuda.empty_cache()
        try:
            heads, ring_rec = c5_sharded_legs(rank, world, device, dist)
        except Exception as exc:  # noqa: BLE001  (the headline record above must survive a failure here)
            heads = ring_rec = {"error": repr(exc)[:300]}
        if result is not None:
            result["c5_heads"], result["c5_ring"] = heads, ring_rec
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if result is not None:
        print(json.dumps(result))


if __name__ == "__main__":
    main()

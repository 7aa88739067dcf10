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
  overlap the compute on separate streams).
* ``roofline`` describes the dominant kernel of the step, timed by itself through the C ABI.
* ``cpu_baseline`` times the CPU oracle (the reference's PyTorch attention restated) on a bounded
  sample of the same workload on this host's cores.
* ``--impl reference`` runs only that CPU path (all host threads) and prints its own line.

N > 1: launched under torchrun, one rank per GPU; every rank runs the full per-GPU workload
(independent (batch x KV-head-group) units, no collective on the data path), so scaling is weak.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
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

FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel on the default
# workload, from the ncu capture summarised under profiles/ (None until captured).
NCU_TRAFFIC_BYTES = {
    # (dram read + write) MB measured at batch 2, scaled x2 to the batch-4 workload (traffic is
    # proportional to batch); the capture is summarised under profiles/
    "c2_gqa_prefill_train": {"bwd_kernel<kv>": 2 * (220.867072e6 + 22.053632e6),
                             "bwd_kernel<kv+dq>": 2 * (468.678144e6 + 205.996544e6),
                             "fwd_kernel": 2 * (101.170944e6 + 31.920384e6)},
}


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


# ------------------------------------------------------------------ clocks sampling
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

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

    def stop(self):
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": sm_max,
                "reasons": reasons, "samples": len(rows)}


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
    # or (D = 128 and 64) the fused dK/dV/dQ kernel and the dQ conversion (the accumulator's memset is the
    # driver's, not counted).
    return 1 + (4 if cfg["mode"] == "fwd+bwd" else 0)


def time_kernels(cfg, q, k, v, do, iters=5):
    """Times the library's kernels one by one through the C ABI (CUDA events on the launching
    stream) and returns {name: ms}."""
    from flagattention_b200 import _lib
    lib = _lib.load()
    dev = q.device
    B, Hq, Hkv, M, N, D = (cfg[x] for x in ("B", "Hq", "Hkv", "M", "N", "D"))
    dt = _lib.dtype_code(q.dtype)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, M, dtype=torch.float32, device=dev)
    sm_scale = 1.0 / math.sqrt(D)
    # dropout: the forward caches its keep decisions for the backward, as flash_attention does
    keep_mask = None
    if cfg["dropout_p"] > 0 and cfg["mode"] == "fwd+bwd":
        keep_mask = torch.empty(lib.b200attn_keep_mask_bytes(B, Hq, M, N) // 4, dtype=torch.int32, device=dev)
    mask_ptr = keep_mask.data_ptr() if keep_mask is not None else None
    fp = _lib.FwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o), lse.data_ptr(),
                        B, Hq, Hkv, M, N, D, dt, dt, int(cfg["causal"]), sm_scale, float(cfg["dropout_p"]),
                        12345, 0, status.data_ptr(), 0, 0, 0, mask_ptr)

    def timed(fn):
        fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / iters

    out = {"fwd_kernel": timed(lambda: _lib.check(lib.b200attn_fwd(fp, stream), "fwd"))}
    if cfg["mode"] == "fwd+bwd":
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        delta = torch.empty_like(lse)
        ws = torch.empty(lib.b200attn_bwd_workspace_bytes(B, Hq, Hkv, M, N, D) // 4, dtype=torch.float32,
                         device=dev)
        bp = _lib.BwdParams(_lib.tensor4(q), _lib.tensor4(k), _lib.tensor4(v), _lib.tensor4(o),
                            _lib.tensor4(do), _lib.tensor4(dq), _lib.tensor4(dk), _lib.tensor4(dv),
                            lse.data_ptr(), delta.data_ptr(), ws.data_ptr(), B, Hq, Hkv, M, N, D, dt, dt,
                            int(cfg["causal"]), sm_scale, float(cfg["dropout_p"]), 12345, 0,
                            status.data_ptr(), 0, 0, 0, mask_ptr)
        # D = 128 and 64: one fused pass makes dK, dV and dQ (plus the zeroing of its fp32 dQ accumulator),
        # followed by the accumulator's conversion; other head dimensions run two separate kernels.
        names = (("bwd_prep_kernels", 1), ("bwd_kernel<kv+dq>", 2), ("dq_convert_kernel", 4)) if D in (64, 128) else \
                (("bwd_prep_kernels", 1), ("bwd_kernel<kv>", 2), ("bwd_kernel<q>", 4))
        for name, mask in names:
            out[name] = timed(lambda m=mask: _lib.check(lib.b200attn_bwd_stages(bp, stream, m), name))
    assert status.item() == 0, "a kernel reported a device-side wait timeout"
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


def cpu_baseline(cfg, budget_s=12.0, max_slices=64):
    """Times the oracle (native-dtype path, i.e. the reference's PyTorch CPU attention) on whole
    (batch, KV-group) units until `budget_s` seconds or `max_slices` units have run."""
    threads = use_all_host_threads()
    q, k, v, do = cpu_slice_inputs(cfg)
    # long-context slices do not fit the budget: shrink the query rows of the sample and say so
    rows = cfg["M"]
    note = ""
    if cfg["M"] * cfg["N"] > 4096 * 4096 * 4:
        rows = max(128, (4096 * 4096 * 4) // cfg["N"])
        q, do = q[:, :, -rows:], do[:, :, -rows:]
        note = f", last {rows} query rows only (work scaled by rows)"
    frac = rows / cfg["M"]
    n = 0
    t0 = time.perf_counter()
    while n < max_slices and (n == 0 or time.perf_counter() - t0 < budget_s):
        cpu_slice_step(cfg, q, k, v, do)
        n += 1
    dt = time.perf_counter() - t0
    flops = slice_flops(cfg) * frac * n
    if cfg["causal"] and frac < 1.0:
        # the last rows of a causal problem see (almost) every key: x2 relative to the average row
        flops = 4.0 * (cfg["Hq"] // cfg["Hkv"]) * rows * cfg["N"] * cfg["D"] * n * \
            (3.5 if cfg["mode"] == "fwd+bwd" else 1.0)
    return {"value": flops / dt * 1e-12, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"{n} of {cfg['B'] * cfg['Hkv']} (batch, KV-group) units of the workload{note}, "
                      f"{dt:.1f} s, native {cfg['dtype']} math, {os.cpu_count()} logical CPUs"}


# ------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=DEFAULT_CONFIG, choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    # runs through the timed region; warm-up steps are the same work, so every sample is under load.
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
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    ring_launches = ring.LAUNCHES if ring_step is not None else 0
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None

    # ---- end-to-end timing: host buffers, copies inside the timed region ----------------------
    if args.no_e2e:
        if rank == 0:
            kern_ms = time_kernels(cfg, q, k, v, do, iters=1)
            print(json.dumps({"profiling_run": True, "ms_per_step": ms_total / K, "kernels_ms": kern_ms}))
        if dist is not None:
            dist.destroy_process_group()
        return
    host_in = [t.cpu().pin_memory() for t in (q, k, v, do)]
    outs = step()
    host_out = [torch.empty(t.shape, dtype=t.dtype, device="cpu").pin_memory() for t in outs]
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

    if dist is not None:
        t = torch.tensor([ms_total, ms_e2e_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e_total = t.tolist()

    # ---- per-kernel timing + roofline (rank 0) -------------------------------------------------
    result = None
    if rank == 0:
        peaks, peak_src = load_peaks()
        kcfg = dict(cfg, M=q.shape[2], N=k.shape[2])   # ring mode: the rank-local problem
        kern_ms = time_kernels(kcfg, q, k, v, do)
        f_fwd = fwd_flops(kcfg)
        # Algorithmic FLOPs per launch: forward 2 GEMMs; dK/dV kernel 4 of the backward's 5 GEMMs
        # (S, dP, dV, dK); dQ kernel 1 (its S and dP are recomputation and not counted).
        # The fused pass (D = 128 and 64) performs all 5 (its launch time includes zeroing the dQ accumulator).
        alg = {"fwd_kernel": f_fwd, "bwd_kernel<kv>": 2.0 * f_fwd, "bwd_kernel<q>": 0.5 * f_fwd,
               "bwd_kernel<kv+dq>": 2.5 * f_fwd}
        dominant = max((n for n in kern_ms if n in alg), key=lambda n: kern_ms[n])
        achieved = alg[dominant] / (kern_ms[dominant] * 1e-3) * 1e-12
        peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        value = total_flops_per_step * K / (ms_total * 1e-3) * 1e-12
        e2e_value = total_flops_per_step * K / (ms_e2e_total * 1e-3) * 1e-12
        result = {
            "metric": metric, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "bf16" if cfg["dtype"] == "bfloat16" else "fp16",
            "data": "synthetic", "config": config_desc,
            "per_gpu_tflops": value / world, "tokens_per_s": CONFIGS[args.config]["B"] * cfg["M"] * K * (world if shard_mode == "replicate" else 1)
            / (ms_total * 1e-3),
            "frac_of_spec_peak_2250": value / world / 2250.0,
            "frac_of_measured_burst_peak": value / world / float(peaks.get("bf16_tflops", 1590.0)),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e_total / K},
            "gpu_launches": kernels_per_step(cfg) * K if ring_step is None else ring_launches,
            "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": f"{peak_src} sustained bf16",
                         "traffic": (NCU_TRAFFIC_BYTES.get(args.config) or {}).get(dominant)
                         if args.batch == 0 else None},
            "kernels_ms": kern_ms,
            "kernels_alg_tflops": {n: alg[n] / (kern_ms[n] * 1e-3) * 1e-12 for n in alg if n in kern_ms},
        }
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(cfg)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if result is not None:
        print(json.dumps(result))


if __name__ == "__main__":
    main()

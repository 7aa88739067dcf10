// Shared host/device helpers: error reporting, dropout RNG, TMA tensor-map encoding.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/b200attn.h"
#include "ptx.cuh"

namespace b200attn {

// --------------------------------------------------------------- host errors
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define B200ATTN_CUDA_OK(expr)                                  \
  do {                                                          \
    cudaError_t _e = (expr);                                    \
    if (_e != cudaSuccess) return ::b200attn::cuda_fail(_e, #expr); \
  } while (0)

// One-time set-up per device (kernel attributes, device properties) that any host thread may
// trigger: `run(f)` executes `f` once for the current device under std::call_once and hands back its
// return code to every caller; a failed attempt is remembered and reported again, not retried.
struct PerDeviceOnce {
  static constexpr int MAX_DEVICES = 64;
  std::once_flag flags[MAX_DEVICES];
  int rc[MAX_DEVICES] = {};
  template <class F>
  int run(F&& f) {
    int dev = 0;
    B200ATTN_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return f();  // beyond the table: set up on every call
    std::call_once(flags[dev], [&] { rc[dev] = f(); });
    return rc[dev];
  }
};

// Encodes a 4-D tiled tensor map over a [B, H, rows, D] tensor of 16-bit elements
// (dims listed innermost first: D, rows, H, B). `box_cols` x `box_rows` is the tile;
// `swizzle` is a CUtensorMapSwizzle value. Returns 0 or a negative B200ATTN_E* code.
int encode_tmap_4d(CUtensorMap* out, const b200attn_tensor& t, int elem_bytes, int64_t B, int64_t H,
                   int64_t rows, int64_t D, int box_cols, int box_rows, int swizzle,
                   const char* name, int box_heads = 1);

// Checks the TMA requirements of one operand; returns 0 or B200ATTN_EINVAL.
int check_tma_operand(const b200attn_tensor& t, int elem_bytes, const char* name);

// Writes the padded per-query statistics the backward / total-attention kernels stream
// (aux_kernels.cu). `delta` may be null (total attention).
// delta[b,h,m] = sum_d o*do; optionally also clears a contiguous fp32 [B, H, M, D] array.
int bwd_delta(const b200attn_tensor* o, int32_t o_dtype, const b200attn_tensor* d_o, int32_t do_dtype,
              float* delta, int32_t B, int32_t H, int32_t M, int32_t D, void* stream, float* zero_rows);
int launch_stats(const float* lse, const float* delta, float2* stats, int B, int H, int M, int Mpad,
                 cudaStream_t stream);

// Smallest integer threshold T such that a Philox word x (folded to [0, 2^31)) is KEPT iff x > T,
// equivalent to `float(x) * 4.6566127342e-10f > dropout_p` evaluated in fp32.
int32_t dropout_keep_threshold(float dropout_p);

// --------------------------------------------------------------- device RNG
// Philox-4x32 with 6 rounds, keyed by the 64-bit seed, counter = (ctr_lo, ctr_hi, 0, 0);
// returns output word 0. This is the generator behind the reference's `tl.rand(seed, offs,
// n_rounds=6)` (flash.py:474-477); only word 0 of each call is consumed there.
__host__ __device__ __forceinline__ uint32_t philox6_word0(uint32_t seed_lo, uint32_t seed_hi,
                                                           uint32_t ctr_lo, uint32_t ctr_hi) {
  constexpr uint32_t KEY_A = 0x9E3779B9u, KEY_B = 0xBB67AE85u;
  constexpr uint32_t ROUND_A = 0xD2511F53u, ROUND_B = 0xCD9E8D57u;
  uint32_t c0 = ctr_lo, c1 = ctr_hi, c2 = 0u, c3 = 0u;
  uint32_t k0 = seed_lo, k1 = seed_hi;
#pragma unroll
  for (int r = 0; r < 6; ++r) {
    const uint64_t pa = static_cast<uint64_t>(ROUND_A) * c0;
    const uint64_t pb = static_cast<uint64_t>(ROUND_B) * c2;
    const uint32_t n0 = static_cast<uint32_t>(pb >> 32) ^ c1 ^ k0;
    const uint32_t n2 = static_cast<uint32_t>(pa >> 32) ^ c3 ^ k1;
    c1 = static_cast<uint32_t>(pb);
    c3 = static_cast<uint32_t>(pa);
    c0 = n0;
    c2 = n2;
    k0 += KEY_A;
    k1 += KEY_B;
  }
  return c0;
}

// Per-launch dropout constants. Element (b,h,m,n) draws counter
// offset + ((b*H + h)*M + m)*N + n (flash.py:387-391). The reference's kernel does this
// arithmetic in 32 bits when `offset` fits in int32 (the counter's high word is then 0) and in
// 64 bits otherwise; `wide` selects between the two.
struct DropoutCtx {
  uint32_t seed_lo, seed_hi;
  uint64_t offset;
  int32_t keep_threshold;
  uint32_t wide;
  float inv_keep;  // 1 / (1 - p)
  // Optional cache of the keep decisions, written by the forward and read by the backward instead of
  // re-evaluating Philox: bit i of word keep_mask[((b * Hq + h) * mask_words + w) * M + m] says whether
  // (query m, key 32 * w + i) is kept. Word-major, so that both a thread per query row (forward,
  // dQ kernel) and 32 lanes holding 32 consecutive queries (dK/dV kernel) touch consecutive words.
  uint32_t* keep_mask;
  int mask_words;  // ceil(N / 32)
};

__host__ inline DropoutCtx make_dropout_ctx(float p, uint64_t seed, uint64_t offset) {
  DropoutCtx c;
  c.seed_lo = static_cast<uint32_t>(seed);
  c.seed_hi = static_cast<uint32_t>(seed >> 32);
  c.offset = offset;
  c.keep_threshold = dropout_keep_threshold(p);
  c.wide = offset >= (1ull << 31) ? 1u : 0u;
  c.inv_keep = 1.0f / (1.0f - p);
  c.keep_mask = nullptr;
  c.mask_words = 0;
  return c;
}

// keep-decision for the element whose exact 64-bit counter is `ctr`.
__device__ __forceinline__ bool dropout_keep(const DropoutCtx& c, uint64_t ctr) {
  const uint32_t lo = static_cast<uint32_t>(ctr);
  const uint32_t hi = c.wide ? static_cast<uint32_t>(ctr >> 32) : 0u;
  const int32_t x = static_cast<int32_t>(philox6_word0(c.seed_lo, c.seed_hi, lo, hi));
  const int32_t folded = x ^ (x >> 31);  // x < 0 ? -x - 1 : x
  return folded > c.keep_threshold;
}

// Keep decisions of 32 consecutive counters base, base+1, ..., base+31 as a bit mask (bit i = element
// i is kept). The counter's high word is the same for all 32 unless the low word wraps inside the
// run, which lets the compiler hoist the first Philox round's key mixing out of the loop.
__device__ __forceinline__ uint32_t dropout_keep_word(const DropoutCtx& c, uint64_t base) {
  const uint32_t lo0 = static_cast<uint32_t>(base);
  uint32_t bits = 0u;
  if (lo0 <= 0xffffffffu - 31u) {
    const uint32_t hi = c.wide ? static_cast<uint32_t>(base >> 32) : 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int32_t x = static_cast<int32_t>(philox6_word0(c.seed_lo, c.seed_hi, lo0 + i, hi));
      bits |= ((x ^ (x >> 31)) > c.keep_threshold ? 1u : 0u) << i;
    }
  } else {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) bits |= (dropout_keep(c, base + i) ? 1u : 0u) << i;
  }
  return bits;
}

// Same for 32 counters base + i * stride (elements of one key column across consecutive queries).
__device__ __forceinline__ uint32_t dropout_keep_word_strided(const DropoutCtx& c, uint64_t base,
                                                              uint64_t stride) {
  uint32_t bits = 0u;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const uint64_t ctr = base + stride * static_cast<uint64_t>(i);
    const uint32_t hi = c.wide ? static_cast<uint32_t>(ctr >> 32) : 0u;
    const int32_t x = static_cast<int32_t>(philox6_word0(c.seed_lo, c.seed_hi, static_cast<uint32_t>(ctr), hi));
    bits |= ((x ^ (x >> 31)) > c.keep_threshold ? 1u : 0u) << i;
  }
  return bits;
}

// ------------------------------------------------------------ small helpers
__host__ __device__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// Band limits of the kernels (see FwdArgs::d_min): `causal` and the optional band of the C ABI
// folded together. Returns whether any side is finite.
__host__ inline bool fold_band(bool causal, int band, int dist_min, int dist_max, int* d_min, int* d_max) {
  constexpr int INF = 1 << 30;
  int lo = causal ? 0 : -INF, hi = INF;
  if (band) {
    const int bmin = dist_min < -INF ? -INF : (dist_min > INF ? INF : dist_min);
    const int bmax = dist_max < -INF ? -INF : (dist_max > INF ? INF : dist_max);
    if (bmin > lo) lo = bmin;
    if (bmax < hi) hi = bmax;
  }
  *d_min = lo;
  *d_max = hi;
  return lo > -INF || hi < INF;
}

// 1-D grid order. Blocks are numbered so that (batch, head) pairs are visited in chunks of `chunk`
// pairs; inside a chunk the row-block index z is the slow coordinate. With z sorted from the
// longest block to the shortest this dispatches long (causal) blocks first, while a chunk's K/V
// (or Q/dO) working set stays small enough to live in L2.
struct BlockCoord { int bh, z; };
__device__ __forceinline__ BlockCoord decode_block(int id, int BH, int n_z, int chunk) {
  const int per_chunk = chunk * n_z;
  const int full = BH / chunk;
  int c = id / per_chunk;
  int width = chunk;
  if (c >= full) { c = full; width = BH - full * chunk; }
  const int rem = id - c * per_chunk;
  BlockCoord out;
  out.z = rem / width;
  out.bh = c * chunk + rem - out.z * width;
  return out;
}
// Division of a non-negative 31-bit integer by a divisor fixed on the host: one high multiply and one
// shift (mul = ceil(2^(31 + ceil(log2 d)) / d)) instead of the ~40-instruction integer division.
struct FastDiv {
  uint32_t d, mul, shr;
  __host__ static FastDiv make(int64_t divisor) {
    FastDiv f;
    f.d = divisor < 1 ? 1u : static_cast<uint32_t>(divisor);
    f.mul = 0;
    f.shr = 0;
    if (f.d > 1) {
      uint32_t lg = 0;
      while ((1ull << lg) < f.d) ++lg;
      const uint32_t p = 31 + lg;
      f.mul = static_cast<uint32_t>(((1ull << p) + f.d - 1) / f.d);
      f.shr = p - 32;
    }
    return f;
  }
  __host__ __device__ __forceinline__ int div(int n) const {
#ifdef __CUDA_ARCH__
    return d == 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shr);
#else
    return d == 1 ? n : static_cast<int>(static_cast<uint32_t>((static_cast<uint64_t>(static_cast<uint32_t>(n)) * mul) >> 32) >> shr);
#endif
  }
};
// decode_block() with the divisions prepared on the host.
struct BlockOrder {
  FastDiv per_chunk, width, tail_width;
  int chunk, full;  // pairs per chunk, number of full chunks
  __host__ static BlockOrder make(int64_t BH, int n_z, int chunk) {
    BlockOrder o;
    o.chunk = chunk;
    o.full = static_cast<int>(BH / chunk);
    o.per_chunk = FastDiv::make(static_cast<int64_t>(chunk) * n_z);
    o.width = FastDiv::make(chunk);
    o.tail_width = FastDiv::make(BH - static_cast<int64_t>(o.full) * chunk);
    return o;
  }
  __host__ __device__ __forceinline__ BlockCoord decode(int id) const {
    int c = per_chunk.div(id);
    const bool tail = c >= full;
    if (tail) c = full;
    const int rem = id - c * static_cast<int>(per_chunk.d);
    BlockCoord out;
    out.z = tail ? tail_width.div(rem) : width.div(rem);
    out.bh = c * chunk + rem - out.z * static_cast<int>(tail ? tail_width.d : width.d);
    return out;
  }
};
// Number of (batch, head) pairs per chunk: all query heads of as many KV heads as fit `budget`
// bytes of streamed operand per KV head (`bytes_per_kv_head`), at least one KV head.
__host__ inline int grid_chunk(int groups, int64_t bytes_per_kv_head, bool causal) {
  if (!causal) return groups;
  const int64_t budget = 96ll << 20;
  int64_t n = budget / (bytes_per_kv_head > 0 ? bytes_per_kv_head : 1);
  if (n < 1) n = 1;
  if (n > 4096) n = 4096;
  return static_cast<int>(n) * groups;
}

// Status codes written to the optional device status word.
enum : int32_t {
  ST_OK = 0,
  ST_WAIT_TMA = 1,   // a TMA "full" barrier never completed
  ST_WAIT_MMA = 2,   // a tensor-core completion barrier never completed
  ST_WAIT_SOFTMAX = 3,
  ST_WAIT_EMPTY = 4,
};

__device__ __forceinline__ void report_status(int32_t* status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// The bounded wait of every kernel role. Returns true once the barrier phase has completed; false
// when it gives up: after `limit_ns`, or as soon as this CTA (`abort_flag`, in shared memory) or any
// CTA of any launch sharing the status word has reported a failure. The caller then records its own
// code (report_status + *abort_flag = 1), leaves its loop and joins the kernel's final barrier, after
// which TMEM is released.
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                             const int32_t* status, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xffu) == 0u) {
      if (*abort_flag) return false;
      if (status != nullptr && *reinterpret_cast<const volatile int32_t*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
}

}  // namespace b200attn

// One-tile tcgen05 product with caller-chosen descriptor fields.
//
// The attention kernels depend on a handful of hardware layout conventions (swizzled
// K-major and MN-major shared-memory operands, 16-bit A operands packed in TMEM). This
// kernel runs a single 128 x n x (16 * k_steps) product with those conventions passed in
// from the host, so a GPU test can pin each of them against a plain matmul.
#include "common.cuh"
#include "ptx.cuh"

namespace b200attn {

struct SelftestArgs {
  const uint16_t* a_gmem;
  float* d;
  int a_cols, b_rows, b_cols, box_cols;
  int a_in_tmem, n, k_steps;
  uint32_t idesc;
  uint64_t a_desc_hi, b_desc_hi;
  int a_step_bytes, b_step_bytes, a_chunk_steps, b_chunk_steps, a_chunk_bytes, b_chunk_bytes;
  int32_t* status;
};

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const SelftestArgs args) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;               // 32 KB
  uint8_t* sB = smem + 32768;       // 32 KB
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    failed = 0;
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (tid == 0) {
    const int a_chunks = args.a_cols / args.box_cols;
    const int b_chunks = args.b_cols / args.box_cols;
    const uint32_t a_bytes = 128u * args.a_cols * 2u;
    const uint32_t b_bytes = static_cast<uint32_t>(args.b_rows) * args.b_cols * 2u;
    mbar_expect_tx(&bar_load, a_bytes + b_bytes);
    for (int c = 0; c < a_chunks; ++c)
      tma_load_4d(sA + c * (128 * args.box_cols * 2), &tmA, &bar_load, c * args.box_cols, 0, 0, 0);
    for (int c = 0; c < b_chunks; ++c)
      tma_load_4d(sB + c * (args.b_rows * args.box_cols * 2), &tmB, &bar_load, c * args.box_cols, 0,
                  0, 0);
  }

  __syncwarp();
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tmem_a = tmem_base + 256;
  if (args.a_in_tmem == 1) {
    // Row `tid` of A, packed two 16-bit values per 32-bit TMEM column.
    const uint32_t* row = reinterpret_cast<const uint32_t*>(args.a_gmem + tid * args.a_cols);
    for (int c = 0; c < args.a_cols / 2; c += 8) {
      uint32_t r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = row[c + i];
      tmem_st8(tmem_a + lane_base + c, r);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (tid == 0) {
    if (!mbar_wait(&bar_load, 0)) {
      report_status(args.status, ST_WAIT_TMA);
      failed = 1;
    } else {
      tc_fence_after();
      for (int s = 0; s < args.k_steps; ++s) {
        const int a_off = args.a_chunk_steps > 0
                              ? (s / args.a_chunk_steps) * args.a_chunk_bytes +
                                    (s % args.a_chunk_steps) * args.a_step_bytes
                              : s * args.a_step_bytes;
        const int b_off = args.b_chunk_steps > 0
                              ? (s / args.b_chunk_steps) * args.b_chunk_bytes +
                                    (s % args.b_chunk_steps) * args.b_step_bytes
                              : s * args.b_step_bytes;
        const uint64_t db = smem_desc(args.b_desc_hi, smem_u32(sB) + b_off);
        if (args.a_in_tmem == 2) {
          // A slice goes shared memory -> TMEM with tcgen05.cp, then feeds the MMA from TMEM.
          const uint64_t da = smem_desc(args.a_desc_hi, smem_u32(sA) + a_off);
          asm volatile("tcgen05.cp.cta_group::1.128x256b [%0], %1;" ::"r"(tmem_a + s * 8), "l"(da) : "memory");
          mma_ts(tmem_base, tmem_a + s * 8, db, args.idesc, s > 0 ? 1u : 0u);
        } else if (args.a_in_tmem) {
          mma_ts(tmem_base, tmem_a + s * 8, db, args.idesc, s > 0 ? 1u : 0u);
        } else {
          const uint64_t da = smem_desc(args.a_desc_hi, smem_u32(sA) + a_off);
          mma_ss(tmem_base, da, db, args.idesc, s > 0 ? 1u : 0u);
        }
      }
      tc_commit(&bar_mma);
      if (!mbar_wait(&bar_mma, 0)) {
        report_status(args.status, ST_WAIT_MMA);
        failed = 1;
      }
    }
  }
  __syncthreads();
  __syncwarp();
  tc_fence_after();
  if (!failed) {
    for (int c = 0; c < args.n; c += 16) {
      uint32_t r[16];
      tmem_ld16(tmem_base + lane_base + c, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) args.d[tid * args.n + c + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace b200attn

extern "C" int b200attn_umma_selftest(const b200attn_selftest_params* p, void* stream) {
  using namespace b200attn;
  if (p == nullptr || p->a == nullptr || p->b == nullptr || p->d == nullptr) {
    set_error("selftest: null argument");
    return B200ATTN_EINVAL;
  }
  if (p->a_cols <= 0 || p->a_cols > 128 || p->b_rows <= 0 || p->b_cols <= 0 ||
      p->b_rows * p->b_cols > 128 * 128 || p->box_cols <= 0 || p->box_cols > 64 ||
      p->a_cols % p->box_cols != 0 || p->b_cols % p->box_cols != 0 || p->n % 16 != 0 || p->n > 256 ||
      p->n <= 0 || p->k_steps <= 0 || p->k_steps > 16 || p->b_rows > 256) {
    set_error("selftest: shape out of range");
    return B200ATTN_EINVAL;
  }
  // Every descriptor start address must stay inside the operand's 32 KB staging area.
  for (int s = 0; s < p->k_steps; ++s) {
    const int a_off = p->a_chunk_steps > 0 ? (s / p->a_chunk_steps) * p->a_chunk_bytes +
                                                 (s % p->a_chunk_steps) * p->a_step_bytes
                                           : s * p->a_step_bytes;
    const int b_off = p->b_chunk_steps > 0 ? (s / p->b_chunk_steps) * p->b_chunk_bytes +
                                                 (s % p->b_chunk_steps) * p->b_step_bytes
                                           : s * p->b_step_bytes;
    if (a_off < 0 || a_off >= 32768 || b_off < 0 || b_off >= 32768 || a_off % 16 || b_off % 16) {
      set_error("selftest: descriptor offset out of range");
      return B200ATTN_EINVAL;
    }
  }
  CUtensorMap tmA, tmB;
  b200attn_tensor ta{const_cast<void*>(p->a), {0, 0, p->a_cols, 1}};
  b200attn_tensor tb{const_cast<void*>(p->b), {0, 0, p->b_cols, 1}};
  int rc = encode_tmap_4d(&tmA, ta, 2, 1, 1, 128, p->a_cols, p->box_cols, 128, p->swizzle, "selftest.a");
  if (rc) return rc;
  rc = encode_tmap_4d(&tmB, tb, 2, 1, 1, p->b_rows, p->b_cols, p->box_cols, p->b_rows, p->swizzle,
                      "selftest.b");
  if (rc) return rc;
  SelftestArgs a;
  a.a_gmem = static_cast<const uint16_t*>(p->a);
  a.d = p->d;
  a.a_cols = p->a_cols; a.b_rows = p->b_rows; a.b_cols = p->b_cols; a.box_cols = p->box_cols;
  a.a_in_tmem = p->a_in_tmem; a.n = p->n; a.k_steps = p->k_steps;
  a.idesc = p->idesc; a.a_desc_hi = p->a_desc_hi; a.b_desc_hi = p->b_desc_hi;
  a.a_step_bytes = p->a_step_bytes; a.b_step_bytes = p->b_step_bytes;
  a.a_chunk_steps = p->a_chunk_steps; a.b_chunk_steps = p->b_chunk_steps;
  a.a_chunk_bytes = p->a_chunk_bytes; a.b_chunk_bytes = p->b_chunk_bytes;
  a.status = p->status;
  const int smem_bytes = 65536 + 1024;
  static PerDeviceOnce attr_once;
  rc = attr_once.run([&]() -> int {
    B200ATTN_CUDA_OK(cudaFuncSetAttribute(umma_selftest_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    return B200ATTN_OK;
  });
  if (rc) return rc;
  umma_selftest_kernel<<<1, 128, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, a);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

// ------------------------------------------------------------------ the give-up path of the waits
namespace b200attn {

// Runs the protocol every kernel follows when a wait does not complete, on purpose and harmlessly:
// the CTA allocates TMEM like the attention kernels, warp 0 waits (bounded_wait, the function those
// kernels use, with a caller-chosen short limit) on an mbarrier that nothing ever arrives at, records
// `code` in the status word and raises the CTA's abort flag; the other warps wait on a second barrier
// with a far longer limit and must be released early by that flag. All warps then meet at the final
// barrier and TMEM is released. `out[0]` = 1 if warp 0's wait gave up, `out[1]` = number of other
// warps that were released by the abort flag, `out[2]` = nanoseconds warp 0 waited.
__global__ void __launch_bounds__(128, 1)
wait_timeout_selftest_kernel(unsigned long long limit_ns, int32_t code, int32_t* status, long long* out) {
  __shared__ uint64_t never_a, never_b;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  __shared__ int released;
  volatile int* abort_flag = &abort_flag_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&never_a, 1);
    mbar_init(&never_b, 1);
    abort_flag_s = 0;
    released = 0;
    fence_barrier_init();
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0) {
    const unsigned long long t0 = globaltimer_ns();
    const bool w = bounded_wait(&never_a, 0, abort_flag, nullptr, limit_ns);
    const unsigned long long waited = globaltimer_ns() - t0;
    if (!__all_sync(0xffffffffu, w)) {
      if (lane == 0) {
        report_status(status, code);
        *abort_flag = 1;
        out[0] = 1;
        out[2] = static_cast<long long>(waited);
      }
    }
  } else {
    // 100 x the short limit: only the abort flag can end this wait in time
    const bool w = bounded_wait(&never_b, 0, abort_flag, nullptr, 100ull * limit_ns);
    if (!__all_sync(0xffffffffu, w) && lane == 0 && *abort_flag) atomicAdd(&released, 1);
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (threadIdx.x == 0) out[1] = released;
  if (warp == 0) tmem_dealloc(tmem_base, 32);
}

}  // namespace b200attn

extern "C" int b200attn_wait_timeout_selftest(int32_t limit_us, int32_t code, int32_t* status, long long* out,
                                              void* stream) {
  using namespace b200attn;
  if (status == nullptr || out == nullptr) {
    set_error("wait_timeout_selftest: null argument");
    return B200ATTN_EINVAL;
  }
  if (limit_us < 1 || limit_us > 1000) {
    set_error("wait_timeout_selftest: limit must be 1..1000 microseconds (got %d)", limit_us);
    return B200ATTN_EINVAL;
  }
  if (code < 1 || code > 4) {
    set_error("wait_timeout_selftest: code must be one of the kernels' status codes 1..4");
    return B200ATTN_EINVAL;
  }
  wait_timeout_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(limit_us) * 1000ull, code, status, out);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

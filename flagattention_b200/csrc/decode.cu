// Decode-shaped split-KV partial pass: at most a handful of query rows per KV head (one new token,
// or a small group of heads sharing a KV head). With so few rows a 128-row tensor-core tile would
// spend its time on padding; the work is one multiply-add per two streamed bytes, far below the
// CUDA cores' rate, so the kernel is a pure HBM stream: 16-byte loads straight into registers,
// D/8 lanes per key, online softmax per lane group, groups merged once at the end.
//
// Replaces `_fwd_split_kv_kernel` (split_kv.py:28-196) for these shapes; the partial format
// (normalised fp32 O per split + natural-log normaliser per split) is the one the combine step
// `_fwd_combine_kv_splits` (split_kv.py:199-231) expects.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "decode.cuh"

namespace b200attn {

namespace {

constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_UNROLL = 4;

template <bool BF16>
__device__ __forceinline__ float round_to_input(float x) {
  if constexpr (BF16) {
    return __bfloat162float(__float2bfloat16_rn(x));
  } else {
    return __half2float(__float2half_rn(x));
  }
}

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack2<BF16>(u.x), b = unpack2<BF16>(u.y), c = unpack2<BF16>(u.z),
               d = unpack2<BF16>(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__device__ __forceinline__ uint4 ldg_stream(const uint16_t* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// exp2 of a difference where the subtrahend may be -inf (nothing seen yet): the caller passes a
// finite stand-in for the subtrahend, so -inf minus finite gives 0 and no NaN can appear.
__device__ __forceinline__ float exp2_diff(float a, float b_finite) { return exp2f(a - b_finite); }

template <int D, int R, bool BF16>
__global__ void __launch_bounds__(DEC_THREADS, R == 1 ? 3 : 2)
decode_partial_kernel(const DecodeArgs a) {
  constexpr int LPK = D / 8;        // lanes that share one key
  constexpr int KPW = 32 / LPK;     // keys per warp-wide load
  constexpr int STEP = DEC_WARPS * KPW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = lane / LPK, sub = lane % LPK;
  const int split = blockIdx.x % a.num_splits;
  const int bhk = blockIdx.x / a.num_splits;
  const int hk = bhk % a.Hkv;
  const int b = bhk / a.Hkv;
  const int rows = a.groups * a.M;  // <= R
  const bool paged = a.block_table != nullptr;
  const int N = paged ? a.context_lens[b] : a.N;
  const int P_SEQ = N - a.M;

  // Query rows (head-major within the KV head's group) and their visible key limits.
  float q[R][8];
  int lim[R];
  int lim_max = 0;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int g = r / a.M, m = r % a.M;
    if (r < rows) {
      const uint16_t* qp = a.q + b * a.q_sb + static_cast<int64_t>(hk * a.groups + g) * a.q_sh +
                           static_cast<int64_t>(m) * a.q_sm + sub * 8;
      unpack8<BF16>(*reinterpret_cast<const uint4*>(qp), q[r]);
      lim[r] = a.causal ? min(N, max(0, P_SEQ + m + 1)) : N;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) q[r][i] = 0.f;
      lim[r] = 0;
    }
    lim_max = max(lim_max, lim[r]);
  }

  const int n_lo = split * a.keys_per_split;
  const int n_hi = min(lim_max, n_lo + a.keys_per_split);
  const uint16_t* kbase = a.k + (paged ? 0 : b * a.k_sb) + static_cast<int64_t>(hk) * a.k_sh + sub * 8;
  const uint16_t* vbase = a.v + (paged ? 0 : b * a.v_sb) + static_cast<int64_t>(hk) * a.v_sh + sub * 8;
  const int32_t* table = paged ? a.block_table + b * a.bt_stride : nullptr;
  const int block_mask = (1 << a.block_shift) - 1;
  // Element offsets of key n's row in K and V.
  auto row_offsets = [&](int n, int64_t& ko, int64_t& vo) {
    if (paged) {
      const int64_t blk = __ldg(table + (n >> a.block_shift));
      const int64_t r = n & block_mask;
      ko = blk * a.k_sb + r * a.k_sn;
      vo = blk * a.v_sb + r * a.v_sn;
    } else {
      ko = static_cast<int64_t>(n) * a.k_sn;
      vo = static_cast<int64_t>(n) * a.v_sn;
    }
  };

  float m_run[R], l_run[R], acc[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
  }

  // The loop bound is warp-uniform (the shuffles below need every lane); a lane group's keys are
  // base + group + u * STEP. The next iteration's loads are issued before this iteration's
  // arithmetic, so every warp always has 2 * DEC_UNROLL 16-byte loads in flight.
  // With two rows the next iteration's loads are issued before this iteration's arithmetic (the
  // arithmetic is long enough to expose the load latency otherwise); with one row the registers
  // are better spent on a third resident CTA per SM.
  constexpr bool PREFETCH = R >= 2;
  uint4 kraw[DEC_UNROLL], vraw[DEC_UNROLL];
  auto fetch = [&](int first_key, uint4 (&kr)[DEC_UNROLL], uint4 (&vr)[DEC_UNROLL]) {
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) {
      const int n = first_key + u * STEP;
      if (n < n_hi) {
        int64_t ko, vo;
        row_offsets(n, ko, vo);
        kr[u] = ldg_stream(kbase + ko);
        vr[u] = ldg_stream(vbase + vo);
      } else {
        kr[u] = make_uint4(0, 0, 0, 0);
        vr[u] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  if constexpr (PREFETCH) fetch(n_lo + warp * KPW + group, kraw, vraw);
  for (int base = n_lo + warp * KPW; base < n_hi; base += STEP * DEC_UNROLL) {
    const int n0 = base + group;
    uint4 knext[PREFETCH ? DEC_UNROLL : 1], vnext[PREFETCH ? DEC_UNROLL : 1];
    if constexpr (PREFETCH) {
      fetch(n0 + STEP * DEC_UNROLL, knext, vnext);
    } else {
      fetch(n0, kraw, vraw);
    }
    float s[DEC_UNROLL][R];
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) {
      float kf[8];
      unpack8<BF16>(kraw[u], kf);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(q[r][i], kf[i], d);
        s[u][r] = d;
      }
    }
#pragma unroll
    for (int off = LPK / 2; off >= 1; off >>= 1) {
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
#pragma unroll
        for (int r = 0; r < R; ++r) s[u][r] += __shfl_xor_sync(0xffffffffu, s[u][r], off);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        const int n = n0 + u * STEP;
        s[u][r] = (n < lim[r] && n < n_hi) ? s[u][r] * a.qk_scale : -INFINITY;
        mx = fmaxf(mx, s[u][r]);
      }
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2_diff(m_run[r], m_use);
      l_run[r] *= alpha;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][i] *= alpha;
      m_run[r] = m_new;
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        const float p = exp2_diff(s[u][r], m_use);
        l_run[r] += p;
        s[u][r] = round_to_input<BF16>(p);  // the reference multiplies P in the value dtype
      }
    }
#pragma unroll
    for (int u = 0; u < DEC_UNROLL; ++u) {
      float vf[8];
      unpack8<BF16>(vraw[u], vf);
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(s[u][r], vf[i], acc[r][i]);
      }
    }
    if constexpr (PREFETCH) {
#pragma unroll
      for (int u = 0; u < DEC_UNROLL; ++u) {
        kraw[u] = knext[u];
        vraw[u] = vnext[u];
      }
    }
  }

  // Merge the lane groups of the warp (they hold the same feature columns, different keys).
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run[r], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run[r], off);
      const float m_new = fmaxf(m_run[r], m_o);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float w_self = exp2_diff(m_run[r], m_use), w_o = exp2_diff(m_o, m_use);
      l_run[r] = l_run[r] * w_self + l_o * w_o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[r][i], off);
        acc[r][i] = acc[r][i] * w_self + a_o * w_o;
      }
      m_run[r] = m_new;
    }
  }

  // Merge the warps through shared memory.
  __shared__ float sm_m[DEC_WARPS][R], sm_l[DEC_WARPS][R];
  __shared__ float sm_acc[DEC_WARPS][R][D];
  if (group == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_acc[warp][r][sub * 8 + i] = acc[r][i];
      if (sub == 0) {
        sm_m[warp][r] = m_run[r];
        sm_l[warp][r] = l_run[r];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * D; idx += DEC_THREADS) {
    const int r = idx / D, d = idx % D;
    float m_new = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m_new = fmaxf(m_new, sm_m[w][r]);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    float l_tot = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wgt = exp2_diff(sm_m[w][r], m_use);
      l_tot += sm_l[w][r] * wgt;
      o += sm_acc[w][r][d] * wgt;
    }
    o = l_tot > 0.f ? o / l_tot : 0.f;
    const int g = r / a.M, m = r % a.M;
    const int64_t h = hk * a.groups + g;
    const float lse = l_tot > 0.f ? m_new * 0.6931471805599453f + logf(l_tot) : -INFINITY;
    if (a.final_o != nullptr) {
      uint16_t* dst = a.final_o + b * a.o_sb + h * a.o_sh + static_cast<int64_t>(m) * a.o_sm + d;
      if constexpr (BF16) {
        const __nv_bfloat16 v = __float2bfloat16_rn(o);
        *dst = *reinterpret_cast<const uint16_t*>(&v);
      } else {
        const __half v = __float2half_rn(o);
        *dst = *reinterpret_cast<const uint16_t*>(&v);
      }
      if (d == 0) a.final_lse[(static_cast<int64_t>(b) * a.Hq + h) * a.M + m] = lse;
    } else {
      const int64_t row = ((static_cast<int64_t>(b) * a.Hq + h) * a.num_splits + split) * a.M + m;
      a.part_o[row * D + d] = o;
      if (d == 0) a.part_lse[row] = lse;
    }
  }
}

template <int D, int R>
int launch_rows(const DecodeArgs& a, bool bf16, unsigned grid, cudaStream_t stream) {
  if (bf16) {
    decode_partial_kernel<D, R, true><<<grid, DEC_THREADS, 0, stream>>>(a);
  } else {
    decode_partial_kernel<D, R, false><<<grid, DEC_THREADS, 0, stream>>>(a);
  }
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

template <int D>
int launch_d(const DecodeArgs& a, bool bf16, unsigned grid, cudaStream_t stream) {
  const int rows = a.groups * a.M;
  if (rows <= 1) return launch_rows<D, 1>(a, bf16, grid, stream);
  return launch_rows<D, 2>(a, bf16, grid, stream);
}

}  // namespace

int launch_decode_partial(const DecodeArgs& a, int D, bool bf16, cudaStream_t stream) {
  const int64_t grid = static_cast<int64_t>(a.B) * a.Hkv * a.num_splits;
  if (grid > 2147483647ll || a.groups * a.M > DECODE_MAX_ROWS) {
    set_error("decode: grid or row count out of range");
    return B200ATTN_EINVAL;
  }
  switch (D) {
    case 16: return launch_d<16>(a, bf16, static_cast<unsigned>(grid), stream);
    case 32: return launch_d<32>(a, bf16, static_cast<unsigned>(grid), stream);
    case 64: return launch_d<64>(a, bf16, static_cast<unsigned>(grid), stream);
    default: return launch_d<128>(a, bf16, static_cast<unsigned>(grid), stream);
  }
}

}  // namespace b200attn

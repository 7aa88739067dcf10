// Bandwidth-bound helper kernels: dropout keep-mask materialisation and the backward
// preprocess delta = rowsum(O * dO).
#include "common.cuh"

namespace b200attn {

// mask[idx] = keep(offset + idx) over the flattened [B, H, M, N] index space; one thread per
// 16 consecutive elements so stores are 16 bytes wide.
__global__ void __launch_bounds__(256)
dropout_mask_kernel(uint8_t* __restrict__ mask, int64_t total, DropoutCtx ctx) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 16;
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 16; base < total;
       base += stride) {
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t idx = base + i;
      const bool keep = idx < total && dropout_keep(ctx, ctx.offset + static_cast<uint64_t>(idx));
      w[i >> 2] |= (keep ? 1u : 0u) << (8 * (i & 3));
    }
    if (base + 16 <= total && (reinterpret_cast<uintptr_t>(mask + base) & 15) == 0) {
      *reinterpret_cast<uint4*>(mask + base) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int i = 0; i < 16 && base + i < total; ++i) mask[base + i] = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
    }
  }
}

// One warp per row of D elements: lanes read 16-byte vectors, shuffle-reduce, lane 0 writes.
template <int D, int O_KIND, bool DO_BF16>
__global__ void __launch_bounds__(256)
delta_kernel(const void* __restrict__ o, const void* __restrict__ d_o, float* __restrict__ delta,
             int64_t o_sb, int64_t o_sh, int64_t o_sm, int64_t do_sb, int64_t do_sh, int64_t do_sm, int B,
             int H, int M, float* __restrict__ zero_rows) {
  constexpr int VEC = 8;                 // elements per lane per step
  constexpr int LANES = D / VEC;         // lanes that carry data for one row (2..16)
  constexpr int ROWS_PER_WARP = 32 / LANES;
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int sub = lane / LANES;
  const int col = (lane % LANES) * VEC;
  const int64_t row_id = static_cast<int64_t>(warp_global) * ROWS_PER_WARP + sub;
  const int64_t total = static_cast<int64_t>(B) * H * M;
  float acc = 0.f;
  if (row_id < total) {
    const int m = static_cast<int>(row_id % M);
    const int h = static_cast<int>((row_id / M) % H);
    const int b = static_cast<int>(row_id / (static_cast<int64_t>(M) * H));
    const int64_t o_off = b * o_sb + h * o_sh + m * o_sm + col;
    const int64_t do_off = b * do_sb + h * do_sh + m * do_sm + col;
    float ov[VEC], gv[VEC];
    if constexpr (O_KIND == B200ATTN_F32) {
      const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(o) + o_off);
      const float4 a = p[0], c = p[1];
      ov[0] = a.x; ov[1] = a.y; ov[2] = a.z; ov[3] = a.w;
      ov[4] = c.x; ov[5] = c.y; ov[6] = c.z; ov[7] = c.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(o) + o_off);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<O_KIND == B200ATTN_BF16>(w[i]);
        ov[2 * i] = f.x; ov[2 * i + 1] = f.y;
      }
    }
    {
      const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(d_o) + do_off);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<DO_BF16>(w[i]);
        gv[2 * i] = f.x; gv[2 * i + 1] = f.y;
      }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc = fmaf(ov[i], gv[i], acc);
    // Optional: clear the matching 8 elements of a contiguous fp32 [B, H, M, D] array (the dQ
    // accumulator of the fused backward), saving a separate pass over it.
    if (zero_rows != nullptr) {
      float4* z = reinterpret_cast<float4*>(zero_rows + row_id * D + col);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int s = LANES / 2; s >= 1; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (row_id < total && (lane % LANES) == 0) delta[row_id] = acc;
}

// Per-query statistics for the backward / total-attention kernels, two queries per float4:
// stats4[b, h, m/2] = (-lse[m]*log2e, -lse[m+1]*log2e, -delta[m], -delta[m+1]); the padding rows
// m in [M, Mpad) get (-inf, 0). Rows without any visible key (lse = -inf) also get -inf, so that
// every probability recomputed against them, exp2(s*c + (-inf)), is exactly 0.
__global__ void __launch_bounds__(256)
stats_kernel(const float* __restrict__ lse, const float* __restrict__ delta, float4* __restrict__ stats,
             int64_t BH, int M, int Mpad) {
  const int half = Mpad / 2;
  const int64_t total = BH * half;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t bh = i / half;
    const int m = static_cast<int>(i - bh * half) * 2;
    float nl[2] = {-INFINITY, -INFINITY}, nd[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (m + j < M) {
        const float l = lse[bh * M + m + j];
        nl[j] = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
        nd[j] = delta != nullptr ? -delta[bh * M + m + j] : 0.f;
      }
    }
    stats[i] = make_float4(nl[0], nl[1], nd[0], nd[1]);
  }
}

int launch_stats(const float* lse, const float* delta, float2* stats, int B, int H, int M, int Mpad,
                 cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(B) * H * (Mpad / 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  stats_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      lse, delta, reinterpret_cast<float4*>(stats), static_cast<int64_t>(B) * H, M, Mpad);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

template <int D>
static int launch_delta(const b200attn_tensor* o, int o_dtype, const b200attn_tensor* d_o, int do_dtype,
                        float* delta, int B, int H, int M, cudaStream_t stream, float* zero_rows) {
  constexpr int ROWS_PER_WARP = 32 / (D / 8);
  const int64_t total = static_cast<int64_t>(B) * H * M;
  const int64_t warps = (total + ROWS_PER_WARP - 1) / ROWS_PER_WARP;
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
#define B200ATTN_DELTA(OK, DB)                                                                        \
  delta_kernel<D, OK, DB><<<blocks, 256, 0, stream>>>(o->ptr, d_o->ptr, delta, o->stride[0],          \
                                                      o->stride[1], o->stride[2], d_o->stride[0],    \
                                                      d_o->stride[1], d_o->stride[2], B, H, M, zero_rows)
  const bool db = do_dtype == B200ATTN_BF16;
  if (o_dtype == B200ATTN_F32) { if (db) B200ATTN_DELTA(B200ATTN_F32, true); else B200ATTN_DELTA(B200ATTN_F32, false); }
  else if (o_dtype == B200ATTN_BF16) { if (db) B200ATTN_DELTA(B200ATTN_BF16, true); else B200ATTN_DELTA(B200ATTN_BF16, false); }
  else { if (db) B200ATTN_DELTA(B200ATTN_F16, true); else B200ATTN_DELTA(B200ATTN_F16, false); }
#undef B200ATTN_DELTA
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

// Log-sum-exp merge of two partial attention results over disjoint key sets:
// lse = log(exp(lse_a) + exp(lse_b)), o = o_a * exp(lse_a - lse) + o_b * exp(lse_b - lse).
// The accumulator is updated in place; a partial with lse = -inf (no visible key) leaves it
// unchanged. Both sides are [heads, rows_per_head, D] fp32 arrays of which `rows` rows per head,
// starting at row0, take part. One thread per 4 features; the threads of a row sit in one warp.
__global__ void __launch_bounds__(256)
merge_partial_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const float* __restrict__ o_part,
                     const float* __restrict__ lse_part, int64_t heads, int rows, int D, int acc_rph,
                     int acc_row0, int part_rph, int part_row0, int first) {
  const int vec_per_row = D / 4;
  const int64_t total = heads * rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t flat_row = i / vec_per_row;
    const int vec = static_cast<int>(i - flat_row * vec_per_row);
    const int64_t head = flat_row / rows;
    const int r = static_cast<int>(flat_row - head * rows);
    const int64_t ra = head * acc_rph + acc_row0 + r;
    const int64_t rb = head * part_rph + part_row0 + r;
    const float lb = lse_part[rb];
    const float la = first ? -INFINITY : lse_acc[ra];
    const float mx = fmaxf(la, lb);
    float wa = 0.f, wb = 0.f, lse = -INFINITY;
    if (mx != -INFINITY) {
      const float ea = __expf(la - mx), eb = __expf(lb - mx);
      const float inv = 1.0f / (ea + eb);
      wa = ea * inv;
      wb = eb * inv;
      lse = mx + __logf(ea + eb);
    }
    float4* pa = reinterpret_cast<float4*>(o_acc + ra * D) + vec;
    float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *pa;
    const float4 b = reinterpret_cast<const float4*>(o_part + rb * D)[vec];
    a.x = a.x * wa + b.x * wb;
    a.y = a.y * wa + b.y * wb;
    a.z = a.z * wa + b.z * wb;
    a.w = a.w * wa + b.w * wb;
    *pa = a;
    // All threads of a row are lanes of one warp and have read lse_acc[ra] above; after the warp
    // re-converges the lane owning the row's last vector publishes the new value.
    __syncwarp(__activemask());
    if (vec == vec_per_row - 1) lse_acc[ra] = lse;
  }
}

// The same merge for two complete partial results [B, H, M, D] whose sum is final: the merged row goes
// straight to the 16-bit output tensor (its own strides) and only the log-normaliser is updated in
// place, which saves the fp32 write-back and the separate conversion pass. One thread per 8 features.
template <bool BF16>
__global__ void __launch_bounds__(256)
merge_store_kernel(const float* __restrict__ o_a, float* __restrict__ lse_a, const float* __restrict__ o_b,
                   const float* __restrict__ lse_b, uint16_t* __restrict__ out, int64_t out_sb, int64_t out_sh,
                   int64_t out_sm, int H, int M, int D, int64_t total) {
  const int vec_per_row = D / 8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int vec = static_cast<int>(i - row * vec_per_row);
    const float la = lse_a[row], lb = lse_b[row];
    const float mx = fmaxf(la, lb);
    float wa = 0.f, wb = 0.f, lse = -INFINITY;
    if (mx != -INFINITY) {
      const float ea = __expf(la - mx), eb = __expf(lb - mx);
      const float inv = 1.0f / (ea + eb);
      wa = ea * inv;
      wb = eb * inv;
      lse = mx + __logf(ea + eb);
    }
    const float4* pa = reinterpret_cast<const float4*>(o_a + row * D) + 2 * vec;
    const float4* pb = reinterpret_cast<const float4*>(o_b + row * D) + 2 * vec;
    const float4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
    uint4 v;
    v.x = pack2<BF16>(a0.x * wa + b0.x * wb, a0.y * wa + b0.y * wb);
    v.y = pack2<BF16>(a0.z * wa + b0.z * wb, a0.w * wa + b0.w * wb);
    v.z = pack2<BF16>(a1.x * wa + b1.x * wb, a1.y * wa + b1.y * wb);
    v.w = pack2<BF16>(a1.z * wa + b1.z * wb, a1.w * wa + b1.w * wb);
    const int64_t bh = row / M;
    const int m = static_cast<int>(row - bh * M);
    const int64_t b = bh / H;
    const int h = static_cast<int>(bh - b * H);
    *reinterpret_cast<uint4*>(out + b * out_sb + h * out_sh + static_cast<int64_t>(m) * out_sm + 8 * vec) = v;
    // (the lanes of a row sit in one warp and have all read lse_a[row] above)
    __syncwarp(__activemask());
    if (vec == vec_per_row - 1) lse_a[row] = lse;
  }
}

static int check_vec_tensor(const b200attn_tensor* t, int eb, const char* name) {
  if (t == nullptr || t->ptr == nullptr) {
    set_error("%s: null tensor", name);
    return B200ATTN_EINVAL;
  }
  if (t->stride[3] != 1 || reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0 || (t->stride[0] * eb) % 16 ||
      (t->stride[1] * eb) % 16 || (t->stride[2] * eb) % 16) {
    set_error("%s: needs feature stride 1 and 16-byte aligned base / strides", name);
    return B200ATTN_EINVAL;
  }
  return B200ATTN_OK;
}

}  // namespace b200attn

extern "C" int b200attn_dropout_mask(uint8_t* mask, int32_t B, int32_t H, int32_t M, int32_t N,
                                     float dropout_p, uint64_t seed, uint64_t offset, void* stream) {
  using namespace b200attn;
  if (mask == nullptr || B <= 0 || H <= 0 || M <= 0 || N <= 0) {
    set_error("dropout_mask: bad argument");
    return B200ATTN_EINVAL;
  }
  if (!(dropout_p >= 0.f && dropout_p < 1.f)) {
    set_error("dropout_mask: dropout_p must be in [0, 1)");
    return B200ATTN_EINVAL;
  }
  const int64_t total = static_cast<int64_t>(B) * H * M * N;
  const DropoutCtx ctx = make_dropout_ctx(dropout_p, seed, offset);
  const int64_t threads = (total + 15) / 16;
  int64_t blocks = (threads + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  dropout_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, total, ctx);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

namespace b200attn {
int bwd_delta(const b200attn_tensor* o, int32_t o_dtype, const b200attn_tensor* d_o, int32_t do_dtype,
              float* delta, int32_t B, int32_t H, int32_t M, int32_t D, void* stream, float* zero_rows) {
  if (delta == nullptr || B <= 0 || H <= 0 || M <= 0) {
    set_error("bwd_delta: bad argument");
    return B200ATTN_EINVAL;
  }
  int rc = check_vec_tensor(o, o_dtype == B200ATTN_F32 ? 4 : 2, "bwd_delta.o");
  if (rc) return rc;
  rc = check_vec_tensor(d_o, 2, "bwd_delta.do");
  if (rc) return rc;
  if (do_dtype != B200ATTN_F16 && do_dtype != B200ATTN_BF16) {
    set_error("bwd_delta: do must be fp16 or bf16");
    return B200ATTN_EINVAL;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (D) {
    case 16: return launch_delta<16>(o, o_dtype, d_o, do_dtype, delta, B, H, M, s, zero_rows);
    case 32: return launch_delta<32>(o, o_dtype, d_o, do_dtype, delta, B, H, M, s, zero_rows);
    case 64: return launch_delta<64>(o, o_dtype, d_o, do_dtype, delta, B, H, M, s, zero_rows);
    case 128: return launch_delta<128>(o, o_dtype, d_o, do_dtype, delta, B, H, M, s, zero_rows);
    default:
      set_error("bwd_delta: head dimension %d not in {16, 32, 64, 128}", D);
      return B200ATTN_EINVAL;
  }
}
}  // namespace b200attn

extern "C" int b200attn_bwd_delta(const b200attn_tensor* o, int32_t o_dtype, const b200attn_tensor* d_o,
                                  int32_t do_dtype, float* delta, int32_t B, int32_t H, int32_t M,
                                  int32_t D, void* stream) {
  return b200attn::bwd_delta(o, o_dtype, d_o, do_dtype, delta, B, H, M, D, stream, nullptr);
}

extern "C" int b200attn_merge_partial(float* o_acc, float* lse_acc, const float* o_part,
                                      const float* lse_part, int64_t heads, int32_t rows, int32_t D,
                                      int32_t acc_rows_per_head, int32_t acc_row0,
                                      int32_t part_rows_per_head, int32_t part_row0, int32_t first,
                                      void* stream) {
  using namespace b200attn;
  if (o_acc == nullptr || lse_acc == nullptr || o_part == nullptr || lse_part == nullptr || heads <= 0 ||
      rows <= 0 || (D != 16 && D != 32 && D != 64 && D != 128) || acc_row0 < 0 || part_row0 < 0 ||
      acc_row0 + rows > acc_rows_per_head || part_row0 + rows > part_rows_per_head) {
    set_error("merge_partial: bad argument");
    return B200ATTN_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(o_acc) % 16 != 0 || reinterpret_cast<uintptr_t>(o_part) % 16 != 0) {
    set_error("merge_partial: o buffers must be 16-byte aligned");
    return B200ATTN_EINVAL;
  }
  const int64_t total = heads * rows * (D / 4);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  merge_partial_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      o_acc, lse_acc, o_part, lse_part, heads, rows, D, acc_rows_per_head, acc_row0, part_rows_per_head,
      part_row0, first ? 1 : 0);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}


extern "C" int b200attn_merge_partial_store(const float* o_a, float* lse_a, const float* o_b, const float* lse_b,
                                            int32_t B, int32_t H, int32_t M, int32_t D, const b200attn_tensor* out,
                                            int32_t out_dtype, void* stream) {
  using namespace b200attn;
  if (o_a == nullptr || lse_a == nullptr || o_b == nullptr || lse_b == nullptr || B <= 0 || H <= 0 || M <= 0 ||
      (D != 16 && D != 32 && D != 64 && D != 128)) {
    set_error("merge_partial_store: bad argument");
    return B200ATTN_EINVAL;
  }
  if (out_dtype != B200ATTN_F16 && out_dtype != B200ATTN_BF16) {
    set_error("merge_partial_store: the output must be fp16 or bf16");
    return B200ATTN_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(o_a) % 16 != 0 || reinterpret_cast<uintptr_t>(o_b) % 16 != 0) {
    set_error("merge_partial_store: partial outputs must be 16-byte aligned");
    return B200ATTN_EINVAL;
  }
  const int rc = check_vec_tensor(out, 2, "merge_partial_store.out");
  if (rc) return rc;
  const int64_t total = static_cast<int64_t>(B) * H * M * (D / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  uint16_t* dst = static_cast<uint16_t*>(out->ptr);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == B200ATTN_BF16) {
    merge_store_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        o_a, lse_a, o_b, lse_b, dst, out->stride[0], out->stride[1], out->stride[2], H, M, D, total);
  } else {
    merge_store_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        o_a, lse_a, o_b, lse_b, dst, out->stride[0], out->stride[1], out->stride[2], H, M, D, total);
  }
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

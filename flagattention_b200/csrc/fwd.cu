// C entry point of the forward pass: argument validation, TMA descriptors, dispatch on D.
#include "decode.cuh"
#include "fwd_launch.cuh"

namespace b200attn {

// `kv_rows`: keys per K/V box (128, or 64 for the 64-key pipeline of the D = 128 kernel).
template <int D>
static int make_fwd_tmaps(const b200attn_fwd_params* p, FwdLaunch& L, int kv_rows = TileCfg<D>::BLOCK) {
  using Cfg = TileCfg<D>;
  int rc = encode_tmap_4d(&L.tmQ, p->q, 2, p->B, p->Hq, p->M, D, Cfg::CHUNK, Cfg::BLOCK, Cfg::TMA_SWZ, "q");
  if (rc) return rc;
  rc = encode_tmap_4d(&L.tmK, p->k, 2, p->B, p->Hkv, p->N, D, Cfg::CHUNK, kv_rows, Cfg::TMA_SWZ, "k");
  if (rc) return rc;
  return encode_tmap_4d(&L.tmV, p->v, 2, p->B, p->Hkv, p->N, D, Cfg::CHUNK, kv_rows, Cfg::TMA_SWZ, "v");
}

// Work-item order of the forward kernel with its divisions prepared (FwdArgs::order and friends).
static void set_item_order(FwdArgs& a, int64_t grid_heads) {
  a.order = BlockOrder::make(static_cast<int64_t>(a.B) * grid_heads, a.n_zblocks, a.grid_chunk);
  a.div_heads = FastDiv::make(grid_heads);
  a.div_groups = FastDiv::make(a.groups);
  a.div_splits = FastDiv::make(a.num_splits);
}

// 16-bit outputs leave through shared memory and TMA stores (one box of 32 rows per softmax warp); when
// the output cannot be described by a tensor map the kernel stores from registers instead.
template <int D>
static void make_o_tmap(const b200attn_fwd_params* p, FwdLaunch& L) {
  using Cfg = TileCfg<D>;
  L.args.o_tma = 0;
  if (p->o_dtype == B200ATTN_F32) return;
  if (encode_tmap_4d(&L.tmO, p->o, 2, p->B, p->Hq, p->M, D, Cfg::CHUNK, 32, Cfg::TMA_SWZ, "o") ==
      B200ATTN_OK) {
    L.args.o_tma = 1;
  }
}

}  // namespace b200attn

namespace b200attn {
namespace {
int cached_sm_count();
}  // namespace
}  // namespace b200attn

extern "C" int b200attn_fwd(const b200attn_fwd_params* p, void* stream) {
  using namespace b200attn;
  if (p == nullptr) {
    set_error("fwd: null params");
    return B200ATTN_EINVAL;
  }
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->M <= 0 || p->N <= 0) {
    set_error("fwd: B, Hq, Hkv, M, N must be positive (got %d %d %d %d %d)", p->B, p->Hq, p->Hkv, p->M,
              p->N);
    return B200ATTN_EINVAL;
  }
  if (p->Hq % p->Hkv != 0) {
    set_error("fwd: number of heads in q must be a multiple of that in k & v");
    return B200ATTN_EINVAL;
  }
  if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) {
    set_error("fwd: head dimension %d not in {16, 32, 64, 128}", p->D);
    return B200ATTN_EINVAL;
  }
  if (p->dtype != B200ATTN_F16 && p->dtype != B200ATTN_BF16) {
    set_error("fwd: dtype must be fp16 or bf16");
    return B200ATTN_EINVAL;
  }
  if (p->o_dtype != p->dtype && p->o_dtype != B200ATTN_F32) {
    set_error("fwd: o_dtype must equal dtype or be fp32");
    return B200ATTN_EINVAL;
  }
  if (p->o.ptr == nullptr || p->lse == nullptr) {
    set_error("fwd: null output pointer");
    return B200ATTN_EINVAL;
  }
  const int o_eb = p->o_dtype == B200ATTN_F32 ? 4 : 2;
  if (p->o.stride[3] != 1 || reinterpret_cast<uintptr_t>(p->o.ptr) % 16 != 0 ||
      (p->o.stride[0] * o_eb) % 16 != 0 || (p->o.stride[1] * o_eb) % 16 != 0 ||
      (p->o.stride[2] * o_eb) % 16 != 0) {
    set_error("fwd: o needs feature stride 1, 16-byte aligned base and row/head/batch strides");
    return B200ATTN_EINVAL;
  }
  if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f)) {
    set_error("fwd: dropout_p must be in [0, 1)");
    return B200ATTN_EINVAL;
  }
  if (static_cast<int64_t>(p->B) * p->Hq * cdiv(p->M, 256) > 2147483647ll) {
    set_error("fwd: B * Hq * ceil(M / 256) exceeds the grid limit");
    return B200ATTN_EINVAL;
  }

  FwdLaunch L{};  // zero: every optional mode (packing, paging) is off unless set below
  // D = 128 with a mask (causal or a band): the 64-key softmax pipeline. Same-GPU A/B against the
  // 128-key pipeline: +3 % to +6 % on causal sequences of 2k to 32k keys, +23 % at 512; without a mask
  // it measured 0 to 4 % slower, so those launches keep the 128-key pipeline.
  int band_lo = 0, band_hi = 0;
  L.split64 = p->D == 128 && fold_band(p->causal != 0, p->band, p->dist_min, p->dist_max, &band_lo, &band_hi);
  int rc;
  switch (p->D) {
    case 16: rc = make_fwd_tmaps<16>(p, L); break;
    case 32: rc = make_fwd_tmaps<32>(p, L); break;
    case 64: rc = make_fwd_tmaps<64>(p, L); break;
    default: rc = make_fwd_tmaps<128>(p, L, L.split64 ? 64 : 128); break;
  }
  if (rc) return rc;

  FwdArgs& a = L.args;
  a.o = p->o.ptr;
  a.lse = p->lse;
  a.o_stride_b = p->o.stride[0];
  a.o_stride_h = p->o.stride[1];
  a.o_stride_m = p->o.stride[2];
  a.o_stride_split = 0;
  a.lse_stride_b = static_cast<int64_t>(p->Hq) * p->M;
  a.lse_stride_h = p->M;
  a.lse_stride_split = 0;
  a.num_splits = 1;
  a.tiles_per_split = cdiv(p->N, 128);
  a.pack_heads = 0;
  a.dual_stream = 0;
  a.ring_stages = 0;
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.groups = p->Hq / p->Hkv;
  a.causal = fold_band(p->causal != 0, p->band, p->dist_min, p->dist_max, &a.d_min, &a.d_max) ? 1 : 0;
  a.o_fp32 = p->o_dtype == B200ATTN_F32 ? 1 : 0;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(p->dropout_p, p->seed, p->offset);
  if (p->dropout_p > 0.f && p->keep_mask != nullptr) {
    a.drop.keep_mask = p->keep_mask;
    a.drop.mask_words = cdiv(p->N, 32);
  }
  a.status = p->status;
  a.n_zblocks = cdiv(p->M, 256);
  a.grid_chunk = grid_chunk(a.groups, 4ll * p->N * p->D, a.causal != 0);
  set_item_order(a, p->Hq);
  switch (p->D) {
    case 16: make_o_tmap<16>(p, L); break;
    case 32: make_o_tmap<32>(p, L); break;
    case 64: make_o_tmap<64>(p, L); break;
    default: make_o_tmap<128>(p, L); break;
  }
  // One CTA per SM walks the list of work items when there are more items than SMs. The list is
  // dealt out in a fixed order, which is even when the items are equally long (no mask) and close
  // to even for short masked ones; with a mask over more than 32 K/V tiles the items differ by
  // enough that one CTA per item, placed by the hardware as SMs fall free, measured 3-7 % faster.
  a.n_items = static_cast<int>(static_cast<int64_t>(p->B) * p->Hq * a.n_zblocks);  // range checked above
  const bool chain = a.causal == 0 || cdiv(p->N, 128) <= 32;
  const int n_ctas = chain ? cached_sm_count() : a.n_items;
  L.grid = dim3(static_cast<unsigned>(a.n_items < n_ctas ? a.n_items : n_ctas));
  L.bf16 = p->dtype == B200ATTN_BF16;
  L.dropout = p->dropout_p > 0.f;
  L.stream = static_cast<cudaStream_t>(stream);
  switch (p->D) {
    case 16: return launch_fwd_d16(L);
    case 32: return launch_fwd_d32(L);
    case 64: return launch_fwd_d64(L);
    default: return launch_fwd_d128(L);
  }
}

// ------------------------------------------------------------------ split-KV
namespace b200attn {

// O[row] = sum_s w_s O_s[row] / sum_s w_s with w_s = exp(lse_s - max_s lse_s);
// LSE[row] = max + log(sum_s w_s). One block of 128 threads per (b, h, m) row. The splits'
// log-normalisers are read, reduced to their maximum and turned into weights by all threads in
// parallel (kept in shared memory for the first 1024 splits); then thread d accumulates feature d
// over the splits with independent, unrolled loads. (Three dependent loops over the splits per thread
// made this kernel as long as the partial pass itself on decode shapes.)
template <bool BF16>
__global__ void __launch_bounds__(128)
splitkv_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                       void* __restrict__ o, float* __restrict__ lse, int64_t o_sb,
                       int64_t o_sh, int64_t o_sm, int H, int M, int D, int S) {
  constexpr int CACHED = 1024;
  __shared__ float w_sh[CACHED];
  __shared__ float red[4];
  const int64_t row = blockIdx.x;  // (b*H + h)*M + m
  const int m = static_cast<int>(row % M);
  const int64_t bh = row / M;
  const int h = static_cast<int>(bh % H);
  const int64_t b = bh / H;
  const float* l = part_lse + bh * S * M + m;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  auto block_reduce = [&](float x, bool is_max) -> float {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float y = __shfl_xor_sync(0xffffffffu, x, off);
      x = is_max ? fmaxf(x, y) : x + y;
    }
    __syncthreads();  // (also orders the writes to w_sh before their readers)
    if (lane == 0) red[wid] = x;
    __syncthreads();
    return is_max ? fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])) : (red[0] + red[1]) + (red[2] + red[3]);
  };
  float mx = -INFINITY;
  for (int s = tid; s < S; s += 128) {
    const float x = l[static_cast<int64_t>(s) * M];
    if (s < CACHED) w_sh[s] = x;
    mx = fmaxf(mx, x);
  }
  mx = block_reduce(mx, true);
  float part = 0.f;
  for (int s = tid; s < S; s += 128) {
    const float x = s < CACHED ? w_sh[s] : l[static_cast<int64_t>(s) * M];
    const float w = (mx == -INFINITY) ? 0.f : expf(x - mx);
    if (s < CACHED) w_sh[s] = w;
    part += w;
  }
  const float denom = block_reduce(part, false);
  const int d = tid;
  if (d < D) {
    float acc = 0.f;
    const float* po = part_o + (bh * S * M + m) * D + d;
    const int64_t step = static_cast<int64_t>(M) * D;
#pragma unroll 8
    for (int s = 0; s < S; ++s) {
      const float w = s < CACHED ? w_sh[s]
                                 : ((mx == -INFINITY) ? 0.f : expf(l[static_cast<int64_t>(s) * M] - mx));
      acc += w * po[s * step];
    }
    const float out = denom > 0.f ? acc / denom : 0.f;
    uint16_t* dst = static_cast<uint16_t*>(o) + b * o_sb + h * o_sh + m * o_sm + d;
    if constexpr (BF16) {
      __nv_bfloat16 v = __float2bfloat16_rn(out);
      *dst = *reinterpret_cast<uint16_t*>(&v);
    } else {
      __half v = __float2half_rn(out);
      *dst = *reinterpret_cast<uint16_t*>(&v);
    }
  }
  if (tid == 0) lse[row] = denom > 0.f ? mx + logf(denom) : -INFINITY;
}

static int launch_splitkv_combine(const b200attn_splitkv_params* p, bool bf16, unsigned rows,
                                  cudaStream_t stream) {
  if (bf16) {
    splitkv_combine_kernel<true><<<rows, 128, 0, stream>>>(
        p->part_o, p->part_lse, p->o.ptr, p->lse, p->o.stride[0], p->o.stride[1], p->o.stride[2], p->Hq,
        p->M, p->D, p->num_splits);
  } else {
    splitkv_combine_kernel<false><<<rows, 128, 0, stream>>>(
        p->part_o, p->part_lse, p->o.ptr, p->lse, p->o.stride[0], p->o.stride[1], p->o.stride[2], p->Hq,
        p->M, p->D, p->num_splits);
  }
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

}  // namespace b200attn

namespace b200attn {

// Paged K/V description for the split-KV pass (nullptr = dense k, v of shape [B, Hkv, N, D]). With
// it, p->k and p->v are caches [num_blocks, Hkv, block, D] and p->N is the largest context length.
struct PagedKV {
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* context_lens;
  int block, block_shift, num_blocks;
};

static int run_splitkv(const b200attn_splitkv_params* p, const PagedKV* paged, void* stream_) {
  if (p == nullptr) {
    set_error("fwd_splitkv: null params");
    return B200ATTN_EINVAL;
  }
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->M <= 0 || p->N <= 0 || p->num_splits < 1 ||
      p->Hq % p->Hkv != 0) {
    set_error("fwd_splitkv: bad shape");
    return B200ATTN_EINVAL;
  }
  if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) {
    set_error("fwd_splitkv: head dimension %d not in {16, 32, 64, 128}", p->D);
    return B200ATTN_EINVAL;
  }
  if (p->dtype != B200ATTN_F16 && p->dtype != B200ATTN_BF16) {
    set_error("fwd_splitkv: dtype must be fp16 or bf16");
    return B200ATTN_EINVAL;
  }
  if (p->o.ptr == nullptr || p->lse == nullptr || p->part_o == nullptr || p->part_lse == nullptr) {
    set_error("fwd_splitkv: null output / scratch pointer");
    return B200ATTN_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(p->part_o) % 16 != 0) {
    set_error("fwd_splitkv: part_o must be 16-byte aligned");
    return B200ATTN_EINVAL;
  }
  const int n_blocks = cdiv(p->N, 128);
  const int S = p->num_splits < n_blocks ? p->num_splits : n_blocks;
  if (static_cast<int64_t>(p->B) * p->Hq * cdiv(p->M, 256) * p->num_splits > 2147483647ll) {
    set_error("fwd_splitkv: grid too large");
    return B200ATTN_EINVAL;
  }
  const int64_t rows = static_cast<int64_t>(p->B) * p->Hq * p->M;
  if (rows > 2147483647ll) {
    set_error("fwd_splitkv: too many rows for the combine grid");
    return B200ATTN_EINVAL;
  }
  const bool bf16 = p->dtype == B200ATTN_BF16;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if ((p->Hq / p->Hkv) * static_cast<int64_t>(p->M) <= DECODE_MAX_ROWS) {
    // A few query rows per KV head: register-resident streaming kernel, no tensor-core tile.
    int rc = check_tma_operand(p->q, 2, "q");
    if (rc == B200ATTN_OK) rc = check_tma_operand(p->k, 2, "k");
    if (rc == B200ATTN_OK) rc = check_tma_operand(p->v, 2, "v");
    if (rc != B200ATTN_OK) return rc;
    const b200attn_tensor* ops[3] = {&p->q, &p->k, &p->v};
    const int64_t kv0 = paged ? paged->num_blocks : p->B, kv2 = paged ? paged->block : p->N;
    const int64_t ext[3][3] = {{p->B, p->Hq, p->M}, {kv0, p->Hkv, kv2}, {kv0, p->Hkv, kv2}};
    for (int t = 0; t < 3; ++t) {
      for (int i = 0; i < 3; ++i) {
        if (ext[t][i] > 1 && ops[t]->stride[i] % 8 != 0) {
          set_error("fwd_splitkv: batch / head / row strides of q, k, v must be multiples of 8 elements");
          return B200ATTN_EINVAL;
        }
      }
    }
    if (p->o.stride[3] != 1) {
      set_error("fwd_splitkv: o needs feature stride 1");
      return B200ATTN_EINVAL;
    }
    DecodeArgs d{};
    d.q = static_cast<const uint16_t*>(p->q.ptr);
    d.k = static_cast<const uint16_t*>(p->k.ptr);
    d.v = static_cast<const uint16_t*>(p->v.ptr);
    d.q_sb = p->q.stride[0]; d.q_sh = p->q.stride[1]; d.q_sm = p->q.stride[2];
    d.k_sb = p->k.stride[0]; d.k_sh = p->k.stride[1]; d.k_sn = p->k.stride[2];
    d.v_sb = p->v.stride[0]; d.v_sh = p->v.stride[1]; d.v_sn = p->v.stride[2];
    d.part_o = p->part_o;
    d.part_lse = p->part_lse;
    d.B = p->B; d.Hq = p->Hq; d.Hkv = p->Hkv; d.M = p->M; d.N = p->N;
    d.groups = p->Hq / p->Hkv;
    d.num_splits = p->num_splits;
    d.keys_per_split = cdiv(n_blocks, S) * 128;
    d.causal = p->causal ? 1 : 0;
    d.qk_scale = p->sm_scale * 1.4426950408889634f;
    if (paged) {
      d.block_table = paged->block_table;
      d.bt_stride = paged->bt_stride;
      d.context_lens = paged->context_lens;
      d.block_shift = paged->block_shift;
    }
    if (p->num_splits == 1) {
      d.final_o = static_cast<uint16_t*>(p->o.ptr);
      d.final_lse = p->lse;
      d.o_sb = p->o.stride[0]; d.o_sh = p->o.stride[1]; d.o_sm = p->o.stride[2];
      return launch_decode_partial(d, p->D, bf16, stream);
    }
    rc = launch_decode_partial(d, p->D, bf16, stream);
    if (rc) return rc;
    return launch_splitkv_combine(p, bf16, static_cast<unsigned>(rows), stream);
  }
  // Partial pass: the forward kernel restricted to a K/V tile range per CTA, writing fp32
  // partial O (normalised within the split) and the split's log-normaliser.
  b200attn_fwd_params f{};
  f.q = p->q; f.k = p->k; f.v = p->v;
  f.B = p->B; f.Hq = p->Hq; f.Hkv = p->Hkv; f.M = p->M; f.N = p->N; f.D = p->D;
  FwdLaunch L{};  // zero: every optional mode (packing, paging) is off unless set below
  int rc;
  switch (p->D) {
    case 16: rc = make_fwd_tmaps<16>(&f, L); break;
    case 32: rc = make_fwd_tmaps<32>(&f, L); break;
    case 64: rc = make_fwd_tmaps<64>(&f, L); break;
    default: rc = make_fwd_tmaps<128>(&f, L); break;
  }
  if (rc) return rc;
  if (paged) {
    if (paged->block < 8) {
      set_error("paged attention: cache blocks of fewer than 8 keys need at most 2 query heads per KV head");
      return B200ATTN_EUNSUPPORTED;
    }
    const int chunk = p->D >= 64 ? 64 : p->D;
    const int swz = p->D >= 64 ? 3 : (p->D == 32 ? 2 : 1);
    const int box_rows = paged->block < 128 ? paged->block : 128;
    rc = encode_tmap_4d(&L.tmK, p->k, 2, paged->num_blocks, p->Hkv, paged->block, p->D, chunk, box_rows, swz,
                        "key_cache");
    if (rc) return rc;
    rc = encode_tmap_4d(&L.tmV, p->v, 2, paged->num_blocks, p->Hkv, paged->block, p->D, chunk, box_rows, swz,
                        "value_cache");
    if (rc) return rc;
  }
  // Decode-style shapes with grouped heads: all query heads of a KV head share one 128-row tile, so
  // every K/V tile is fetched once per KV head instead of once per query head.
  const int groups = p->Hq / p->Hkv;
  const bool packed = groups > 1 && groups * p->M <= 128;
  if (packed) {
    const int chunk = p->D >= 64 ? 64 : p->D;
    const int swz = p->D >= 64 ? 3 : (p->D == 32 ? 2 : 1);
    rc = encode_tmap_4d(&L.tmQ, p->q, 2, p->B, p->Hq, p->M, p->D, chunk, p->M, swz, "q", groups);
    if (rc) return rc;
  }
  const int64_t MD = static_cast<int64_t>(p->M) * p->D;
  FwdArgs& a = L.args;
  a.o = p->part_o;
  a.lse = p->part_lse;
  a.o_stride_b = static_cast<int64_t>(p->Hq) * p->num_splits * MD;
  a.o_stride_h = p->num_splits * MD;
  a.o_stride_m = p->D;
  a.o_stride_split = MD;
  a.lse_stride_b = static_cast<int64_t>(p->Hq) * p->num_splits * p->M;
  a.lse_stride_h = static_cast<int64_t>(p->num_splits) * p->M;
  a.lse_stride_split = p->M;
  // With an even split count the packed mode runs two partials per CTA (one per query tile).
  const bool dual = packed && p->num_splits % 2 == 0;
  const int cta_splits = dual ? p->num_splits / 2 : p->num_splits;
  a.num_splits = cta_splits;
  a.tiles_per_split = cdiv(n_blocks, cta_splits < n_blocks ? cta_splits : n_blocks);
  a.pack_heads = packed ? groups : 0;
  a.dual_stream = dual ? 1 : 0;
  if (paged) {
    a.block_table = paged->block_table;
    a.bt_stride = paged->bt_stride;
    a.context_lens = paged->context_lens;
    a.block_shift = paged->block_shift;
  }
  a.ring_stages = p->D == 128 ? FwdSmem<128>::DUAL_STAGES
                  : p->D == 64 ? FwdSmem<64>::DUAL_STAGES
                  : p->D == 32 ? FwdSmem<32>::DUAL_STAGES : FwdSmem<16>::DUAL_STAGES;
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.groups = p->Hq / p->Hkv;
  a.causal = fold_band(p->causal != 0, 0, 0, 0, &a.d_min, &a.d_max) ? 1 : 0;
  a.o_fp32 = 1;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(0.f, 0, 0);
  a.status = p->status;
  a.n_zblocks = cdiv(p->M, 256) * cta_splits;
  a.grid_chunk = packed ? 1 : grid_chunk(a.groups, 4ll * p->N * p->D, a.causal != 0);
  set_item_order(a, packed ? p->Hkv : p->Hq);
  a.o_tma = 0;  // fp32 partial outputs are stored from registers
  const int64_t n_items = static_cast<int64_t>(p->B) * (packed ? p->Hkv : p->Hq) * a.n_zblocks;
  if (n_items > 0x7fffffff) {
    set_error("fwd_splitkv: too many work items");
    return B200ATTN_EUNSUPPORTED;
  }
  a.n_items = static_cast<int>(n_items);  // one CTA per item: the packed, split and paged modes do not chain items
  L.grid = dim3(static_cast<unsigned>(n_items));
  L.bf16 = p->dtype == B200ATTN_BF16;
  L.dropout = false;
  L.stream = static_cast<cudaStream_t>(stream_);
  switch (p->D) {
    case 16: rc = launch_fwd_d16(L); break;
    case 32: rc = launch_fwd_d32(L); break;
    case 64: rc = launch_fwd_d64(L); break;
    default: rc = launch_fwd_d128(L); break;
  }
  if (rc) return rc;
  return launch_splitkv_combine(p, L.bf16, static_cast<unsigned>(rows), L.stream);
}

}  // namespace b200attn

extern "C" size_t b200attn_keep_mask_bytes(int32_t B, int32_t Hq, int32_t M, int32_t N) {
  if (B <= 0 || Hq <= 0 || M <= 0 || N <= 0) return 0;
  return static_cast<size_t>(B) * Hq * ((N + 31) / 32) * M * sizeof(uint32_t);
}

extern "C" int b200attn_fwd_splitkv(const b200attn_splitkv_params* p, void* stream) {
  return b200attn::run_splitkv(p, nullptr, stream);
}

extern "C" int b200attn_paged_attention(const b200attn_paged_params* p, void* stream) {
  using namespace b200attn;
  if (p == nullptr) {
    set_error("paged_attention: null params");
    return B200ATTN_EINVAL;
  }
  if (p->num_seqs <= 0 || p->num_blocks <= 0 || p->block_size <= 0 || p->max_context_len <= 0 ||
      p->block_table == nullptr || p->context_lens == nullptr) {
    set_error("paged_attention: bad shape or null table");
    return B200ATTN_EINVAL;
  }
  if ((p->block_size & (p->block_size - 1)) != 0) {
    set_error("paged_attention: block size %d is not a power of two", p->block_size);
    return B200ATTN_EUNSUPPORTED;
  }
  PagedKV pk{};
  pk.block_table = p->block_table;
  pk.bt_stride = p->block_table_stride;
  pk.context_lens = p->context_lens;
  pk.block = p->block_size;
  pk.num_blocks = p->num_blocks;
  while ((1 << pk.block_shift) < p->block_size) ++pk.block_shift;
  b200attn_splitkv_params sp{};
  sp.q = p->q; sp.k = p->key_cache; sp.v = p->value_cache; sp.o = p->o;
  sp.lse = p->lse; sp.part_o = p->part_o; sp.part_lse = p->part_lse;
  sp.B = p->num_seqs; sp.Hq = p->Hq; sp.Hkv = p->Hkv; sp.M = 1; sp.N = p->max_context_len; sp.D = p->D;
  sp.num_splits = p->num_splits;
  sp.dtype = p->dtype;
  sp.causal = 0;
  sp.sm_scale = p->sm_scale;
  sp.status = p->status;
  return run_splitkv(&sp, &pk, stream);
}

namespace b200attn {
namespace {

// Multiprocessor count of the current device, looked up once per device.
int cached_sm_count() {
  static PerDeviceOnce once;
  static int counts[PerDeviceOnce::MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PerDeviceOnce::MAX_DEVICES) return 148;
  once.run([&]() -> int {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;   // written inside call_once, read only after it has returned
    return B200ATTN_OK;
  });
  return counts[dev];
}

}  // namespace
}  // namespace b200attn

extern "C" int b200attn_splitkv_num_splits(int32_t B, int32_t Hq, int32_t Hkv, int32_t M, int32_t N,
                                           int32_t D, int32_t num_sms) {
  using namespace b200attn;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || M <= 0 || N <= 0 || Hq % Hkv != 0) return 1;
  if (num_sms <= 0) num_sms = cached_sm_count();
  const int groups = Hq / Hkv;
  const int n_blocks = cdiv(N, 128);
  if (static_cast<int64_t>(groups) * M <= DECODE_MAX_ROWS) {
    // Streaming kernel: light CTAs, two or three resident per SM. Choose the smallest split count
    // whose CTAs keep the resident slots at least 90 % as busy as the best count does, with at
    // least 512 keys per split so that the merge stays a small fraction of the work.
    const int64_t units = static_cast<int64_t>(B) * Hkv;
    const int64_t slots = static_cast<int64_t>(num_sms) * decode_resident_ctas(groups * M);
    int cap = cdiv(n_blocks, 4);
    if (cap > 128) cap = 128;
    auto busy = [&](int s) {
      const int64_t ctas = units * s;
      return static_cast<double>(ctas) / static_cast<double>(cdiv(ctas, slots) * slots);
    };
    auto admissible = [&](int s) {
      const int per = cdiv(n_blocks, s);
      return s == 1 || per * s - n_blocks < per;  // no empty split
    };
    double best = 0.0;
    for (int s = 1; s <= cap; ++s)
      if (admissible(s) && busy(s) > best) best = busy(s);
    for (int s = 1; s <= cap; ++s)
      if (admissible(s) && busy(s) >= 0.9 * best) return s;
    return 1;
  }
  // Tensor-core kernel: one CTA per SM. The smallest CTA count per unit whose last wave is at least
  // 85 % as full as the best achievable, with at least four 128-key tiles per CTA. In the packed
  // mode every CTA carries two partials (one per query tile), so the split count is twice that.
  const bool packed = groups > 1 && groups * M <= 128;
  const int64_t ctas = static_cast<int64_t>(B) * (packed ? Hkv : Hq) * cdiv(M, 256);
  const int per_cta = packed ? 2 : 1;
  if (!packed && ctas >= 0.8 * num_sms) return 1;
  int limit = n_blocks / 4;
  if (limit > 128 / per_cta) limit = 128 / per_cta;
  if (limit < 1) return n_blocks >= 2 ? per_cta : 1;
  auto admissible = [&](int s) {
    const int per = cdiv(n_blocks, s);
    return s == 1 || per * s - n_blocks < per;
  };
  auto eff = [&](int s) {
    const double waves = static_cast<double>(ctas) * s / num_sms;
    return waves / ceil(waves);
  };
  double best = 0.0;
  for (int s = 1; s <= limit; ++s)
    if (admissible(s) && eff(s) > best) best = eff(s);
  for (int s = 1; s <= limit; ++s)
    if (admissible(s) && eff(s) >= 0.85 * best) return s * per_cta;
  return 1;
}

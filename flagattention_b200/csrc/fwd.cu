// C entry point of the forward pass: argument validation, TMA descriptors, dispatch on D.
#include "fwd_launch.cuh"

namespace b200attn {

template <int D>
static int make_fwd_tmaps(const b200attn_fwd_params* p, FwdLaunch& L) {
  using Cfg = TileCfg<D>;
  int rc = encode_tmap_4d(&L.tmQ, p->q, 2, p->B, p->Hq, p->M, D, Cfg::CHUNK, Cfg::BLOCK, Cfg::TMA_SWZ, "q");
  if (rc) return rc;
  rc = encode_tmap_4d(&L.tmK, p->k, 2, p->B, p->Hkv, p->N, D, Cfg::CHUNK, Cfg::BLOCK, Cfg::TMA_SWZ, "k");
  if (rc) return rc;
  return encode_tmap_4d(&L.tmV, p->v, 2, p->B, p->Hkv, p->N, D, Cfg::CHUNK, Cfg::BLOCK, Cfg::TMA_SWZ, "v");
}

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

  FwdLaunch L;
  int rc;
  switch (p->D) {
    case 16: rc = make_fwd_tmaps<16>(p, L); break;
    case 32: rc = make_fwd_tmaps<32>(p, L); break;
    case 64: rc = make_fwd_tmaps<64>(p, L); break;
    default: rc = make_fwd_tmaps<128>(p, L); break;
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
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.groups = p->Hq / p->Hkv;
  a.causal = p->causal ? 1 : 0;
  a.o_fp32 = p->o_dtype == B200ATTN_F32 ? 1 : 0;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(p->dropout_p, p->seed, p->offset);
  a.status = p->status;
  a.n_zblocks = cdiv(p->M, 256);
  a.grid_chunk = grid_chunk(a.groups, 4ll * p->N * p->D, a.causal != 0);
  L.grid = dim3(static_cast<unsigned>(static_cast<int64_t>(p->B) * p->Hq * a.n_zblocks));
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
// LSE[row] = max + log(sum_s w_s). One block per (b, h, m) row, one thread per feature.
template <bool BF16>
__global__ void splitkv_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                       void* __restrict__ o, float* __restrict__ lse, int64_t o_sb,
                                       int64_t o_sh, int64_t o_sm, int H, int M, int D, int S) {
  const int64_t row = blockIdx.x;  // (b*H + h)*M + m
  const int m = static_cast<int>(row % M);
  const int64_t bh = row / M;
  const int h = static_cast<int>(bh % H);
  const int64_t b = bh / H;
  const float* l = part_lse + bh * S * M + m;
  float mx = -INFINITY;
  for (int s = 0; s < S; ++s) mx = fmaxf(mx, l[static_cast<int64_t>(s) * M]);
  float denom = 0.f;
  for (int s = 0; s < S; ++s) denom += (mx == -INFINITY) ? 0.f : expf(l[static_cast<int64_t>(s) * M] - mx);
  const int d = threadIdx.x;
  if (d < D) {
    float acc = 0.f;
    for (int s = 0; s < S; ++s) {
      const float w = (mx == -INFINITY) ? 0.f : expf(l[static_cast<int64_t>(s) * M] - mx);
      acc += w * part_o[((bh * S + s) * M + m) * D + d];
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
  if (threadIdx.x == 0) lse[row] = denom > 0.f ? mx + logf(denom) : -INFINITY;
}

}  // namespace b200attn

extern "C" int b200attn_fwd_splitkv(const b200attn_splitkv_params* p, void* stream_) {
  using namespace b200attn;
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
  const int n_blocks = cdiv(p->N, 128);
  const int S = p->num_splits < n_blocks ? p->num_splits : n_blocks;
  if (static_cast<int64_t>(p->B) * p->Hq * cdiv(p->M, 256) * p->num_splits > 2147483647ll) {
    set_error("fwd_splitkv: grid too large");
    return B200ATTN_EINVAL;
  }
  // Partial pass: the forward kernel restricted to a K/V tile range per CTA, writing fp32
  // partial O (normalised within the split) and the split's log-normaliser.
  b200attn_fwd_params f{};
  f.q = p->q; f.k = p->k; f.v = p->v;
  f.B = p->B; f.Hq = p->Hq; f.Hkv = p->Hkv; f.M = p->M; f.N = p->N; f.D = p->D;
  FwdLaunch L;
  int rc;
  switch (p->D) {
    case 16: rc = make_fwd_tmaps<16>(&f, L); break;
    case 32: rc = make_fwd_tmaps<32>(&f, L); break;
    case 64: rc = make_fwd_tmaps<64>(&f, L); break;
    default: rc = make_fwd_tmaps<128>(&f, L); break;
  }
  if (rc) return rc;
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
  a.num_splits = p->num_splits;
  a.tiles_per_split = cdiv(n_blocks, S);
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.groups = p->Hq / p->Hkv;
  a.causal = p->causal ? 1 : 0;
  a.o_fp32 = 1;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(0.f, 0, 0);
  a.status = p->status;
  a.n_zblocks = cdiv(p->M, 256) * p->num_splits;
  a.grid_chunk = grid_chunk(a.groups, 4ll * p->N * p->D, a.causal != 0);
  L.grid = dim3(static_cast<unsigned>(static_cast<int64_t>(p->B) * p->Hq * a.n_zblocks));
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
  const int64_t rows = static_cast<int64_t>(p->B) * p->Hq * p->M;
  if (rows > 2147483647ll) {
    set_error("fwd_splitkv: too many rows for the combine grid");
    return B200ATTN_EINVAL;
  }
  if (L.bf16) {
    splitkv_combine_kernel<true><<<static_cast<unsigned>(rows), 128, 0, L.stream>>>(
        p->part_o, p->part_lse, p->o.ptr, p->lse, p->o.stride[0], p->o.stride[1], p->o.stride[2], p->Hq,
        p->M, p->D, p->num_splits);
  } else {
    splitkv_combine_kernel<false><<<static_cast<unsigned>(rows), 128, 0, L.stream>>>(
        p->part_o, p->part_lse, p->o.ptr, p->lse, p->o.stride[0], p->o.stride[1], p->o.stride[2], p->Hq,
        p->M, p->D, p->num_splits);
  }
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

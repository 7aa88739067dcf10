// C entry points of the backward pass and of total attention: validation, TMA descriptors,
// the preprocess launches and the dispatch on head dimension.
#include <mutex>

#include "bwd_launch.cuh"

namespace b200attn {

static int pad128(int m) { return (m + 127) / 128 * 128; }

static int check_common(const char* who, int B, int Hq, int Hkv, int M, int N, int D, int dtype) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || M <= 0 || N <= 0) {
    set_error("%s: B, Hq, Hkv, M, N must be positive", who);
    return B200ATTN_EINVAL;
  }
  if (Hq % Hkv != 0) {
    set_error("%s: number of heads in q must be a multiple of that in k & v", who);
    return B200ATTN_EINVAL;
  }
  if (D != 16 && D != 32 && D != 64 && D != 128) {
    set_error("%s: head dimension %d not in {16, 32, 64, 128}", who, D);
    return B200ATTN_EINVAL;
  }
  if (dtype != B200ATTN_F16 && dtype != B200ATTN_BF16) {
    set_error("%s: dtype must be fp16 or bf16", who);
    return B200ATTN_EINVAL;
  }
  if (static_cast<int64_t>(B) * Hq * ((M + 127) / 128) > 2147483647ll ||
      static_cast<int64_t>(B) * Hq * ((N + 127) / 128) > 2147483647ll) {
    set_error("%s: problem exceeds the grid limit", who);
    return B200ATTN_EINVAL;
  }
  return B200ATTN_OK;
}

static int check_out(const b200attn_tensor& t, const char* name) {
  if (t.ptr == nullptr || t.stride[3] != 1 || reinterpret_cast<uintptr_t>(t.ptr) % 16 != 0 ||
      (t.stride[0] * 2) % 16 != 0 || (t.stride[1] * 2) % 16 != 0 || (t.stride[2] * 2) % 16 != 0) {
    set_error("%s: needs a non-null 16-byte aligned base, feature stride 1 and 16-byte strides", name);
    return B200ATTN_EINVAL;
  }
  return B200ATTN_OK;
}

template <int D>
static int encode_pair(CUtensorMap* m128, CUtensorMap* m64, const b200attn_tensor& t, int B, int H,
                       int rows, const char* name) {
  using Cfg = TileCfg<D>;
  if (m128 != nullptr) {
    int rc = encode_tmap_4d(m128, t, 2, B, H, rows, D, Cfg::CHUNK, 128, Cfg::TMA_SWZ, name);
    if (rc) return rc;
  }
  if (m64 != nullptr) {
    int rc = encode_tmap_4d(m64, t, 2, B, H, rows, D, Cfg::CHUNK, 64, Cfg::TMA_SWZ, name);
    if (rc) return rc;
  }
  return B200ATTN_OK;
}

static int dispatch(int D, const BwdLaunch& L) {
  switch (D) {
    case 16: return launch_bwd_d16(L);
    case 32: return launch_bwd_d32(L);
    case 64: return launch_bwd_d64(L);
    default: return launch_bwd_d128(L);
  }
}

// FUSED path: dQ = sm_scale * accumulator, rounded to the 16-bit output. 8 elements per thread.
template <bool BF16>
__global__ void dq_convert_kernel(const float* __restrict__ acc, uint16_t* __restrict__ dq, int64_t sb,
                                  int64_t sh, int64_t sr, int Hq, int M, int D, float scale, int64_t n_vec) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    const int d = static_cast<int>(e % D);
    const int64_t row = e / D;
    const int m = static_cast<int>(row % M);
    const int64_t bh = row / M;
    const int h = static_cast<int>(bh % Hq);
    const int64_t b = bh / Hq;
    const float4 x = *reinterpret_cast<const float4*>(acc + e);
    const float4 y = *reinterpret_cast<const float4*>(acc + e + 4);
    uint4 v;
    v.x = pack2<BF16>(x.x * scale, x.y * scale);
    v.y = pack2<BF16>(x.z * scale, x.w * scale);
    v.z = pack2<BF16>(y.x * scale, y.y * scale);
    v.w = pack2<BF16>(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(dq + b * sb + h * sh + static_cast<int64_t>(m) * sr + d) = v;
  }
}

// Whether the backward of this head dimension produces dQ inside the dK/dV pass.
static bool fused_dq(int D, int stages) { return (D == 128 || D == 64) && !(stages & B200ATTN_BWD_STAGE_UNFUSED); }

template <int D>
static int run_bwd(const b200attn_bwd_params* p, float2* stats, cudaStream_t stream, int stages) {
  BwdLaunch kv, qq;
  int rc;
  // MODE_KV: resident K, V (128-row boxes); streamed Q, dO (64-row boxes).
  if ((rc = encode_pair<D>(&kv.tmA1, &qq.tmB1, p->k, p->B, p->Hkv, p->N, "k"))) return rc;
  if ((rc = encode_pair<D>(&kv.tmA2, &qq.tmB2, p->v, p->B, p->Hkv, p->N, "v"))) return rc;
  if ((rc = encode_pair<D>(&qq.tmA1, &kv.tmB1, p->q, p->B, p->Hq, p->M, "q"))) return rc;
  if ((rc = encode_pair<D>(&qq.tmA2, &kv.tmB2, p->d_o, p->B, p->Hq, p->M, "do"))) return rc;

  BwdArgs a{};
  a.stats = stats;
  a.tot = nullptr;
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.Mpad = pad128(p->M);
  a.groups = p->Hq / p->Hkv;
  a.causal = fold_band(p->causal != 0, p->band, p->dist_min, p->dist_max, &a.d_min, &a.d_max) ? 1 : 0;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(p->dropout_p, p->seed, p->offset);
  if (p->dropout_p > 0.f && p->keep_mask != nullptr) {
    a.drop.keep_mask = const_cast<uint32_t*>(p->keep_mask);
    a.drop.mask_words = cdiv(p->N, 32);
  }
  a.status = p->status;

  kv.args = a;
  kv.args.out1 = p->dk.ptr;
  kv.args.out1_sb = p->dk.stride[0]; kv.args.out1_sh = p->dk.stride[1]; kv.args.out1_sr = p->dk.stride[2];
  kv.args.out2 = p->dv.ptr;
  kv.args.out2_sb = p->dv.stride[0]; kv.args.out2_sh = p->dv.stride[1]; kv.args.out2_sr = p->dv.stride[2];
  kv.args.out2_accumulate = p->dv_accumulate != 0 ? 1 : 0;
  // Results leave through TMA stores when the output tensors can be described by tensor maps.
  kv.tmO1 = kv.tmA1; kv.tmO2 = kv.tmA1;
  kv.args.out_tma = (encode_tmap_4d(&kv.tmO1, p->dk, 2, p->B, p->Hkv, p->N, D, TileCfg<D>::CHUNK, 128,
                                    TileCfg<D>::TMA_SWZ, "dk") == B200ATTN_OK &&
                     encode_tmap_4d(&kv.tmO2, p->dv, 2, p->B, p->Hkv, p->N, D, TileCfg<D>::CHUNK, 128,
                                    TileCfg<D>::TMA_SWZ, "dv") == B200ATTN_OK) ? 1 : 0;
  kv.args.n_zblocks = cdiv(p->N, 128);
  kv.args.grid_chunk = grid_chunk(1, 4ll * a.groups * p->M * D, a.causal != 0);
  kv.grid = dim3(static_cast<unsigned>(static_cast<int64_t>(p->B) * p->Hkv * kv.args.n_zblocks));
  kv.bf16 = p->dtype == B200ATTN_BF16;
  kv.dropout = p->dropout_p > 0.f;
  kv.mode = MODE_KV;
  kv.stream = stream;

  qq.args = a;
  qq.args.out1 = p->dq.ptr;
  qq.args.out1_sb = p->dq.stride[0]; qq.args.out1_sh = p->dq.stride[1]; qq.args.out1_sr = p->dq.stride[2];
  qq.args.out2 = nullptr;
  qq.tmO1 = qq.tmA1; qq.tmO2 = qq.tmA1;
  qq.args.out_tma = encode_tmap_4d(&qq.tmO1, p->dq, 2, p->B, p->Hq, p->M, D, TileCfg<D>::CHUNK, 128,
                                   TileCfg<D>::TMA_SWZ, "dq") == B200ATTN_OK ? 1 : 0;
  qq.args.n_zblocks = cdiv(p->M, 128);
  qq.args.grid_chunk = grid_chunk(a.groups, 4ll * p->N * D, a.causal != 0);
  qq.grid = dim3(static_cast<unsigned>(static_cast<int64_t>(p->B) * p->Hq * qq.args.n_zblocks));
  qq.bf16 = kv.bf16;
  qq.dropout = kv.dropout;
  qq.mode = MODE_Q;
  qq.stream = stream;

  if (fused_dq(D, stages)) {
    // One pass for dK, dV and dQ; the fp32 dQ accumulator sits behind the statistics in the workspace.
    float* dq_acc = reinterpret_cast<float*>(stats + static_cast<size_t>(p->B) * p->Hq * a.Mpad);
    const int64_t n_acc = static_cast<int64_t>(p->B) * p->Hq * p->M * D;
    if (stages & B200ATTN_BWD_STAGE_KV) {
      // (cleared by the preprocess when that ran in this call)
      if (!(stages & (B200ATTN_BWD_STAGE_PREP | B200ATTN_BWD_STAGE_ACC_ZEROED)))
        B200ATTN_CUDA_OK(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(n_acc) * sizeof(float), stream));
      kv.fused = true;
      kv.args.dq_acc = dq_acc;
      if ((rc = dispatch(D, kv))) return rc;
    }
    if (stages & B200ATTN_BWD_STAGE_Q) {
      const int64_t n_vec = n_acc / 8;
      const unsigned blocks = static_cast<unsigned>(n_vec / 256 + 1 < 148 * 16 ? n_vec / 256 + 1 : 148 * 16);
      uint16_t* out = static_cast<uint16_t*>(p->dq.ptr);
      if (kv.bf16) {
        dq_convert_kernel<true><<<blocks, 256, 0, stream>>>(dq_acc, out, p->dq.stride[0], p->dq.stride[1],
                                                           p->dq.stride[2], p->Hq, p->M, D, p->sm_scale, n_vec);
      } else {
        dq_convert_kernel<false><<<blocks, 256, 0, stream>>>(dq_acc, out, p->dq.stride[0], p->dq.stride[1],
                                                            p->dq.stride[2], p->Hq, p->M, D, p->sm_scale, n_vec);
      }
      B200ATTN_CUDA_OK(cudaGetLastError());
    }
    return B200ATTN_OK;
  }
  if ((stages & B200ATTN_BWD_STAGE_KV) && (rc = dispatch(D, kv))) return rc;
  if ((stages & B200ATTN_BWD_STAGE_Q) && (rc = dispatch(D, qq))) return rc;
  return B200ATTN_OK;
}

template <int D>
static int run_total(const b200attn_total_params* p, float2* stats, cudaStream_t stream) {
  BwdLaunch L;
  int rc;
  if ((rc = encode_pair<D>(&L.tmA1, nullptr, p->k, p->B, p->Hkv, p->N, "k"))) return rc;
  if ((rc = encode_pair<D>(nullptr, &L.tmB1, p->q, p->B, p->Hq, p->M, "q"))) return rc;
  L.tmA2 = L.tmA1;
  L.tmB2 = L.tmB1;
  L.tmO1 = L.tmA1;
  L.tmO2 = L.tmA1;
  BwdArgs a{};
  a.stats = stats;
  a.tot = p->tot;
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.Mpad = pad128(p->M);
  a.groups = p->Hq / p->Hkv;
  a.causal = fold_band(p->causal != 0, 0, 0, 0, &a.d_min, &a.d_max) ? 1 : 0;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(0.f, 0, 0);
  a.status = p->status;
  L.args = a;
  L.args.n_zblocks = cdiv(p->N, 128);
  L.args.grid_chunk = grid_chunk(1, 2ll * p->M * D, a.causal != 0);
  L.grid = dim3(static_cast<unsigned>(static_cast<int64_t>(p->B) * p->Hq * L.args.n_zblocks));
  L.bf16 = p->dtype == B200ATTN_BF16;
  L.dropout = false;
  L.mode = MODE_TOTAL;
  L.stream = stream;
  return dispatch(D, L);
}

}  // namespace b200attn

extern "C" size_t b200attn_bwd_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t M, int32_t N,
                                               int32_t D) {
  (void)Hkv; (void)N;
  if (B <= 0 || Hq <= 0 || M <= 0) return 0;
  size_t bytes = static_cast<size_t>(B) * Hq * b200attn::pad128(M) * sizeof(float2);
  // D = 128 and 64: fp32 dQ accumulator of the fused pass behind the statistics
  if (D == 128 || D == 64) bytes += static_cast<size_t>(B) * Hq * M * D * sizeof(float);
  return bytes;
}

extern "C" size_t b200attn_total_workspace_bytes(int32_t B, int32_t Hq, int32_t M) {
  if (B <= 0 || Hq <= 0 || M <= 0) return 0;
  return static_cast<size_t>(B) * Hq * b200attn::pad128(M) * sizeof(float2);
}

extern "C" int b200attn_bwd(const b200attn_bwd_params* p, void* stream_) {
  return b200attn_bwd_stages(p, stream_, B200ATTN_BWD_STAGE_ALL);
}

extern "C" int b200attn_bwd_stages(const b200attn_bwd_params* p, void* stream_, int32_t stages) {
  using namespace b200attn;
  if (p == nullptr) {
    set_error("bwd: null params");
    return B200ATTN_EINVAL;
  }
  int rc = check_common("bwd", p->B, p->Hq, p->Hkv, p->M, p->N, p->D, p->dtype);
  if (rc) return rc;
  if (p->o_dtype != p->dtype && p->o_dtype != B200ATTN_F32) {
    set_error("bwd: o_dtype must equal dtype or be fp32");
    return B200ATTN_EINVAL;
  }
  if (p->lse == nullptr || p->delta == nullptr || p->workspace == nullptr) {
    set_error("bwd: lse, delta and workspace must be non-null");
    return B200ATTN_EINVAL;
  }
  if (!(p->dropout_p >= 0.f && p->dropout_p < 1.f)) {
    set_error("bwd: dropout_p must be in [0, 1)");
    return B200ATTN_EINVAL;
  }
  if ((rc = check_out(p->dq, "bwd.dq"))) return rc;
  if ((rc = check_out(p->dk, "bwd.dk"))) return rc;
  if ((rc = check_out(p->dv, "bwd.dv"))) return rc;
  if (reinterpret_cast<uintptr_t>(p->workspace) % 16 != 0) {
    set_error("bwd: workspace must be 16-byte aligned");
    return B200ATTN_EINVAL;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float2* stats = static_cast<float2*>(p->workspace);
  if (stages & B200ATTN_BWD_STAGE_PREP) {
    // When the fused pass follows in the same call, the preprocess also clears its dQ accumulator.
    float* zero_rows = nullptr;
    if (fused_dq(p->D, stages) && (stages & B200ATTN_BWD_STAGE_KV))
      zero_rows = reinterpret_cast<float*>(stats + static_cast<size_t>(p->B) * p->Hq * pad128(p->M));
    rc = bwd_delta(&p->o, p->o_dtype, &p->d_o, p->dtype, p->delta, p->B, p->Hq, p->M, p->D, stream_, zero_rows);
    if (rc) return rc;
    rc = launch_stats(p->lse, p->delta, stats, p->B, p->Hq, p->M, pad128(p->M), stream);
    if (rc) return rc;
  }
  switch (p->D) {
    case 16: return run_bwd<16>(p, stats, stream, stages);
    case 32: return run_bwd<32>(p, stats, stream, stages);
    case 64: return run_bwd<64>(p, stats, stream, stages);
    default: return run_bwd<128>(p, stats, stream, stages);
  }
}

extern "C" int b200attn_total_attention(const b200attn_total_params* p, void* stream_) {
  using namespace b200attn;
  if (p == nullptr) {
    set_error("total_attention: null params");
    return B200ATTN_EINVAL;
  }
  int rc = check_common("total_attention", p->B, p->Hq, p->Hkv, p->M, p->N, p->D, p->dtype);
  if (rc) return rc;
  if (p->lse == nullptr || p->tot == nullptr || p->workspace == nullptr) {
    set_error("total_attention: lse, tot and workspace must be non-null");
    return B200ATTN_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(p->workspace) % 16 != 0) {
    set_error("total_attention: workspace must be 16-byte aligned");
    return B200ATTN_EINVAL;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float2* stats = static_cast<float2*>(p->workspace);
  rc = launch_stats(p->lse, nullptr, stats, p->B, p->Hq, p->M, pad128(p->M), stream);
  if (rc) return rc;
  switch (p->D) {
    case 16: return run_total<16>(p, stats, stream);
    case 32: return run_total<32>(p, stats, stream);
    case 64: return run_total<64>(p, stats, stream);
    default: return run_total<128>(p, stats, stream);
  }
}


// ----------------------------------------------------- total attention without caller scratch
namespace b200attn {

// Per-query statistics scratch that lives inside the library image: B200ATTN_STATIC_STATS_MAX
// (lse*log2e, delta) pairs = 4 MiB, resident on every GPU that loads the library until the
// process exits. In host code this name only stands for the symbol; the device address is
// looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float2 g_static_stats[B200ATTN_STATIC_STATS_MAX];

static std::mutex g_static_stats_mutex;
static float2* g_static_stats_ptr[64] = {};

// Device address of g_static_stats on the current device (looked up on first use).
static int static_stats_ptr(float2** out) {
  int dev = 0;
  B200ATTN_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("total_attention_static: device ordinal %d out of range", dev);
    return B200ATTN_EUNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_static_stats_mutex);
  if (g_static_stats_ptr[dev] == nullptr) {
    float2* ptr = nullptr;
    B200ATTN_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_stats));
    g_static_stats_ptr[dev] = ptr;
  }
  *out = g_static_stats_ptr[dev];
  return B200ATTN_OK;
}

}  // namespace b200attn

extern "C" int b200attn_total_attention_static(const b200attn_total_params* p, void* stream_) {
  using namespace b200attn;
  if (p == nullptr) {
    set_error("total_attention_static: null params");
    return B200ATTN_EINVAL;
  }
  int rc = check_common("total_attention_static", p->B, p->Hq, p->Hkv, p->M, p->N, p->D, p->dtype);
  if (rc) return rc;
  if (p->lse == nullptr || p->tot == nullptr) {
    set_error("total_attention_static: lse and tot must be non-null");
    return B200ATTN_EINVAL;
  }
  const int64_t need = static_cast<int64_t>(p->B) * p->Hq * pad128(p->M);
  if (need > B200ATTN_STATIC_STATS_MAX) {
    set_error("total_attention_static: B*Hq*roundup(M,128) = %lld exceeds the built-in scratch of %d "
              "entries; use b200attn_total_attention with caller scratch",
              static_cast<long long>(need), B200ATTN_STATIC_STATS_MAX);
    return B200ATTN_EUNSUPPORTED;
  }
  float2* stats = nullptr;
  if ((rc = static_stats_ptr(&stats))) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // Every entry the kernel reads ([0, need)) is rewritten here first, so whatever an earlier call
  // left in the array never matters.
  rc = launch_stats(p->lse, nullptr, stats, p->B, p->Hq, p->M, pad128(p->M), stream);
  if (rc) return rc;
  switch (p->D) {
    case 16: return run_total<16>(p, stats, stream);
    case 32: return run_total<32>(p, stats, stream);
    case 64: return run_total<64>(p, stats, stream);
    default: return run_total<128>(p, stats, stream);
  }
}

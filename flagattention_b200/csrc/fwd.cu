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
  if (static_cast<int64_t>(p->B) > 65535 || static_cast<int64_t>(p->Hq) > 65535) {
    set_error("fwd: B and Hq are limited to 65535");
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
  a.B = p->B; a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N;
  a.groups = p->Hq / p->Hkv;
  a.causal = p->causal ? 1 : 0;
  a.o_fp32 = p->o_dtype == B200ATTN_F32 ? 1 : 0;
  a.sm_scale = p->sm_scale;
  a.qk_scale = p->sm_scale * 1.4426950408889634f;
  a.drop = make_dropout_ctx(p->dropout_p, p->seed, p->offset);
  a.status = p->status;
  L.grid = dim3(static_cast<unsigned>(cdiv(p->M, 256)), static_cast<unsigned>(p->Hq),
                static_cast<unsigned>(p->B));
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

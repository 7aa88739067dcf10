// Host launchers of the backward / total-attention kernel family; bwd_d*.cu instantiate one head
// dimension each so the variants compile in parallel.
#pragma once
#include "bwd_kernel.cuh"

namespace b200attn {

struct BwdLaunch {
  CUtensorMap tmA1, tmA2, tmB1, tmB2;
  CUtensorMap tmO1, tmO2;  // outputs, when args.out_tma
  BwdArgs args;
  dim3 grid;
  bool bf16, dropout;
  bool fused = false;  // MODE_KV, D = 128 or 64: dQ produced in the same pass (args.dq_acc)
  int mode;
  cudaStream_t stream;
};

template <int D, bool BF16, bool DROPOUT, int MODE, bool FUSED = false>
int launch_bwd_variant(const BwdLaunch& L) {
  auto kernel = bwd_kernel<D, BF16, DROPOUT, MODE, FUSED>;
  constexpr int smem = BwdSmem<D, MODE, FUSED>::TOTAL;
  static PerDeviceOnce attr_once;  // one per kernel variant
  const int rc = attr_once.run([&]() -> int {
    B200ATTN_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return B200ATTN_OK;
  });
  if (rc) return rc;
  kernel<<<L.grid, BwdSmem<D, MODE, FUSED>::THREADS, smem, L.stream>>>(L.tmA1, L.tmA2, L.tmB1, L.tmB2, L.tmO1, L.tmO2, L.args);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

template <int D>
int launch_bwd_d(const BwdLaunch& L) {
  if (L.mode == MODE_TOTAL) {
    return L.bf16 ? launch_bwd_variant<D, true, false, MODE_TOTAL>(L)
                  : launch_bwd_variant<D, false, false, MODE_TOTAL>(L);
  }
  if constexpr (D == 128 || D == 64) {
    if (L.mode == MODE_KV && L.fused) {
      if (L.bf16) return L.dropout ? launch_bwd_variant<D, true, true, MODE_KV, true>(L) : launch_bwd_variant<D, true, false, MODE_KV, true>(L);
      return L.dropout ? launch_bwd_variant<D, false, true, MODE_KV, true>(L) : launch_bwd_variant<D, false, false, MODE_KV, true>(L);
    }
  }
  if (L.mode == MODE_KV) {
    if (L.bf16) return L.dropout ? launch_bwd_variant<D, true, true, MODE_KV>(L) : launch_bwd_variant<D, true, false, MODE_KV>(L);
    return L.dropout ? launch_bwd_variant<D, false, true, MODE_KV>(L) : launch_bwd_variant<D, false, false, MODE_KV>(L);
  }
  if (L.bf16) return L.dropout ? launch_bwd_variant<D, true, true, MODE_Q>(L) : launch_bwd_variant<D, true, false, MODE_Q>(L);
  return L.dropout ? launch_bwd_variant<D, false, true, MODE_Q>(L) : launch_bwd_variant<D, false, false, MODE_Q>(L);
}

int launch_bwd_d16(const BwdLaunch& L);
int launch_bwd_d32(const BwdLaunch& L);
int launch_bwd_d64(const BwdLaunch& L);
int launch_bwd_d128(const BwdLaunch& L);

}  // namespace b200attn

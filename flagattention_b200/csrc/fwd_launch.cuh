// Host launcher for one head dimension of the forward kernel; each fwd_d*.cu instantiates one D
// so the variants compile in parallel.
#pragma once
#include "fwd_kernel.cuh"

namespace b200attn {

struct FwdLaunch {
  CUtensorMap tmQ, tmK, tmV, tmO;  // tmO only when args.o_tma
  FwdArgs args;
  dim3 grid;
  bool bf16, dropout;
  bool split64 = false;  // D = 128, plain mode: the 64-key softmax pipeline (fwd_kernel's SPLIT64)
  cudaStream_t stream;
};

template <int D, bool BF16, bool DROPOUT, bool SPLIT64 = false>
int launch_fwd_variant(const FwdLaunch& L) {
  auto kernel = fwd_kernel<D, BF16, DROPOUT, SPLIT64>;
  constexpr int smem_max = FwdSmem<D>::TOTAL > FwdSmem<D>::DUAL_TOTAL ? FwdSmem<D>::TOTAL : FwdSmem<D>::DUAL_TOTAL;
  const int smem = L.args.dual_stream ? FwdSmem<D>::DUAL_TOTAL : FwdSmem<D>::TOTAL;
  static PerDeviceOnce attr_once;  // one per kernel variant
  const int rc = attr_once.run([&]() -> int {
    B200ATTN_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max));
    return B200ATTN_OK;
  });
  if (rc) return rc;
  kernel<<<L.grid, 384, smem, L.stream>>>(L.tmQ, L.tmK, L.tmV, L.tmO, L.args);
  B200ATTN_CUDA_OK(cudaGetLastError());
  return B200ATTN_OK;
}

template <int D>
int launch_fwd_d(const FwdLaunch& L) {
  if constexpr (D == 128) {
    if (L.split64) {
      if (L.bf16) return L.dropout ? launch_fwd_variant<D, true, true, true>(L) : launch_fwd_variant<D, true, false, true>(L);
      return L.dropout ? launch_fwd_variant<D, false, true, true>(L) : launch_fwd_variant<D, false, false, true>(L);
    }
  }
  if (L.bf16) {
    return L.dropout ? launch_fwd_variant<D, true, true>(L) : launch_fwd_variant<D, true, false>(L);
  }
  return L.dropout ? launch_fwd_variant<D, false, true>(L) : launch_fwd_variant<D, false, false>(L);
}

int launch_fwd_d16(const FwdLaunch& L);
int launch_fwd_d32(const FwdLaunch& L);
int launch_fwd_d64(const FwdLaunch& L);
int launch_fwd_d128(const FwdLaunch& L);

}  // namespace b200attn

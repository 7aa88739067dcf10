// Entry points whose kernels are not written yet report B200ATTN_EUNSUPPORTED.
#include "common.cuh"
extern "C" {
int b200attn_total_attention(const b200attn_total_params*, void*) {
  b200attn::set_error("total_attention: not implemented");
  return B200ATTN_EUNSUPPORTED;
}
size_t b200attn_bwd_workspace_bytes(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t) { return 0; }
int b200attn_bwd(const b200attn_bwd_params*, void*) {
  b200attn::set_error("bwd: not implemented");
  return B200ATTN_EUNSUPPORTED;
}
int b200attn_fwd_splitkv(const b200attn_splitkv_params*, void*) {
  b200attn::set_error("fwd_splitkv: not implemented");
  return B200ATTN_EUNSUPPORTED;
}
}

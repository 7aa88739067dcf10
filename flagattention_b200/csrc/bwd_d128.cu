// Backward / total-attention kernel instantiations for head dimension 128.
#include "bwd_launch.cuh"
namespace b200attn {
int launch_bwd_d128(const BwdLaunch& L) { return launch_bwd_d<128>(L); }
}  // namespace b200attn

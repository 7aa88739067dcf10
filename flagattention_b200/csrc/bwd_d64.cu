// Backward / total-attention kernel instantiations for head dimension 64.
#include "bwd_launch.cuh"
namespace b200attn {
int launch_bwd_d64(const BwdLaunch& L) { return launch_bwd_d<64>(L); }
}  // namespace b200attn

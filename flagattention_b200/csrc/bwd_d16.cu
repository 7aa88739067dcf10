// Backward / total-attention kernel instantiations for head dimension 16.
#include "bwd_launch.cuh"
namespace b200attn {
int launch_bwd_d16(const BwdLaunch& L) { return launch_bwd_d<16>(L); }
}  // namespace b200attn

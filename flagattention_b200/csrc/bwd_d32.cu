// Backward / total-attention kernel instantiations for head dimension 32.
#include "bwd_launch.cuh"
namespace b200attn {
int launch_bwd_d32(const BwdLaunch& L) { return launch_bwd_d<32>(L); }
}  // namespace b200attn

// Forward kernel instantiations for head dimension 32.
#include "fwd_launch.cuh"
namespace b200attn {
int launch_fwd_d32(const FwdLaunch& L) { return launch_fwd_d<32>(L); }
}  // namespace b200attn

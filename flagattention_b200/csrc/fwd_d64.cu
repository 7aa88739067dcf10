// Forward kernel instantiations for head dimension 64.
#include "fwd_launch.cuh"
namespace b200attn {
int launch_fwd_d64(const FwdLaunch& L) { return launch_fwd_d<64>(L); }
}  // namespace b200attn

// Forward kernel instantiations for head dimension 16.
#include "fwd_launch.cuh"
namespace b200attn {
int launch_fwd_d16(const FwdLaunch& L) { return launch_fwd_d<16>(L); }
}  // namespace b200attn

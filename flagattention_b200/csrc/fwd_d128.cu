// Forward kernel instantiations for head dimension 128.
#include "fwd_launch.cuh"
namespace b200attn {
int launch_fwd_d128(const FwdLaunch& L) { return launch_fwd_d<128>(L); }
}  // namespace b200attn

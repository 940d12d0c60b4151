// Kernel instantiations and dispatch for f32 storage.
#include "dispatch.cuh"

namespace ascan {

int launch_f32(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp) {
    if (variant == VARIANT_PLAIN) return launch_plain<TraitsF32>(kind, reverse, p, pl, st, sp);
    if (variant == VARIANT_SIGMOID) return launch_sigmoid<TraitsF32>(kind, p, pl, st);
    return ASCAN_ERR_UNSUPPORTED;
}

}  // namespace ascan

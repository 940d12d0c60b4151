// Kernel instantiations and dispatch for complex64 storage.
#include "dispatch.cuh"

namespace ascan {

int launch_c64(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp) {
    if (variant == VARIANT_PLAIN) return launch_plain<TraitsC64>(kind, reverse, p, pl, st, sp);
    if (variant == VARIANT_REAL_TOKENS) {
        // stream plan, bulk loader, one row or segment per item, three chunks per lane
        if (pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
        if (kind == ASCAN_KIND_FORWARD) {
            return reverse ? launch_kernel(stream_kernel<TraitsC64, 3, K_SCAN, true, true, false, true>, p, pl, st)
                           : launch_kernel(stream_kernel<TraitsC64, 3, K_SCAN, false, true, false, true>, p, pl, st);
        }
        if (kind == ASCAN_KIND_BACKWARD)
            return launch_kernel(stream_kernel<TraitsC64, 3, K_BWD, true, true, false, true>, p, pl, st);
    }
    return ASCAN_ERR_UNSUPPORTED;
}

}  // namespace ascan

#include "planner.h"

#include <stdlib.h>

namespace ascan {

int dtype_size(int dtype) {
    switch (dtype) {
        case ASCAN_F32: return 4;
        case ASCAN_BF16: return 2;
        case ASCAN_F16: return 2;
        case ASCAN_C64: return 8;
        default: return 0;
    }
}

static int env_int(const char *name, int fallback) {
    const char *v = getenv(name);
    if (!v || !*v) return fallback;
    return atoi(v);
}

static int nin_of(int kind) { return kind == ASCAN_KIND_BACKWARD ? 3 : 2; }
static int nout_of(int kind) {
    return kind == ASCAN_KIND_FORWARD ? 1 : (kind == ASCAN_KIND_BACKWARD ? 2 : 0);
}

// Shared memory one warp of the row-stream kernel needs (must match
// rowstream_warp_smem in rowstream.cuh).
static int warp_smem(int nch, int stages, int kind, bool bulk) {
    const int tb = 32 * nch * 16;
    const int nstg = bulk ? stages : 1;
    const int outbufs = bulk ? 2 : 1;
    return nstg * nin_of(kind) * tb + outbufs * nout_of(kind) * tb + 128;
}

int make_plan(const PlanInput &in, ascan_plan *plan) {
    if (!plan) return ASCAN_ERR_INVALID_ARG;
    const int esize = dtype_size(in.dtype);
    if (esize == 0 || in.kind < 0 || in.kind > ASCAN_KIND_REDUCE_BACKWARD) return ASCAN_ERR_INVALID_ARG;
    if (in.rows < 0 || in.seqlen < 1 || in.sm_count < 1) return ASCAN_ERR_INVALID_ARG;

    ascan_plan pl = {};
    pl.kernel = 0;

    // 16-byte chunks per lane: odd, so that the 16-byte shared accesses of a
    // quarter-warp hit distinct bank groups.  Tuning override: ASCAN_NCH (3 or 5).
    int nch = env_int("ASCAN_NCH", 3);
    if (nch != 3 && nch != 5) nch = 3;
    pl.chunks_per_lane = nch;
    pl.tile_elems = 32 * nch * (16 / esize);

    // Bulk copies need every item to start on a 16-byte boundary and to be a
    // multiple of 16 bytes long: group rows until that holds.
    const int64_t row_bytes_mod = (in.seqlen % 16) * esize % 16;
    int64_t rpi = 1;
    while ((rpi * row_bytes_mod) % 16 != 0) rpi *= 2;          // at most 16
    // ... and the whole matrix must end on a 16-byte boundary (last item may be short)
    const bool total_ok = ((in.rows % 16) * row_bytes_mod) % 16 == 0;
    const bool bulk = in.aligned && total_ok && env_int("ASCAN_FORCE_PLAIN", 0) == 0;
    pl.loader = bulk ? 0 : 1;
    pl.rows_per_item = bulk ? rpi : 1;
    pl.items = (in.rows + pl.rows_per_item - 1) / pl.rows_per_item;

    int stages = env_int("ASCAN_STAGES", in.kind == ASCAN_KIND_BACKWARD ? 3 : 4);
    if (stages < 1) stages = 1;
    if (stages > 8) stages = 8;
    pl.stages = bulk ? stages : 1;

    const int wsm = warp_smem(nch, pl.stages, in.kind, bulk);
    int wpc = kMaxSmemPerCta / wsm;
    if (wpc > kMaxWarpsPerCta) wpc = kMaxWarpsPerCta;
    const int wpc_env = env_int("ASCAN_WPC", 0);
    if (wpc_env > 0 && wpc_env < wpc) wpc = wpc_env;
    if (wpc < 1) return ASCAN_ERR_UNSUPPORTED;

    // One CTA per SM.  With fewer items than warps, spread the items over all SMs
    // before filling the warps of a CTA.
    int64_t grid = in.sm_count;
    if (pl.items < grid * wpc) {
        int64_t w = (pl.items + grid - 1) / grid;
        if (w < 1) w = 1;
        wpc = static_cast<int>(w);
        grid = (pl.items + wpc - 1) / wpc;
        if (grid < 1) grid = 1;
    }
    pl.warps_per_cta = wpc;
    pl.grid = static_cast<int32_t>(grid);
    pl.tiles_per_row = 0;
    pl.smem_bytes = static_cast<uint64_t>(wpc) * wsm;
    pl.workspace_bytes = 0;
    *plan = pl;
    return ASCAN_OK;
}

}  // namespace ascan

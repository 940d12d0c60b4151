// Kernel dispatch for one element type: turns a launch plan into the matching template
// instantiation.  Each element type is compiled in a translation unit of its own
// (inst_*.cu), which exports one plain function declared in launch.h.
#pragma once

#include <cuda_runtime.h>

#include <mutex>
#include <set>
#include <utility>

#include "launch.h"
#include "planner.h"
#include "lookback.cuh"
#include "stream.cuh"
#include "team.cuh"

namespace ascan {

// Opt in to the large dynamic shared-memory carve-out once per (kernel, device).
inline int ensure_smem(const void *fn) {
    static std::mutex mu;
    static std::set<std::pair<const void *, int>> done;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (done.count({fn, dev})) return ASCAN_OK;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemPerCta) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_LAUNCH;
    }
    done.insert({fn, dev});
    return ASCAN_OK;
}

template <class KFN>
static int launch_kernel(KFN kfn, const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    int rc = ensure_smem(reinterpret_cast<const void *>(kfn));
    if (rc != ASCAN_OK) return rc;
    kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
}

// The look-back plan (bulk loader, three chunks per lane, the two scan kinds).
template <class TR, int KIND, bool REVERSE>
static int launch_lookback(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream, const ShardParams *sp) {
    auto kfn = lookback_kernel<TR, 3, KIND, REVERSE>;
    // the planner restates the kernel's shared-memory layout: refuse a plan that disagrees with it
    const int workers = pl.warps_per_cta - 1;
    if (workers < 1 || workers > LB_MAX_WORKERS || pl.stages < 1 || pl.stages > LB_MAX_TILES ||
        pl.smem_bytes != static_cast<uint64_t>(workers) * lb_warp_smem(3, pl.stages, KIND, sizeof(typename TR::V) == 8) + LB_TEAM_BYTES ||
        pl.seg_elems != static_cast<int64_t>(workers) * pl.stages * 32 * 3 * TR::EPC)
        return ASCAN_ERR_UNSUPPORTED;
    int rc = ensure_smem(reinterpret_cast<const void *>(kfn));
    if (rc != ASCAN_OK) return rc;
    ShardParams none = {};
    kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, stream>>>(p, sp ? *sp : none);
    return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
}

// INTERIOR: items that group several rows have row boundaries inside their tiles.
template <class TR, int NCH, int KIND, bool REVERSE, bool BULK>
static int launch_interior(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    // team plans exist for the bulk loader: the scan kinds, and the carry-only kinds of the real dtypes
    if constexpr (BULK && (KIND == K_SCAN || KIND == K_BWD || sizeof(typename TR::V) == 4)) {
        if (pl.kernel == 2) return launch_kernel(team_kernel<TR, NCH, KIND, REVERSE>, p, pl, stream);
    }
    if (pl.kernel != 0) return ASCAN_ERR_UNSUPPORTED;
    return pl.rows_per_item > 1 ? launch_kernel(stream_kernel<TR, NCH, KIND, REVERSE, BULK, true>, p, pl, stream)
                                : launch_kernel(stream_kernel<TR, NCH, KIND, REVERSE, BULK, false>, p, pl, stream);
}

template <class TR, int NCH, int KIND, bool REVERSE>
static int launch_loader(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    return pl.loader == 0 ? launch_interior<TR, NCH, KIND, REVERSE, true>(p, pl, stream)
                          : launch_interior<TR, NCH, KIND, REVERSE, false>(p, pl, stream);
}

template <class TR, int KIND, bool REVERSE>
static int launch_nch(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    switch (pl.chunks_per_lane) {
        case 3: return launch_loader<TR, 3, KIND, REVERSE>(p, pl, stream);
        case 2:
            // two chunks per lane: rows on the tile grid (short power-of-two rows, scan kinds) ...
            if constexpr (KIND == K_SCAN || KIND == K_BWD) {
                if (pl.row_grid) {
                    if (pl.kernel != 0 || pl.loader != 0) return ASCAN_ERR_UNSUPPORTED;
                    return launch_kernel(stream_kernel<TR, 2, KIND, REVERSE, true, false, false, 0, true>, p, pl, stream);
                }
            }
            // ... and the fused backward of the 16-bit dtypes
            if constexpr (KIND == K_BWD && TR::EPC == 8) {
                if (pl.kernel == 0) return launch_loader<TR, 2, KIND, REVERSE>(p, pl, stream);
            }
            return ASCAN_ERR_UNSUPPORTED;
        case 4:
            // four chunks per lane: the forward of the 16-bit dtypes on rows of exactly one 1024-element
            // tile (instead of a full three-chunk tile and a ragged one)
            if constexpr (KIND == K_SCAN && TR::EPC == 8) {
                if (pl.kernel == 0 && pl.loader == 0 && pl.rows_per_item == 1 && !pl.row_grid)
                    return launch_kernel(stream_kernel<TR, 4, KIND, REVERSE, true, false>, p, pl, stream);
            }
            return ASCAN_ERR_UNSUPPORTED;
        default: return ASCAN_ERR_UNSUPPORTED;
    }
}

// The plain kinds of one element type.
template <class TR>
static int launch_plain(int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t stream,
                        const ShardParams *sp) {
    if (pl.kernel == 1) {
        if (pl.loader != 0 || pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
        if (kind == ASCAN_KIND_FORWARD)
            return reverse ? launch_lookback<TR, K_SCAN, true>(p, pl, stream, sp) : launch_lookback<TR, K_SCAN, false>(p, pl, stream, sp);
        if (kind == ASCAN_KIND_BACKWARD) return launch_lookback<TR, K_BWD, true>(p, pl, stream, sp);
        return ASCAN_ERR_UNSUPPORTED;
    }
    if (sp) return ASCAN_ERR_UNSUPPORTED;       // time sharding exists in the look-back plan only
    switch (kind) {
        case ASCAN_KIND_FORWARD:
            return reverse ? launch_nch<TR, K_SCAN, true>(p, pl, stream) : launch_nch<TR, K_SCAN, false>(p, pl, stream);
        case ASCAN_KIND_BACKWARD: return launch_nch<TR, K_BWD, true>(p, pl, stream);
        case ASCAN_KIND_REDUCE_FORWARD: return launch_nch<TR, K_REDUCE, false>(p, pl, stream);
        case ASCAN_KIND_REDUCE_BACKWARD: return launch_nch<TR, K_REDUCE_BWD, true>(p, pl, stream);
        default: return ASCAN_ERR_INVALID_ARG;
    }
}

// Gates given as logits, sigmoid evaluated in the kernel (real dtypes; stream plan, bulk
// loader, one row or segment per item, three chunks per lane).
template <class TR>
static int launch_sigmoid(int kind, const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    if (pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
    if (kind == ASCAN_KIND_FORWARD)
        return launch_kernel(stream_kernel<TR, 3, K_SCAN, false, true, false, false, 1>, p, pl, stream);
    return launch_kernel(stream_kernel<TR, 3, K_BWD, true, true, false, false, 1>, p, pl, stream);
}

}  // namespace ascan

// Chunking / launch planner: pure host arithmetic that turns (rows, T, dtype, kind,
// alignment, workspace, SM count) into a launch plan.  It replaces the reference's
// 12-case sequence-length ladder (warp.cuh:282-380), which accepts powers of two from
// 32 to 65536 only and fixes one CTA per row; this planner accepts any T >= 1.
#pragma once

#include <stdint.h>

#include "../../include/ascan_b200.h"

namespace ascan {

constexpr int kMaxSmemPerCta = 227 * 1024;   // opt-in dynamic shared memory per CTA on sm_100
constexpr int kMaxWarpsPerCta = 12;          // warps per CTA of the kernels for grouped rows and of the backward team kernels
constexpr int kTeamSmemBytes = 384;          // shared memory per team of the team kernel (TEAM_SMEM_BYTES)
constexpr int kCtrlBytes = 256;              // control block at the start of a workspace
constexpr int kCarryRecordBytes = 32;        // per-row carry record behind it

// Tuning values of the planner.  The defaults are the measured optimum; tests and sweeps
// change them through ascan_set_option (the library reads no environment variables).
struct PlanTuning {
    int stages = 2;            // shared-memory stages per warp of the stream and team kernels
    int warps_per_cta = 0;     // 0 = planner's choice; otherwise an upper bound
    int lookback_tiles = 0;    // tiles per segment of the look-back plan; 0 = the default (2)
    int items_per_warp = 4;    // items per warp that grouped short rows aim for (at most two: dealt statically)
    int static_below = 8;      // unsplit rows: at most this many items per warp are dealt round-robin, without tickets
    int disable_plans = 0;     // bit 0: no look-back, bit 1: no team, bit 2: static deal (no tickets), bit 3: plain loader, bit 4: no row grid, bit 5: no four-chunk tiles
};

struct PlanInput {
    int64_t rows;
    int64_t seqlen;
    int dtype;        // ascan_dtype
    int kind;         // ascan_kind
    bool reverse;     // forward kind processed from the row end
    bool aligned;     // every pointer 16-byte aligned
    bool workspace;   // a workspace of the plan's workspace_bytes is available
    bool allow_lookback = true;   // false: never choose the look-back plan (smaller workspace)
    bool allow_team = true;       // false: never choose the team plan
    bool three_chunks = false;    // true: always 3 chunks per lane (variants without a 2-chunk kernel)
    bool force_lookback = false;  // true: the look-back plan whatever the row count (time-sharded calls)
    bool allow_grid = true;       // false: the call has seeds (carry_in, halos), which the row-grid kernels do not take
    int sm_count;
    PlanTuning tune;
};

int dtype_size(int dtype);   // bytes per element, 0 if unknown

constexpr int kLookbackRecordBytes = 32;     // per record of the look-back plan (segments, blocks, super-blocks)

// Records per row of the look-back plan: segments + blocks of 32 + super-blocks of 32 blocks.
uint64_t lookback_records_per_row(int64_t segs);

// Workspace of the chained plans: control block + one carry record per row.
uint64_t workspace_bytes(int64_t rows);

// Fills `plan`; returns an ascan_status.
int make_plan(const PlanInput &in, ascan_plan *plan);

}  // namespace ascan

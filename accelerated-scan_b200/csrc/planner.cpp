#include "planner.h"

#include <initializer_list>

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

uint64_t workspace_bytes(int64_t rows) {
    if (rows < 0) rows = 0;
    return static_cast<uint64_t>(kCtrlBytes) + static_cast<uint64_t>(rows) * kCarryRecordBytes;
}

uint64_t lookback_records_per_row(int64_t segs) {
    const uint64_t s1 = static_cast<uint64_t>((segs + 31) / 32);
    const uint64_t s2 = (s1 + 31) / 32;
    return static_cast<uint64_t>(segs) + s1 + s2;
}

static int nin_of(int kind) { return kind == ASCAN_KIND_BACKWARD ? 3 : 2; }
static int nout_of(int kind) {
    return kind == ASCAN_KIND_FORWARD ? 1 : (kind == ASCAN_KIND_BACKWARD ? 2 : 0);
}

// Shared memory one warp of the stream kernel needs (must match stream_warp_smem
// in stream.cuh).
static int warp_smem(int nch, int stages, int kind, bool bulk) {
    const int tb = 32 * nch * 16;
    const int nstg = bulk ? stages : 1;
    const int outbufs = bulk ? 2 : 1;
    // + halo slot (the stream kernel needs it for the fused backward only; sized for both)
    const int stage = nin_of(kind) * tb + ((kind == ASCAN_KIND_BACKWARD || kind == ASCAN_KIND_REDUCE_BACKWARD) ? 128 : 0);
    return nstg * stage + outbufs * nout_of(kind) * tb + 128;
}

int make_plan(const PlanInput &in, ascan_plan *plan) {
    if (!plan) return ASCAN_ERR_INVALID_ARG;
    const int esize = dtype_size(in.dtype);
    if (esize == 0 || in.kind < 0 || in.kind > ASCAN_KIND_REDUCE_BACKWARD) return ASCAN_ERR_INVALID_ARG;
    if (in.rows < 0 || in.seqlen < 1 || in.sm_count < 1) return ASCAN_ERR_INVALID_ARG;

    ascan_plan pl = {};
    // 16-byte chunks per lane.  3 everywhere (odd: the 16-byte shared accesses of a quarter-warp
    // hit distinct bank groups; 4 loses 15 % to conflicts), except the fused backward of the
    // 16-bit dtypes in the plain stream plan: 24 elements x 3 streams per lane leave too few
    // registers, and 2 chunks (16 elements) measured 2-6 % faster there despite 2-way conflicts.
    const int64_t stream_warps = static_cast<int64_t>(in.sm_count) * kMaxWarpsPerCta;
    // Teams take over below four rows per warp: with few rows per warp the chained stream plan
    // has every segment of a row in flight right behind the one before it, so carries are
    // waited for (fp32, 1800-3000 rows of 65536: stream 6.0-6.3 TB/s, teams of two 6.3-6.5;
    // 4096-6000 rows of 8192: 5.3-5.6 against 5.7-6.3).  Above two rows per warp only for rows
    // long enough to be split (whole short rows run better one warp each); from 8000 rows on
    // the stream plan is ahead again.
    const int64_t team_rows = 4 * stream_warps;
    // Short rows on the tile grid: with two chunks per lane (512 16-bit, 256 fp32, 128 complex64
    // elements per tile) every power-of-two row length from one lane's elements up to the tile
    // divides the tile, so items can group whole rows without any per-element row-boundary
    // arithmetic (GRID kernels; measured at 12288 rows of bf16: 128 steps 14.3 -> 10.2 us forward,
    // 18.4 -> 12.3 us backward; 256 steps 20.5 -> 14.3 / 30.7 -> 18.4 us).  Rows longer than a tile
    // keep three chunks per lane: the two-chunk forward kernel pays its per-tile costs on a third
    // fewer bytes (bf16, 2048 to 16384 steps: 14-19 % slower).  Not where teams apply.
    const int64_t k2 = 2 * (16 / esize), te2 = 32 * k2, te3 = 32 * 3 * (16 / esize);
    const bool scan_kind_early = in.kind == ASCAN_KIND_FORWARD || in.kind == ASCAN_KIND_BACKWARD;
    const bool row_grid = in.allow_grid && scan_kind_early && in.aligned && !in.three_chunks && in.rows >= team_rows &&
                      in.seqlen % k2 == 0 && te2 % in.seqlen == 0 && (in.tune.disable_plans & (8 | 16)) == 0;
    // Forward of the 16-bit dtypes on rows of exactly 1024 steps: four chunks per lane, so that a row
    // is one tile instead of a full one and a ragged one of a third ((8,1536,1024) bf16 forward 2836 ->
    // 3356 GB/s).  Longer rows keep three chunks: there the four-way conflicts of the 16-byte shared
    // accesses cost more than the ragged tile (2048 steps 4608 -> 4096, 4096 steps 5671 -> 4757 GB/s).
    const int64_t te4 = 32 * 4 * (16 / esize);
    const bool four = !row_grid && in.kind == ASCAN_KIND_FORWARD && esize == 2 && in.aligned && !in.three_chunks &&
                      in.allow_grid && in.rows >= team_rows && in.seqlen == te4 &&
                      (in.tune.disable_plans & (8 | 32)) == 0;
    const int nch = four ? 4
                         : ((row_grid || (in.kind == ASCAN_KIND_BACKWARD && esize == 2 && in.rows >= team_rows && !in.three_chunks))
                                ? 2
                                : 3);
    pl.row_grid = row_grid ? 1 : 0;
    const int64_t te = 32 * nch * (16 / esize);
    // tickets and split-row item numbers are 32-bit
    const bool use_ws = in.workspace && (in.tune.disable_plans & 4) == 0 && in.rows < (1ll << 30) &&
                        in.rows * ((in.seqlen + te - 1) / te) < (1ll << 31);
    pl.dynamic = use_ws ? 1 : 0;

    pl.chunks_per_lane = nch;
    pl.tile_elems = static_cast<int32_t>(te);

    // Bulk copies need every item to start on a 16-byte boundary and to be a
    // multiple of 16 bytes long: group `align_rows` rows until that holds ...
    const int64_t row_bytes_mod = ((in.seqlen % 16) * esize) % 16;
    int64_t align_rows = 1;
    while ((align_rows * row_bytes_mod) % 16 != 0) align_rows *= 2;          // at most 16
    // ... and the whole matrix must end on a 16-byte boundary (the last item may be short)
    const bool total_ok = ((in.rows % 16) * row_bytes_mod) % 16 == 0;
    const bool bulk = in.aligned && total_ok && (in.tune.disable_plans & 8) == 0;
    pl.loader = bulk ? 0 : 1;

    // Item size.  Long rows are split into segments (needs the workspace for the per-row
    // carry records and, with the bulk loader, rows that start 16-byte aligned): coarse
    // segments of `seg_tiles` tiles, then, in the part of every row that is processed last,
    // fine segments of `fine_tiles` tiles, so that the warps run out of work within one
    // small item of each other.  The fine part holds about one coarse item per warp.
    // Short rows are grouped into items of about four per warp, at most `seg_tiles` tiles.
    int seg_tiles = 16;
    int fine_tiles = 4;
    if (row_grid) seg_tiles = 32;
    const int64_t max_warps = static_cast<int64_t>(in.sm_count) * kMaxWarpsPerCta;
    const int64_t tiles_row = (in.seqlen + te - 1) / te;
    const bool reverse_order = in.kind == ASCAN_KIND_BACKWARD || in.kind == ASCAN_KIND_REDUCE_BACKWARD || in.reverse;
    const bool can_split = use_ws && (!bulk || align_rows == 1);
    // Clearly fewer rows than SMs: a whole CTA per row (the team plan below) would leave SMs
    // idle.  The look-back plan cuts rows into segments of a few tiles that a warp keeps in
    // shared memory; segments of one row are scanned concurrently by warps of many CTAs, each
    // taking its incoming state from the aggregates of the segments before it.  Also the plan
    // of time-sharded calls, whatever their row count.
    const bool scan_kind = in.kind == ASCAN_KIND_FORWARD || in.kind == ASCAN_KIND_BACKWARD;
    {
        int lb_tiles = in.tune.lookback_tiles > 0 ? in.tune.lookback_tiles : 2;
        if (lb_tiles > 8) lb_tiles = 8;
        // The fused backward: below three rows per four SMs (measured on 148 SMs, fp32, 268 MB per
        // tensor: at 128 rows teams of 12 warps run at 5.9 TB/s, look-back at 5.5).  The forward:
        // below three rows per two SMs (teams / look-back at 128 rows 4.2 / 5.4 TB/s, 147 rows
        // 4.7 / 5.4, 200 rows 5.2 / 5.4, 296 rows 5.9 / 5.4; bf16 the same way).
        const int64_t lookback_rows = in.kind == ASCAN_KIND_FORWARD ? in.sm_count * 3 / 2 : in.sm_count * 3 / 4;
        const int64_t te3 = 32 * 3 * (16 / esize);
        const int64_t tiles_row3 = (in.seqlen + te3 - 1) / te3;
        const bool possible = can_split && bulk && scan_kind && in.rows > 0 && (in.tune.disable_plans & 1) == 0;
        const bool wanted = in.force_lookback || (in.allow_lookback && in.rows < lookback_rows && tiles_row3 >= 2 * lb_tiles);
        if (possible && wanted && in.rows * ((tiles_row3 + lb_tiles - 1) / lb_tiles) < (1ll << 31)) {
            // A CTA is a team of worker warps plus one bookkeeper.  Per worker: its lb_tiles tiles
            // of two resident segments (lb_warp_smem in lookback.cuh); 3072 bytes for the team.
            const int stage = nin_of(in.kind) * 32 * 3 * 16 + (in.kind == ASCAN_KIND_BACKWARD ? 128 : 0);
            const int staging = in.kind == ASCAN_KIND_BACKWARD ? 0 : 32 * 3 * 16;
            // prefix maps: two values of the compute type per stage and lane
            const int prefix = in.dtype != ASCAN_C64 ? 8 : 16;
            const int wsm = 2 * lb_tiles * stage + staging + 128 + 2 * lb_tiles * 32 * prefix;
            int64_t workers = (kMaxSmemPerCta - 3072) / wsm;
            if (workers > 15) workers = 15;
            if (in.tune.warps_per_cta > 1 && in.tune.warps_per_cta - 1 < workers) workers = in.tune.warps_per_cta - 1;
            if (workers < 1) return ASCAN_ERR_UNSUPPORTED;
            // a segment is one part (lb_tiles tiles) per worker; rows are cut into segments of equal
            // size, and short rows get no more workers than they have parts
            const int64_t parts_row = (tiles_row3 + lb_tiles - 1) / lb_tiles;
            const int64_t segs = (parts_row + workers - 1) / workers;
            workers = (parts_row + segs - 1) / segs;
            const int wpc = static_cast<int>(workers) + 1;
            pl.kernel = 1;
            pl.loader = 0;
            pl.chunks_per_lane = 3;
            pl.tile_elems = static_cast<int32_t>(te3);
            pl.stages = lb_tiles;
            pl.dynamic = 1;
            pl.team_size = 1;
            pl.rows_per_item = 1;
            pl.row_groups = in.rows;
            pl.seg_elems = workers * lb_tiles * te3;
            pl.fine_elems = pl.seg_elems;
            pl.coarse_segs = 0;
            pl.fine_segs = segs;
            pl.segs_per_row = segs;
            pl.items = in.rows * segs;
            int64_t grid = in.sm_count;
            if (pl.items < grid) grid = pl.items;
            pl.warps_per_cta = wpc;
            pl.grid = static_cast<int32_t>(grid);
            pl.smem_bytes = static_cast<uint64_t>(workers) * wsm + 3072;
            pl.workspace_bytes = static_cast<uint64_t>(kCtrlBytes) +
                                 static_cast<uint64_t>(in.rows) * lookback_records_per_row(segs) * kLookbackRecordBytes;
            *plan = pl;
            return ASCAN_OK;
        }
        if (in.force_lookback) return ASCAN_ERR_UNSUPPORTED;
    }
    // Fewer rows than warps, but too many for look-back to pay: teams of G warps share an
    // item, so that all warps work although only rows/G... teams can be busy at once.  G is
    // the smallest divisor of the warps per CTA with (warps / G) <= rows.
    int team = 1;
    int team_wpc = kMaxWarpsPerCta;      // warps per CTA of a team plan
    const bool team_kind = scan_kind || in.dtype != ASCAN_C64;     // carry-only kinds: real dtypes
    if (can_split && bulk && team_kind && in.allow_team && in.rows > 0 && in.rows < team_rows &&
        (in.tune.disable_plans & 2) == 0) {
        // The forward kinds need fewer registers and less shared memory per warp, so 16 warps
        // fit in a CTA (teams of 2, 4, 8 or 16): with 12 the forward is bound by the time a warp
        // needs per tile (4.4-5.4 TB/s at 150-800 rows), with 16 by HBM.
        const bool wide_kind = in.kind == ASCAN_KIND_FORWARD || in.kind == ASCAN_KIND_REDUCE_FORWARD;
        if (wide_kind) {
            const int64_t want16 = (static_cast<int64_t>(in.sm_count) * 16 + in.rows - 1) / in.rows;
            for (int cand : {2, 4, 8, 16}) {
                if (cand >= want16) {
                    if (tiles_row >= 2 * cand) {       // else: rows too short for so wide a team
                        team = cand;
                        team_wpc = 16;
                    }
                    break;
                }
            }
        }
        if (team == 1) {
            const int64_t want = (max_warps + in.rows - 1) / in.rows;
            for (int cand : {2, 3, 4, 6, 12}) {
                if (cand >= want) {
                    team = cand;
                    break;
                }
            }
            if (team == 1) team = 12;
        }
        // eight tiles per warp and coarse item, four per fine item: the team's barrier and
        // ticket hand-over per item cost about a tile (4 and 2 per warp measured 10 % slower
        // for teams of 16)
        const int seg_tiles_single = seg_tiles, fine_tiles_single = fine_tiles;
        if (seg_tiles < 8 * team) seg_tiles = 8 * team;
        if (fine_tiles < 4 * team) fine_tiles = 4 * team;
        if (tiles_row < 2 * team) team = 1;           // rows too short to share
        if (in.rows >= 2 * stream_warps && tiles_row < 2 * fine_tiles) team = 1;   // whole short rows: one warp each
        if (team == 1) {
            seg_tiles = seg_tiles_single;
            fine_tiles = fine_tiles_single;
        }
    }
    const int64_t workers = static_cast<int64_t>(in.sm_count) * team_wpc / team;
    const int64_t split_min = team > 1 ? 2 * fine_tiles : 32;
    if (can_split && !row_grid && tiles_row >= split_min && tiles_row >= 2 * fine_tiles) {
        int64_t fine_region = (static_cast<int64_t>(seg_tiles) * workers + in.rows - 1) / (in.rows > 0 ? in.rows : 1);
        fine_region = (fine_region + fine_tiles - 1) / fine_tiles * fine_tiles;      // tiles, multiple of a fine item
        if (fine_region > tiles_row) fine_region = tiles_row;
        int64_t coarse_tiles = tiles_row - fine_region;                               // may be 0
        int64_t seg_c = seg_tiles;
        if (coarse_tiles < seg_c) seg_c = coarse_tiles;
        // carry tags hold the segment number in 15 bits
        while (seg_c > 0 && coarse_tiles / seg_c + (tiles_row + fine_tiles - 1) / fine_tiles > 30000) {
            seg_c *= 2;
            fine_tiles *= 2;
        }
        pl.rows_per_item = 1;
        pl.row_groups = in.rows;
        pl.fine_elems = fine_tiles * te;
        if (seg_c <= 0) {
            pl.seg_elems = pl.fine_elems;
            pl.coarse_segs = 0;
            pl.fine_segs = (in.seqlen + pl.fine_elems - 1) / pl.fine_elems;
        } else if (!reverse_order) {
            // coarse segments first, all full; the fine part takes the rest of the row
            pl.seg_elems = seg_c * te;
            pl.coarse_segs = coarse_tiles / seg_c;
            const int64_t rest = in.seqlen - pl.coarse_segs * pl.seg_elems;
            pl.fine_segs = (rest + pl.fine_elems - 1) / pl.fine_elems;
        } else {
            // processed from the row end: the fine part is the start of the row, all full
            pl.seg_elems = seg_c * te;
            pl.fine_segs = fine_region / fine_tiles;
            const int64_t rest = in.seqlen - pl.fine_segs * pl.fine_elems;
            pl.coarse_segs = (rest + pl.seg_elems - 1) / pl.seg_elems;
        }
        pl.segs_per_row = pl.coarse_segs + pl.fine_segs;
    } else {
        const int64_t total_tiles = (in.rows * in.seqlen + te - 1) / te;
        // about four items per warp; a row-grid problem of at most 16 tiles per warp is dealt as one
        // item per warp (a launch of some 10 us gains nothing from balancing, and saves the tickets)
        int ipw = in.tune.items_per_warp > 0 ? in.tune.items_per_warp : 4;
        if (row_grid && total_tiles <= 16 * max_warps) ipw = 1;
        int64_t fit = total_tiles / (ipw * max_warps);
        if (fit < 1) fit = 1;
        if (fit < seg_tiles) seg_tiles = static_cast<int>(fit);
        int64_t rpi = (seg_tiles * te) / in.seqlen;
        if (rpi < 1) rpi = 1;
        // Rows of a tile or more are never grouped: the kernels for grouped rows find the row
        // boundaries per element and run at a third to a half of the one-row-per-item kernels'
        // rate ((32,1536,L) bf16 forward / backward GB/s, grouped -> one row per item: L = 1024
        // 2303 / 2409 -> 3511 / 4962, 2048 3429 / 3536 -> 5362 / 5922, 4096 4537 / 4499 -> 6411 / 6467).
        if (in.seqlen >= te && !row_grid) rpi = 1;
        if (bulk) rpi = (rpi + align_rows - 1) / align_rows * align_rows;
        if (row_grid && te > in.seqlen) {
            // whole tiles per item: a multiple of the rows of one tile
            const int64_t per_tile = te / in.seqlen;
            rpi = (rpi + per_tile - 1) / per_tile * per_tile;
        }
        pl.rows_per_item = rpi;
        pl.row_groups = (in.rows + rpi - 1) / rpi;
        pl.seg_elems = in.seqlen;
        pl.fine_elems = in.seqlen;
        pl.coarse_segs = 1;
        pl.fine_segs = 0;
        pl.segs_per_row = 1;
    }
    pl.items = pl.row_groups * pl.segs_per_row;

    int stages = in.tune.stages;
    if (stages < 1) stages = 1;
    if (stages > 8) stages = 8;
    pl.stages = bulk ? stages : 1;

    // (the team kernel's backward stage has the same 128-byte halo slot, so the sizes agree)
    const int wsm = warp_smem(nch, pl.stages, in.kind, bulk);
    int wpc = (kMaxSmemPerCta - (team > 1 ? team_wpc / team * kTeamSmemBytes : 0)) / wsm;
    // the stream kernels are compiled for 16 warps per CTA (14 for the fused backward, which
    // needs more registers); 14 measured best (more warps hide more of a tile's dependent
    // latency, 15-16 leave too few registers and shared memory per warp)
    const int wpc_cap = team > 1 ? team_wpc : ((in.kind == ASCAN_KIND_BACKWARD && nch > 2) ? 14 : 16);
    if (wpc > wpc_cap) wpc = wpc_cap;
    const int wpc_env = in.tune.warps_per_cta;
    if (wpc_env > 0 && wpc_env < wpc) wpc = wpc_env;
    else if (wpc > 14) wpc = 14;
    if (wpc < 1) return ASCAN_ERR_UNSUPPORTED;
    // kernels for items that group rows keep more state per thread: compiled for 12 warps
    if (pl.rows_per_item > 1 && !row_grid && wpc > kMaxWarpsPerCta) wpc = kMaxWarpsPerCta;

    // One persistent CTA per SM.  With fewer items than warps, spread the items over
    // all SMs before filling the warps of a CTA.
    int64_t grid = in.sm_count;
    if (pl.items < grid * wpc) {
        int64_t w = (pl.items + grid - 1) / grid;
        if (w < 1) w = 1;
        wpc = static_cast<int>(w);
        grid = (pl.items + wpc - 1) / wpc;
        if (grid < 1) grid = 1;
    }
    if (team > 1) {
        // whole teams only, one persistent CTA per SM
        if (pl.rows_per_item != 1 ||
            static_cast<int64_t>(team_wpc) * wsm + team_wpc / team * kTeamSmemBytes > kMaxSmemPerCta) {
            team = 1;              // does not fit (deep rings): the chained stream kernel, as planned above
        } else {
            wpc = team_wpc;
            grid = in.sm_count;
        }
    }
    // A problem of a few items per warp gains less from tickets than they cost (an atomic, its
    // broadcast and the exit counter per item): deal round-robin.  (8,1536,L) bf16 at about six
    // one-row items per warp, forward / backward GB/s: L = 1024 2458 / 3614 -> 2836 / 4389, 2048
    // 4092 / 4726 -> 4608 / 5343, 4096 5085 / 5715 -> 5671 / 5996, 8192 6142 / 5994 -> 6279 / 5994.
    // Only for launches of up to 48 three-chunk tiles per warp (some 100 us): beyond that the tickets' balancing
    // wins again (fp32 (8,1536,4096) backward 6222 -> 5990, (8,1536,8192) 6205 -> 5915 without them).
    const int64_t bytes_all = in.rows * in.seqlen * esize;               // per stream
    if (pl.dynamic && team == 1 && pl.segs_per_row == 1 && bytes_all <= 48 * 1536 * grid * wpc &&
        pl.items <= static_cast<int64_t>(in.tune.static_below > 0 ? in.tune.static_below : 0) * grid * wpc) {
        pl.dynamic = 0;
    }
    pl.team_size = team;
    pl.warps_per_cta = wpc;
    pl.grid = static_cast<int32_t>(grid);
    pl.smem_bytes = static_cast<uint64_t>(wpc) * wsm + (team > 1 ? static_cast<uint64_t>(wpc / team) * kTeamSmemBytes : 0);
    pl.kernel = team > 1 ? 2 : 0;
    // carry records are only needed when rows are split; the control block (ticket, status) always
    pl.workspace_bytes = (!use_ws || !pl.dynamic) ? 0 : (pl.segs_per_row > 1 ? workspace_bytes(in.rows) : kCtrlBytes);
    *plan = pl;
    return ASCAN_OK;
}

}  // namespace ascan

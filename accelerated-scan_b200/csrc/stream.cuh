// Warp-stream scan kernel.
//
// Work decomposition
//   * The rows x T matrix is cut into ITEMS.  Short rows are grouped (an item is a few
//     whole rows); longer rows are split into segments (an item is one segment of one
//     row): coarse segments first and, in the part of each row that is processed last,
//     fine segments, so that the warps run out of work within a small item of each
//     other.  Items are numbered segment-major: all first segments, then all second
//     segments, ... in processing order (the reverse directions start from the row end).
//   * Persistent warps draw item numbers from a global ticket counter, so SMs that
//     stream faster take more items and all SMs finish together.  Without a workspace
//     the items are dealt round-robin instead and rows are never split.
//   * The state leaving a segment is published in a per-row record of self-tagged
//     64-bit words; the warp that draws the next segment of that row reads it.  Because
//     of the segment-major order the record is normally written long before it is
//     needed; if it is not there yet the reader polls with a bound, records a status
//     bit on expiry and carries on, so the kernel always terminates.
//
// Inside an item
//   * An item is a flat range of the matrix; fixed-size tiles of it move through the
//     warp's own shared-memory ring.
//   * Bulk loader: one lane issues 1-D bulk asynchronous copies (global -> shared,
//     mbarrier completion, no multicast) up to `stages` tiles ahead, across item
//     boundaries; results leave through bulk asynchronous stores from a
//     double-buffered staging area.  Each lane owns NCH consecutive 16-byte chunks of a
//     tile; with NCH odd the 16-byte shared accesses of a quarter-warp fall in
//     distinct bank groups.
//   * Plain loader: the same arithmetic fed by element-wise loads/stores, for data
//     that is not 16-byte aligned.
//   * Per tile: sequential pass over the lane's elements for the lane aggregate
//     (A, B) of x -> A*x + B, Kogge-Stone combine across lanes by shuffles, then a
//     second sequential pass from the lane's incoming state.  The state crossing
//     tiles is one register per warp; there is no block-level barrier in the loop.
//   * Row boundaries.  When an item is one row or one segment (INTERIOR = false) a row
//     can only start where the item starts and end where it ends, so the incoming
//     state is simply the warp's running state at the first tile, and only the ragged
//     last tile of a row needs per-element masking.  When an item groups several short
//     rows (INTERIOR = true) row starts fall inside tiles; the gate of a row's first
//     processed element is forced to zero there, which resets the running state.
//
// Kinds: forward scan (optionally reversed), fused backward (reverse scan over the
// gates shifted by one step plus the d_gates epilogue; shifted operands come from
// neighbouring lanes by shuffle, tile halos from one scalar load), and the two
// carry-only reductions used by time-sharded callers.
#pragma once

#include "common.cuh"

namespace ascan {

enum : int { K_SCAN = 0, K_BWD = 1, K_REDUCE = 2, K_REDUCE_BWD = 3 };

// Control words at the start of the workspace (uint32 each).  Words 4-5 hold an optional
// 64-bit device-accessible address (for instance mapped pinned host memory) of a second
// status word: a kernel that records status bits also ORs them in there, so the host can
// notice a failure by reading its own memory, without a copy or a synchronisation.
enum : int { CTRL_STATUS = 0, CTRL_TICKET = 1, CTRL_DONE = 2, CTRL_EPOCH = 3, CTRL_SINK = 4 };
constexpr int EPOCH_SHIFT = 15;        // a carry tag is (epoch << 15) | segment number
constexpr int CTRL_BYTES = 256;        // control block, then one carry record per row
constexpr int CARRY_RECORD_BYTES = 32;

struct StreamParams {
    const void *in0;         // gates
    const void *in1;         // tokens (scan, reduce) or grad_out (backward kinds)
    const void *in2;         // saved states (backward only)
    void *out0;              // out (scan) or d_tokens (backward)
    void *out1;              // d_gates (backward)
    const void *carry_in;    // rows values of V, or null
    const void *halo_gate;   // rows values of V, or null (backward kinds)
    const void *halo_state;  // rows values of V, or null (backward)
    void *carry_out;         // rows x 2 values of V (reduce kinds)
    int64_t rows, T;
    int64_t rows_per_item;   // rows grouped into one item when rows are not split
    int64_t row_groups;      // ceil(rows / rows_per_item)
    int64_t seg_elems;       // steps per coarse segment (multiple of the tile) when rows are split
    int64_t fine_elems;      // steps per fine segment (multiple of the tile)
    int64_t coarse_segs;     // coarse segments per row
    int64_t fine_segs;       // fine segments per row, processed after the coarse ones
    int64_t segs_per_row;    // coarse_segs + fine_segs; 1 = rows are not split
    int64_t items;           // row_groups * segs_per_row
    uint32_t *ctrl;          // control words, or null (static dealing, no status)
    unsigned char *records;  // per-row carry records (segs_per_row > 1)
    int32_t stages;          // shared-memory stages per warp (bulk loader)
    int32_t team_size;       // warps per team (team kernel only)
    int32_t test_drop_carry; // test hook: drop one carry hand-over (see the item epilogue); 0 in production
    uint32_t epoch_mask;     // the launch epoch is taken modulo epoch_mask + 1 (2^17 - 1 unless a test lowers it)
    uint64_t scratch_bytes;  // bytes of records behind the control block (wiped when the epoch wraps)
};

// Records status bits in the workspace and, when the caller registered one, in the
// second status word (control words 4-5; typically mapped host memory, hence a plain
// system-scope store: any non-zero value means "a wait expired").
__device__ __forceinline__ void report_status(uint32_t *ctrl, uint32_t bits) {
    atomicOr(ctrl + CTRL_STATUS, bits);
    const unsigned long long sink = *reinterpret_cast<volatile unsigned long long *>(ctrl + CTRL_SINK);
    if (sink) {
        *reinterpret_cast<volatile uint32_t *>(sink) = bits;
        __threadfence_system();
    }
}

// Called by every warp (all lanes) as it leaves a kernel that runs on a workspace.  The
// last warp out rearms the ticket and the exit counter for the next launch and opens a
// new epoch.  When the epoch wraps, tags of old launches would repeat, so that warp first
// zeroes every record behind the control block (all other warps are done with them).
__device__ __forceinline__ void leave_kernel(const StreamParams &p, int64_t W, uint32_t status_bits, int lane) {
    uint32_t last = 0;
    if (lane == 0) {
        if (status_bits) report_status(p.ctrl, status_bits);
        __threadfence();
        last = (atomicAdd(p.ctrl + CTRL_DONE, 1u) == static_cast<uint32_t>(W - 1)) ? 1u : 0u;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    const uint32_t next = (*reinterpret_cast<volatile uint32_t *>(p.ctrl + CTRL_EPOCH) + 1u) & p.epoch_mask;
    if (next == 0) {
        uint4 *rec = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(p.ctrl) + CTRL_BYTES);
        const uint64_t n16 = p.scratch_bytes / 16;
        for (uint64_t i = lane; i < n16; i += 32) rec[i] = make_uint4(0, 0, 0, 0);
        __threadfence();
        __syncwarp();
    }
    if (lane == 0) {
        p.ctrl[CTRL_TICKET] = 0;
        p.ctrl[CTRL_DONE] = 0;
        p.ctrl[CTRL_EPOCH] = next;
        __threadfence();
    }
}

__host__ __device__ constexpr int stream_nin(int kind) { return kind == K_BWD ? 3 : 2; }
__host__ __device__ constexpr int stream_nout(int kind) { return kind == K_SCAN ? 1 : (kind == K_BWD ? 2 : 0); }
// Bytes of one ring stage: the tiles of the input streams and, for the fused backward, a
// 128-byte slot whose first 16 bytes receive the chunk of saved states just below the tile
// (its last element is the state before the tile's first step).
__host__ __device__ constexpr int stream_stage_bytes(int nch, int kind) {
    return stream_nin(kind) * 32 * nch * 16 + ((kind == K_BWD || kind == K_REDUCE_BWD) ? 128 : 0);
}
__host__ __device__ constexpr int stream_warp_smem(int nch, int stages, int kind, bool bulk) {
    const int tb = 32 * nch * 16;
    const int nstg = bulk ? stages : 1;
    const int outbufs = bulk ? 2 : 1;
    return nstg * stream_stage_bytes(nch, kind) + outbufs * stream_nout(kind) * tb + 128;
}

constexpr uint32_t LOAD_WAIT_POLLS = 1u << 22;
constexpr uint32_t CARRY_WAIT_POLLS = 1u << 20;

// sigmoid in fp32 from the approximate exp2 and reciprocal instructions.  REFINE adds one
// Newton step to the reciprocal: the raw instruction is biased by up to an ulp, and a bias
// in gates near one grows by 1 / (1 - gate) in the states (seen as 2e-5 at gates of 0.9995),
// which fp32 storage shows and the 16-bit dtypes do not.
template <bool REFINE>
__device__ __forceinline__ float sigmoid_fast(float z) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
    const float d = 1.0f + e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    if (REFINE && e < 1e30f) r = fmaf(r, fmaf(-d, r, 1.0f), r);
    return r;
}

struct ItemDesc {
    int64_t e_begin;   // first element of the item in the flat matrix
    int64_t row0;      // row of that element
    int64_t pos0;      // its position inside the row
    int64_t n;         // elements in the item
    int32_t s_log;     // segment index in processing order
    int32_t nt;        // tiles in the item
    bool valid;
};

// TOKR (complex64, K_SCAN and K_BWD): the tokens of the caller are real fp32.  Forward: the
// token stream has half the bytes per tile and its imaginary part is taken as zero, which
// fuses the reference's promotion `torch.complex(inputs, zeros)` (complex.py:168-169) into
// the scan.  Backward: only the real part of d_tokens is written, as fp32, which is what the
// reference returns for real inputs (`d_inputs.real`, complex.py:217-218).
//
// ACT = 1 (real dtypes, K_SCAN and K_BWD, one row or segment per item): the first input holds
// gate pre-activations z and the gate is sigmoid(z), computed in fp32 as the tile is read.
// The fused backward returns d_z[t] = x[t-1] * g[t] * s(1 - s) in place of d_gates, which
// removes the caller's sigmoid pass and its backward pass over the (B, C, T) tensors.
//
// GRID (K_SCAN and K_BWD without seeds, INTERIOR = false): items group whole rows, and the rows
// fall on the grid of tiles and lanes -- the row length is a multiple of the elements of a lane
// and either divides the tile or is a multiple of it -- so a row can only start at the first
// element of a lane and which lanes those are is known once per kernel.  The gate that would
// carry a state into a row (its first element, forward; the step after its last element,
// backward) is set to zero there; everything else is the one-row-per-item code, packed
// arithmetic included.  This is the plan of the short power-of-two rows.
template <class TR, int NCH, int KIND, bool REVERSE, bool BULK, bool INTERIOR, bool TOKR = false, int ACT = 0,
          bool GRID = false>
__global__ void __launch_bounds__(INTERIOR ? 384 : ((KIND == K_BWD && NCH > 2) ? 448 : 512), 1) stream_kernel(const StreamParams p) {
    using V = typename TR::V;
    using Raw = typename TR::Raw;
    constexpr int EPC = TR::EPC;
    constexpr int K = NCH * EPC;          // elements per lane per tile
    constexpr int TE = 32 * K;            // elements per tile
    constexpr int TB = 32 * NCH * 16;     // bytes per tile per stream
    constexpr bool BACK = (KIND == K_BWD || KIND == K_REDUCE_BWD);
    constexpr bool REV = REVERSE || BACK;
    constexpr bool REDUCE = (KIND == K_REDUCE || KIND == K_REDUCE_BWD);
    constexpr int NIN = stream_nin(KIND);
    constexpr int NOUT = stream_nout(KIND);
    constexpr int OUTBUFS = BULK ? 2 : 1;
    constexpr bool TOK_IN_REAL = TOKR && KIND == K_SCAN;
    constexpr bool TOK_OUT_REAL = TOKR && KIND == K_BWD;
    const int NSTG = BULK ? p.stages : 1;
    const int WARP_SMEM = stream_warp_smem(NCH, p.stages, KIND, BULK);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    unsigned char *wsm = smem_raw + static_cast<size_t>(wib) * WARP_SMEM;
    unsigned char *stage_base = wsm;
    constexpr int STAGE_BYTES = stream_stage_bytes(NCH, KIND);
    unsigned char *out_base = wsm + NSTG * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(out_base + OUTBUFS * NOUT * TB);

    const int64_t w = static_cast<int64_t>(blockIdx.x) * wpc + wib;
    const int64_t W = static_cast<int64_t>(gridDim.x) * wpc;
    const int64_t T = p.T;
    static_assert(!GRID || (!INTERIOR && (KIND == K_SCAN || KIND == K_BWD)), "GRID: scan kinds, rows on the tile grid");
    // GRID: lanes per row when several rows share a tile (else a row takes whole tiles)
    const int grid_lpr = (GRID && T < TE) ? static_cast<int>(T / K) : 32;
    const bool grid_lane_first = GRID && (lane % grid_lpr == 0), grid_lane_last = GRID && (lane % grid_lpr == grid_lpr - 1);
    const bool dynamic = (p.ctrl != nullptr);
    const bool split = p.segs_per_row > 1;
    const unsigned char *gbase[3] = {static_cast<const unsigned char *>(p.in0), static_cast<const unsigned char *>(p.in1),
                                     static_cast<const unsigned char *>(p.in2)};
    unsigned char *obase[2] = {static_cast<unsigned char *>(p.out0), static_cast<unsigned char *>(p.out1)};
    const V *cin = static_cast<const V *>(p.carry_in);
    const V *hgate = static_cast<const V *>(p.halo_gate);
    const V *hstate = static_cast<const V *>(p.halo_state);

    // tag of a carry word: launch epoch above the segment number (segments < 2^15).  The
    // epoch counts launches modulo 2^17; the launch that wraps it wipes the records (see
    // leave_kernel), so a word with this launch's tag was written by this launch.
    uint32_t epoch = 0;
    if (dynamic) epoch = *reinterpret_cast<volatile uint32_t *>(p.ctrl + CTRL_EPOCH) << EPOCH_SHIFT;

    // ---- item numbers: a global ticket (dynamic) or round-robin (static)
    // draw() only issues the atomic (its result sits in lane 0); resolve() broadcasts it.
    // The two are called an item apart so that the atomic's latency is never waited for.
    int64_t static_next = w;
    auto draw = [&]() -> uint32_t {
        uint32_t t = 0;
        if (dynamic) {
            if (lane == 0) t = atomicAdd(p.ctrl + CTRL_TICKET, 1u);
        }
        return t;
    };
    auto resolve = [&](uint32_t raw) -> int64_t {
        int64_t q;
        if (dynamic) {
            q = __shfl_sync(0xffffffffu, raw, 0);
        } else {
            q = static_next;
            static_next += W;
        }
        return q;
    };
    auto describe = [&](int64_t q) -> ItemDesc {
        ItemDesc d;
        d.valid = q < p.items;
        d.e_begin = 0; d.row0 = 0; d.pos0 = 0; d.s_log = 0; d.n = 0; d.nt = 0;
        if (!d.valid) return d;
        if (!split) {
            const int64_t r0 = q * p.rows_per_item;
            int64_t r1 = r0 + p.rows_per_item;
            if (r1 > p.rows) r1 = p.rows;
            d.row0 = r0;
            d.e_begin = r0 * T;
            d.n = (r1 - r0) * T;
        } else {
            // item numbers and row counts of split plans fit 32 bits (planner)
            const uint32_t qq = static_cast<uint32_t>(q), rg = static_cast<uint32_t>(p.row_groups);
            const uint32_t sl = qq / rg;
            d.s_log = static_cast<int32_t>(sl);
            d.row0 = qq - sl * rg;
            // Coarse segments are processed first, fine ones last.  Forward: coarse from the
            // row start, the fine part is the rest of the row.  Reverse: coarse from the row
            // end down to the fine part, which is the start of the row.
            int64_t len;
            if (d.s_log < p.coarse_segs) {
                len = p.seg_elems;
                d.pos0 = REV ? p.fine_segs * p.fine_elems + (p.coarse_segs - 1 - d.s_log) * p.seg_elems
                             : d.s_log * p.seg_elems;
            } else {
                len = p.fine_elems;
                const int64_t f = d.s_log - p.coarse_segs;
                d.pos0 = REV ? (p.fine_segs - 1 - f) * p.fine_elems : p.coarse_segs * p.seg_elems + f * p.fine_elems;
            }
            d.e_begin = d.row0 * T + d.pos0;
            const int64_t left = T - d.pos0;
            d.n = left < len ? left : len;
        }
        d.nt = static_cast<int32_t>((d.n + TE - 1) / TE);
        return d;
    };

    auto tile_of_step = [&](const ItemDesc &d, int i) -> int { return REV ? d.nt - 1 - i : i; };
    auto tile_valid = [&](const ItemDesc &d, int t) -> int {
        const int64_t left = d.n - static_cast<int64_t>(t) * TE;
        return left < TE ? static_cast<int>(left) : TE;
    };
    // bulk loader: lane 0 arms the stage's mbarrier and issues one copy per stream
    auto issue = [&](const ItemDesc &d, int t, int s) {
        const uint32_t bytes = static_cast<uint32_t>(tile_valid(d, t)) * TR::ESIZE;
        const int64_t goff = (d.e_begin + static_cast<int64_t>(t) * TE) * TR::ESIZE;
        // fused backward: also the 16 bytes of saved states just below the tile (tiles start
        // 16-byte aligned, so that chunk is aligned too); skipped at the start of the matrix
        const bool halo = (KIND == K_BWD) && goff > 0;
        unsigned char *dst = stage_base + s * STAGE_BYTES;
        if constexpr (TOK_IN_REAL) {
            // complex gates, real tokens: the token tile has half the bytes
            mbar_expect_tx(&bars[s], bytes + bytes / 2);
            bulk_g2s(dst, gbase[0] + goff, bytes, &bars[s]);
            bulk_g2s(dst + TB, gbase[1] + goff / 2, bytes / 2, &bars[s]);
            return;
        }
        mbar_expect_tx(&bars[s], bytes * NIN + (halo ? 16u : 0u));
#pragma unroll
        for (int k = 0; k < NIN; ++k) bulk_g2s(dst + k * TB, gbase[k] + goff, bytes, &bars[s]);
        if (halo) bulk_g2s(dst + NIN * TB, gbase[2] + goff - 16, 16, &bars[s]);
    };

    if (BULK) {
        if (lane == 0) {
            for (int s = 0; s < NSTG; ++s) mbar_init(&bars[s], 1);
            mbar_init_fence();
        }
        __syncwarp();
    }

    ItemDesc cur = describe(resolve(draw()));
    uint32_t raw_next = draw();    // ticket of the item after `cur`, not yet looked at
    bool nxt_ready = false;        // `nxt` has been derived from raw_next
    ItemDesc nxt = cur;
    auto need_next = [&]() {
        if (!nxt_ready) {
            nxt = describe(cur.valid ? resolve(raw_next) : p.items);
            nxt_ready = true;
        }
    };

    // producer cursor: tiles are issued in consumption order, at most NSTG ahead, and
    // at most one item ahead of the consumer
    bool prod_in_next = false;
    int p_i = 0;          // next step of the producer's item to issue
    int in_flight = 0;    // issued and not yet consumed
    int ps = 0;           // ring stage the producer fills next
    auto produce = [&]() {
        while (in_flight < NSTG) {
            if (!prod_in_next) {
                if (p_i < cur.nt) {
                    if (lane == 0) issue(cur, tile_of_step(cur, p_i), ps);
                } else {
                    need_next();
                    if (!nxt.valid) break;
                    prod_in_next = true;
                    p_i = 0;
                    continue;
                }
            } else {
                if (p_i < nxt.nt) {
                    if (lane == 0) issue(nxt, tile_of_step(nxt, p_i), ps);
                } else {
                    break;
                }
            }
            ++p_i;
            ++in_flight;
            if (++ps == NSTG) ps = 0;
        }
    };
    if (BULK && cur.valid) produce();

    bool failed = false;
    uint32_t status_bits = 0;
    int cs = 0;                // ring stage of the tile being consumed
    uint32_t parity = 0;       // mbarrier phase parity of that stage
    uint32_t step_count = 0;   // tiles consumed by this warp (selects the staging buffer)

    // Item header: what an item needs from outside its own range -- the state published
    // by the previous segment of its row and (backward kinds) the gate of the step right
    // after it.  It is fetched during the last tile of the item before, so its latency
    // hides behind that tile's arithmetic; the tags tell whether the state was there yet.
    // The header holds the loaded registers untouched; they are decoded in the next item's
    // prologue, so the first use of each load sits a whole tile after its issue.
    struct ItemHeader {
        TaggedWords x, x2;
        Raw gate;
        int gate_kind;     // 0 = none (one), 1 = `gate` is a raw element of the gates, 2 = caller's halo gate
        V halo;
    };
    constexpr bool TWO_WORDS = sizeof(V) > 4;
    auto fetch_header = [&](const ItemDesc &d) -> ItemHeader {
        ItemHeader h;
        h.x.w0 = 0; h.x.w1 = 0; h.x2.w0 = 0; h.x2.w1 = 0;
        h.gate = 0;
        h.gate_kind = 0;
        h.halo = vone(V());
        if (!d.valid) return h;
        if (split && d.s_log > 0) {
            const unsigned char *rec = p.records + d.row0 * CARRY_RECORD_BYTES;
            h.x = fetch_tagged(rec, 0, TWO_WORDS);
            if (REDUCE) h.x2 = fetch_tagged(rec, 1, TWO_WORDS);
        }
        if (BACK && !INTERIOR) {
            if (d.pos0 + d.n < T) {
                h.gate = TR::load_raw(p.in0, d.e_begin + d.n);          // next step of the same row
                h.gate_kind = 1;
            } else if (hgate) {
                h.halo = hgate[d.row0];                                  // the row ends here
                h.gate_kind = 2;
            }
        }
        return h;
    };
    ItemHeader head = fetch_header(cur);

    while (cur.valid && !failed) {
        // ---------------- item prologue: incoming state, halo gate, running position
        V x_carry = vzero(V());    // state entering the tile
        V x2_carry = vzero(V());   // reduce kinds: response to a unit incoming state
        // backward kinds: gate of the first element above the tile
        V item_end_gate = head.gate_kind == 1 ? TR::decode(head.gate) : (head.gate_kind == 2 ? head.halo : vone(V()));
        if constexpr (ACT == 1) {
            if (head.gate_kind == 1) item_end_gate = sigmoid_fast<TR::ESIZE == 4>(item_end_gate);
        }
        V next_gate = item_end_gate;
        if (split && cur.s_log > 0) {
            // state published by the warp that processed the previous segment of this row
            const unsigned char *rec = p.records + cur.row0 * CARRY_RECORD_BYTES;
            const uint32_t want = epoch | static_cast<uint32_t>(cur.s_log);
            bool got = decode_tagged(head.x, want, x_carry);
            if (REDUCE) got = decode_tagged(head.x2, want, x2_carry) && got;
            // not published when the header was fetched: poll, with a bound
            for (uint32_t poll = 0; !got && poll < CARRY_WAIT_POLLS; ++poll) {
                __nanosleep(64);
                got = read_tagged(rec, 0, want, x_carry);
                if (REDUCE) got = read_tagged(rec, 1, want, x2_carry) && got;
            }
            if (!got) {
                status_bits |= STATUS_LOOKBACK_TIMEOUT;
                x_carry = vzero(V());
                x2_carry = vzero(V());
            }
        } else if (!INTERIOR) {
            // the item opens its row: the caller's incoming state, and a unit state for the
            // product carried by the reduce kinds
            if (cin) x_carry = cin[cur.row0];
            if (REDUCE) x2_carry = vone(V());
        }
        int64_t ts_mod, row_ts;   // (tile start) mod T and the row of the tile start
        {
            const int64_t pos = cur.pos0 + static_cast<int64_t>(tile_of_step(cur, 0)) * TE;
            if (pos < T) {
                ts_mod = pos;
                row_ts = cur.row0;
            } else {
                ts_mod = pos % T;
                row_ts = cur.row0 + pos / T;
            }
        }

        for (int i = 0; i < cur.nt; ++i) {
            const int t = tile_of_step(cur, i);
            const int64_t toff = static_cast<int64_t>(t) * TE;
            const int nvalid = tile_valid(cur, t);
            const unsigned char *stg = stage_base + cs * STAGE_BYTES;

            // backward: the state just below the tile, needed by lane 0 for d_gates
            Raw x_halo_raw = 0;
            V x_halo_row = vzero(V());
            const bool halo_in_row = (ts_mod != 0);
            if (KIND == K_BWD) {
                // (the bulk loader brings this state with the tile, see issue())
                if (halo_in_row && !BULK) x_halo_raw = TR::load_raw(p.in2, cur.e_begin + toff - 1);
                else if (!halo_in_row && !INTERIOR && hstate) x_halo_row = hstate[row_ts];
            }
            // last tile of the item: fetch the header of the next one now
            ItemHeader head_next = head;
            if (i == cur.nt - 1) {
                need_next();
                head_next = fetch_header(nxt);
            }

            if (BULK) {
                bool ok = mbar_wait_bounded(&bars[cs], parity, LOAD_WAIT_POLLS);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    failed = true;
                    status_bits |= STATUS_LOAD_TIMEOUT;
                    break;
                }
            } else {
                // plain loader: element-wise copy of the valid part of the tile
                __syncwarp();
#pragma unroll
                for (int k = 0; k < NIN; ++k) {
                    const Raw *src = reinterpret_cast<const Raw *>(gbase[k]) + cur.e_begin + toff;
                    Raw *dst = reinterpret_cast<Raw *>(wsm + k * TB);
                    for (int idx = lane; idx < nvalid; idx += 32) dst[idx] = src[idx];
                }
                __syncwarp();
            }

            // ---- shared -> registers
            V a[K], b[K];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const uint4 qa = *reinterpret_cast<const uint4 *>(stg + 0 * TB + (lane * NCH + c) * 16);
                TR::unpack(qa, &a[c * EPC]);
                if constexpr (TOK_IN_REAL) {
                    // K real tokens of 4 bytes per lane, read as 8-byte pairs; imaginary part zero
                    const float2 tk = *reinterpret_cast<const float2 *>(stg + TB + lane * (K * 4) + c * 8);
                    b[2 * c] = make_float2(tk.x, 0.0f);
                    b[2 * c + 1] = make_float2(tk.y, 0.0f);
                } else {
                    const uint4 qb = *reinterpret_cast<const uint4 *>(stg + 1 * TB + (lane * NCH + c) * 16);
                    TR::unpack(qb, &b[c * EPC]);
                }
            }
            if constexpr (ACT == 1) {
#pragma unroll
                for (int j = 0; j < K; ++j) a[j] = sigmoid_fast<TR::ESIZE == 4>(a[j]);
            }
            V xp[KIND == K_BWD ? K : 1];
            V x_below = vzero(V());   // state just below the tile, from the halo chunk
            if (KIND == K_BWD) {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const uint4 qx = *reinterpret_cast<const uint4 *>(stg + 2 * TB + (lane * NCH + c) * 16);
                    TR::unpack(qx, &xp[c * EPC]);
                }
                if (BULK && halo_in_row) {
                    V hv[EPC];
                    TR::unpack(*reinterpret_cast<const uint4 *>(stg + NIN * TB), hv);
                    x_below = hv[EPC - 1];
                }
            }
            if (BULK) {
                // the stage is free again: refill the ring
                __syncwarp();
                --in_flight;
                if (++cs == NSTG) {
                    cs = 0;
                    parity ^= 1u;
                }
                if (lane == 0) fence_async_smem();
                produce();
            }

            // ---- backward kinds: shift the gates by one step inside registers
            V gate_first = vone(V());   // gate of the lane's first element, before the shift
            if (BACK) {
                const V g0 = a[0];
                gate_first = g0;
                V up = shfl_down(g0, 1);
                if (lane == 31) up = next_gate;
#pragma unroll
                for (int j = 0; j < K - 1; ++j) a[j] = vconj(a[j + 1]);
                a[K - 1] = vconj(up);
                next_gate = shfl_idx(g0, 0);
            }

            const int jv = nvalid - lane * K;   // elements j >= jv lie beyond the item
            // GRID: does a row start at this lane's first element / end at its last one in this tile
            const bool row_first = grid_lane_first && (T <= TE || ts_mod == 0);
            const bool row_last = grid_lane_last && (T <= TE || ts_mod + TE == T);
            V b2[(REDUCE && INTERIOR) ? K : 1];
            uint32_t start_mask_lo = 0, start_mask_hi = 0;   // INTERIOR backward: elements that open a row
            bool has_boundary = false;
            // Where the row boundaries fall among this lane's K elements (INTERIOR only).
            const bool tiny = T < K;            // several rows inside one lane: per-element arithmetic
            int js = -1, je = -1, jwrap = K;    // row start, row end, first element of the next row
            int64_t rowq = row_ts;              // row of the lane's first element
            // Row starts and row ends as bit masks over the lane's elements: testing a constant
            // bit keeps a[] and b[] in registers (an equality test `j == js` invites the compiler
            // to turn the chain into one indexed store, which moves the arrays to local memory).
            uint32_t smask = 0, emask = 0;
            auto row_of = [&](int j) -> int64_t {
                if (!tiny) return rowq + (j >= jwrap ? 1 : 0);
                return row_ts + (static_cast<int>(ts_mod) + lane * K + j) / static_cast<int>(T);
            };
            auto classify = [&](int j, bool &is_start, bool &is_end, int64_t &row) {
                is_start = (smask >> j) & 1u;
                is_end = (emask >> j) & 1u;
                row = row_of(j);
            };

            if (!INTERIOR) {
                // ---- the ragged last tile of a row: identity beyond the row's end
                if (nvalid < TE) {
                    V gate_end = vone(V());
                    if (BACK) gate_end = vconj(item_end_gate);
#pragma unroll
                    for (int j = 0; j < K; ++j) {
                        // (range tests on purpose: an equality test on j invites the compiler to
                        // turn the chain into one indexed store, which puts a[] in local memory)
                        if (j >= jv) {
                            a[j] = vone(V());
                            b[j] = vzero(V());
                        } else if (BACK && j + 1 >= jv) {
                            // the last step of the row takes the gate of the step after the row
                            a[j] = gate_end;
                        }
                    }
                }
                if constexpr (GRID) {
                    // nothing is carried into a row: zero the gate of its first processed element
                    if (!REV) {
                        if (row_first) a[0] = vzero(V());
                    } else {
                        if (row_last) a[K - 1] = vzero(V());
                    }
                }
            } else {
                // ---- items that group rows: row boundaries inside the tile
                if (REDUCE) {
#pragma unroll
                    for (int j = 0; j < K; ++j) b2[j] = vzero(V());
                }
                has_boundary = (ts_mod == 0) || (ts_mod + nvalid >= T);
                const bool slow = has_boundary || (nvalid < TE);
                if (slow && !tiny) {
                    const int64_t p0 = ts_mod + lane * K;
                    int64_t q0, r;
                    if (T > TE) {
                        q0 = p0 >= T ? 1 : 0;
                        r = p0 - (q0 ? T : 0);
                    } else {
                        const int pi = static_cast<int>(p0), ti = static_cast<int>(T);
                        const int qi = pi / ti;
                        q0 = qi;
                        r = pi - qi * ti;
                    }
                    rowq = row_ts + q0;
                    const int64_t tr = T - r;       // distance to the next row start, 1..T
                    jwrap = tr < K ? static_cast<int>(tr) : K;
                    js = (r == 0) ? 0 : (tr < K ? static_cast<int>(tr) : -1);
                    je = (tr <= K) ? static_cast<int>(tr - 1) : -1;
                    if (js >= 0) smask = 1u << js;
                    if (je >= 0) emask = 1u << je;
                }
                if (slow && tiny) {
#pragma unroll
                    for (int j = 0; j < K; ++j) {
                        const int pi = static_cast<int>(ts_mod) + lane * K + j, ti = static_cast<int>(T);
                        const int rem = pi - (pi / ti) * ti;
                        smask |= (rem == 0 ? 1u : 0u) << j;
                        emask |= (rem == ti - 1 ? 1u : 0u) << j;
                    }
                }
                if (slow) {
#pragma unroll
                    for (int j = 0; j < K; ++j) {
                        bool is_start, is_end;
                        int64_t row;
                        classify(j, is_start, is_end, row);
                        const bool first = REV ? is_end : is_start;
                        if (j >= jv) {
                            a[j] = vone(V());
                            b[j] = vzero(V());
                        } else {
                            if (first) {
                                V a_orig = a[j];
                                if (BACK) a_orig = hgate ? vconj(hgate[row]) : vone(V());
                                if (cin) b[j] = vfma(a_orig, cin[row], b[j]);
                                if (REDUCE) b2[j] = a_orig;
                                a[j] = vzero(V());
                            }
                            if (KIND == K_BWD && is_start) {
                                if (j < 32) start_mask_lo |= 1u << (j & 31);
                                else start_mask_hi |= 1u << (j & 31);
                            }
                        }
                    }
                }
            }

            // ---- pass 1: lane aggregate in processing order
            // Real types without interior boundaries run the lane's elements as two half-length
            // chains side by side in packed fp32x2 instructions (half the instructions, half the
            // dependent latency); (A0h, B0h) is the aggregate of the first half.
            constexpr bool PACKED = !INTERIOR && sizeof(V) == 4 && (K % 2 == 0);
            constexpr int H = K / 2;
            constexpr int JF = REV ? K - 1 : 0;
            V A0h = vone(V()), B0h = vzero(V());
            V x = vzero(V());    // state entering this lane
            V x2 = vzero(V());
            {
            V A, B;
            V B2 = vzero(V());
            if constexpr (PACKED) {
                auto J = [](int q) { return REV ? K - 1 - q : q; };
                float2 Av = make_float2(a[J(0)], a[J(H)]);
                float2 Bv = make_float2(b[J(0)], b[J(H)]);
#pragma unroll
                for (int q = 1; q < H; ++q) {
                    const float2 av = make_float2(a[J(q)], a[J(H + q)]);
                    const float2 bv = make_float2(b[J(q)], b[J(H + q)]);
                    Bv = __ffma2_rn(av, Bv, bv);
                    Av = __fmul2_rn(Av, av);
                }
                A0h = Av.x;
                B0h = Bv.x;
                A = Av.x * Av.y;
                B = fmaf(Av.y, Bv.x, Bv.y);
            } else {
                A = a[JF];
                B = b[JF];
                if (REDUCE && INTERIOR) B2 = b2[JF];
#pragma unroll
                for (int q = 1; q < K; ++q) {
                    const int j = REV ? K - 1 - q : q;
                    B = vfma(a[j], B, b[j]);
                    if (REDUCE && INTERIOR) B2 = vfma(a[j], B2, b2[j]);
                    A = vmul(A, a[j]);
                }
            }
            // the warp's incoming state enters through the first lane in processing order
            const int ll = REV ? 31 - lane : lane;
            constexpr bool unit_channel = REDUCE;            // also carry the response to a unit state
            if (ll == 0) {
                B = vfma(A, x_carry, B);
                if (unit_channel) B2 = vfma(A, x2_carry, B2);
            }
            // ---- Kogge-Stone inclusive combine across lanes
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const V Ap = REV ? shfl_down(A, d) : shfl_up(A, d);
                const V Bp = REV ? shfl_down(B, d) : shfl_up(B, d);
                V B2p = vzero(V());
                if (unit_channel) B2p = REV ? shfl_down(B2, d) : shfl_up(B2, d);
                if (ll >= d) {
                    B = vfma(A, Bp, B);
                    if (unit_channel) B2 = vfma(A, B2p, B2);
                    if (d < 16) A = vmul(A, Ap);
                }
            }
            // state entering this lane = inclusive result of the previous lane
            x = REV ? shfl_down(B, 1) : shfl_up(B, 1);
            if (ll == 0) x = x_carry;
            if (REDUCE && INTERIOR) {
                x2 = REV ? shfl_down(B2, 1) : shfl_up(B2, 1);
                if (ll == 0) x2 = x2_carry;
            }
            x_carry = shfl_idx(B, REV ? 0 : 31);
            if (unit_channel) x2_carry = shfl_idx(B2, REV ? 0 : 31);
            }

            if (!REDUCE) {
                // ---- pass 2: the recurrence itself from the lane's incoming state
                if (PACKED) {
                  if constexpr (PACKED) {
                    auto J = [](int q) { return REV ? K - 1 - q : q; };
                    float2 Xv = make_float2(x, fmaf(A0h, x, B0h));   // states entering the two halves
#pragma unroll
                    for (int q = 0; q < H; ++q) {
                        const float2 av = make_float2(a[J(q)], a[J(H + q)]);
                        const float2 bv = make_float2(b[J(q)], b[J(H + q)]);
                        Xv = __ffma2_rn(av, Xv, bv);
                        b[J(q)] = Xv.x;
                        b[J(H + q)] = Xv.y;
                    }
                  }
                } else {
#pragma unroll
                    for (int q = 0; q < K; ++q) {
                        const int j = REV ? K - 1 - q : q;
                        x = vfma(a[j], x, b[j]);
                        b[j] = x;
                    }
                }
                if (KIND == K_BWD) {
                    // d_gates[t] = conj(x[t-1]) * g[t]: the previous state comes from the
                    // element below (neighbouring lane by shuffle, tile halo for lane 0)
                    V dn = shfl_up(xp[K - 1], 1);
                    if (lane == 0) dn = halo_in_row ? (BULK ? x_below : TR::decode(x_halo_raw)) : x_halo_row;
                    if (GRID && row_first) dn = vzero(V());       // a row starts here: the state before it is zero
                    if constexpr (ACT == 1) {
                        // after the shift a[j-1] is the gate s of element j: chain rule through
                        // the sigmoid, d_z = d_gate * s * (1 - s); downwards, so that each gate
                        // is read before its slot receives a gradient
#pragma unroll
                        for (int j = K - 1; j >= 1; --j) {
                            const V sg = a[j - 1];
                            a[j] = vmul(vmul(xp[j - 1], b[j]), fmaf(-sg, sg, sg));
                        }
                        a[0] = vmul(vmul(dn, b[0]), fmaf(-gate_first, gate_first, gate_first));
                    } else {
#pragma unroll
                        for (int j = 1; j < K; ++j) a[j] = vmul(vconj(xp[j - 1]), b[j]);
                        a[0] = vmul(vconj(dn), b[0]);
                    }
                    if (INTERIOR && (start_mask_lo | start_mask_hi)) {
#pragma unroll
                        for (int j = 0; j < K; ++j) {
                            const bool st = j < 32 ? (start_mask_lo >> (j & 31)) & 1u : (start_mask_hi >> (j & 31)) & 1u;
                            if (st) {
                                bool is_start, is_end;
                                int64_t row;
                                classify(j, is_start, is_end, row);
                                const V xs = hstate ? hstate[row] : vzero(V());
                                a[j] = vmul(vconj(xs), b[j]);
                            }
                        }
                    }
                }
                // ---- registers -> staging -> global
                unsigned char *ob = out_base + (BULK ? static_cast<int>(step_count & 1u) : 0) * NOUT * TB;
                if (BULK) {
                    if (lane == 0) bulk_wait_read<1>();
                }
                __syncwarp();
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    if constexpr (TOK_OUT_REAL) {
                        // real parts only: K values of 4 bytes per lane, written as 8-byte pairs
                        *reinterpret_cast<float2 *>(ob + lane * (K * 4) + c * 8) = make_float2(b[2 * c].x, b[2 * c + 1].x);
                    } else {
                        *reinterpret_cast<uint4 *>(ob + (lane * NCH + c) * 16) = TR::pack(&b[c * EPC]);
                    }
                    if (NOUT > 1) *reinterpret_cast<uint4 *>(ob + TB + (lane * NCH + c) * 16) = TR::pack(&a[c * EPC]);
                }
                if (BULK) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const uint32_t bytes = static_cast<uint32_t>(nvalid) * TR::ESIZE;
                        const int64_t goff = (cur.e_begin + toff) * TR::ESIZE;
#pragma unroll
                        for (int k = 0; k < NOUT; ++k) {
                            if (TOK_OUT_REAL && k == 0)
                                bulk_s2g(obase[0] + goff / 2, ob, bytes / 2);
                            else
                                bulk_s2g(obase[k] + goff, ob + k * TB, bytes);
                        }
                        bulk_commit();
                    }
                } else {
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < NOUT; ++k) {
                        const Raw *src = reinterpret_cast<const Raw *>(ob + k * TB);
                        Raw *dst = reinterpret_cast<Raw *>(obase[k]) + cur.e_begin + toff;
                        for (int idx = lane; idx < nvalid; idx += 32) dst[idx] = src[idx];
                    }
                }
            } else if (INTERIOR && has_boundary) {
                // reduce kinds over grouped rows: tiles that finish a row need the element states
                V *cout = static_cast<V *>(p.carry_out);
#pragma unroll
                for (int q = 0; q < K; ++q) {
                    const int j = REV ? K - 1 - q : q;
                    x = vfma(a[j], x, b[j]);
                    x2 = vfma(a[j], x2, b2[j]);
                    bool is_start, is_end;
                    int64_t row;
                    classify(j, is_start, is_end, row);
                    const bool last = REV ? is_start : is_end;
                    if (last && j < jv) {
                        cout[2 * row] = x2;
                        cout[2 * row + 1] = x;
                    }
                }
            }
            ++step_count;
            head = head_next;

            // ---- advance the running tile position
            if (!REV) {
                ts_mod += TE;
                if (ts_mod >= T) {
                    if (T > TE) {
                        ts_mod -= T;
                        row_ts += 1;
                    } else {
                        row_ts += ts_mod / T;
                        ts_mod %= T;
                    }
                }
            } else {
                ts_mod -= TE;
                if (ts_mod < 0) {
                    if (T > TE) {
                        ts_mod += T;
                        row_ts -= 1;
                    } else {
                        const int64_t k = (-ts_mod + T - 1) / T;
                        ts_mod += k * T;
                        row_ts -= k;
                    }
                }
            }
        }
        if (failed) break;

        // ---------------- item epilogue: hand the outgoing state on, move to the next item
        if (split && cur.s_log + 1 < p.segs_per_row) {
            // (fault injection for the tests: the hand-over of row 0's first segment is dropped,
            // so exactly one reader runs into its bound and reports it)
            const bool drop = p.test_drop_carry && cur.row0 == 0 && cur.s_log == 0;
            if (lane == 0 && !drop) {
                unsigned char *rec = p.records + cur.row0 * CARRY_RECORD_BYTES;
                const uint32_t tag = epoch | static_cast<uint32_t>(cur.s_log + 1);
                publish_tagged(rec, 0, x_carry, tag);
                if (REDUCE) publish_tagged(rec, 1, x2_carry, tag);
            }
        } else if (REDUCE && !INTERIOR) {
            // the item closes its row: the running state is the row's carry
            if (lane == 0) {
                V *cout = static_cast<V *>(p.carry_out);
                cout[2 * cur.row0] = x2_carry;
                cout[2 * cur.row0 + 1] = x_carry;
            }
        }
        need_next();
        cur = nxt;
        raw_next = cur.valid ? draw() : 0u;
        nxt_ready = false;
        if (prod_in_next) {
            prod_in_next = false;      // the producer's item is now the current one
        } else {
            p_i = 0;                   // the producer had nothing to run ahead into
        }
        if (BULK && cur.valid) produce();
    }

    if (BULK) {
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
    }
    if (dynamic) leave_kernel(p, W, status_bits, lane);
}

}  // namespace ascan

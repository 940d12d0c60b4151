// Look-back scan kernel: single pass, for matrices with clearly fewer rows than SMs and for
// rows whose time axis is sharded over several GPUs.
//
// A row is cut into SEGMENTS; an item is one segment, drawn from the ticket counter by
// persistent CTAs, so segments of many rows are in flight at any time, spread over every SM.
// Tickets run over groups of rows, segment-major inside a group (all rows' first segments in
// processing order, then all second ones, ...): when a segment is drawn, the one before it in
// its row was drawn a group's worth of tickets earlier and its aggregate is published by the
// time it is asked for.
//
// A CTA works on a segment as a team.  Its G worker warps each take NT consecutive tiles of
// the segment (a segment is G * NT tiles) and keep them in shared memory; the last warp of
// the CTA keeps the books.  For a segment
//   1. every worker loads its tiles with bulk asynchronous copies (one stage per tile) and
//      computes the AGGREGATE of its part, the affine map x -> A*x + B from the state before
//      the part to the state after it, leaving in shared memory, per tile and lane, the map
//      from the part's start to the lane's first element;
//   2. the worker that finishes last composes the G parts into the segment's aggregate and
//      publishes it in the segment's record;
//   3. the bookkeeper composes the aggregates of all earlier segments of the row into the
//      state entering the segment, and hands every worker the state entering its part;
//   4. every worker runs the recurrence from shared memory (no second read of global memory)
//      and stores the results with bulk copies; stages that have drained are refilled with
//      the worker's tiles of the segment after the next.
// Step 1 of the next segment runs before step 4 of this one, so two segments are resident
// per CTA and step 3 has a whole aggregate pass to finish.  The bookkeeper also draws the
// tickets, each only after the look-back of the segment two before it: nothing that a
// published aggregate depends on ever waits for a look-back, so step 3 never waits for
// another CTA's step 3 (such waits would chain up).  Tickets, records and look-backs cost
// one warp's time per segment instead of every warp's time per few tiles.
//
// Aggregates are kept at three levels -- segments, blocks of 32 segments, super-blocks of 32
// blocks; the warp that publishes the last segment of a block (super-block) composes and
// publishes the block's (super-block's) aggregate -- so a look-back reads at most 31 records
// per level (plus one window per 32 super-blocks in very long rows).  Which records are
// composed, and in which order, depends only on the segment's number: results are bitwise
// reproducible.  Records are self-tagged 64-bit words (payload, launch tag); every wait is
// bounded and ends in a status bit.
//
// Time sharding over GPUs (ShardParams.world > 1): every rank runs this kernel on its time
// slice of all rows.  The warp that publishes the last segment of a row's slice composes the
// slice's aggregate and stores it, with plain 64-bit stores, into the exchange buffers of
// the ranks that come later in processing order; a segment's incoming state is then the
// fold, in rank order, of the earlier ranks' slice aggregates (read from this rank's own
// exchange buffer) followed by the local look-back.  No rank waits for another rank's
// results, only for its aggregates, so all ranks stream at the same time.
#pragma once

#include "stream.cuh"

namespace ascan {

constexpr int LB_RECORD_BYTES = 32;          // one affine pair of the compute type in tagged 64-bit words
constexpr int LB_MAX_TILES = 8;              // tiles per worker and segment, at most (a worker holds two segments: 2 stages per tile)
constexpr uint32_t LB_SHARDED_GROUP_ROWS = 16;  // rows whose segments are interleaved in ticket order when time is sharded (half as many from eight ranks on)
constexpr int LB_MAX_WORKERS = 15;           // worker warps per CTA, at most (plus the bookkeeper)
constexpr int LB_TEAM_BYTES = 3072;          // shared memory of the team: parts, incoming states, mbarriers, part descriptors
constexpr int MAX_WORLD = 16;                // ranks of a time-sharded scan, at most
constexpr uint32_t LB_WAIT_POLLS = 1u << 20;      // about a second
constexpr uint32_t LB_TEAM_POLLS = 1u << 22;      // waits inside a CTA: a safety net, they end on the abort flag

// Exchange buffer of one rank and one direction (forward or backward channel), written by the
// other ranks with peer stores:
//   [0, 256)                      done[src]: last call that rank `src` has completed (u64 each)
//   [256, +2*rows*16)             gate halo per (call parity, row): first gate of the next rank's slice
//   [.., +2*world*rows*32)        slice aggregates per (call parity, source rank, row)
__host__ __device__ constexpr uint64_t xchg_halo_offset() { return 256; }
__host__ __device__ constexpr uint64_t xchg_carry_offset(int64_t rows) { return 256 + 2ull * rows * 16; }
__host__ __device__ constexpr uint64_t xchg_bytes(int64_t rows, int world) {
    return xchg_carry_offset(rows) + 2ull * world * rows * LB_RECORD_BYTES;
}

struct ShardParams {
    int32_t rank, world;              // world <= 1: the rows are not sharded along time
    uint32_t call;                    // number of this call on the channel (same on every rank, 1, 2, 3, ...)
    int32_t reserved;
    unsigned char *xchg[MAX_WORLD];   // xchg[j]: exchange buffer of rank j as mapped in this process (xchg[rank]: local)
    void *carry_save;                 // forward: rows values of the compute type, the state entering this rank's slice
};

__host__ __device__ constexpr int lb_stage_bytes(int nch, int kind) {
    return stream_nin(kind) * 32 * nch * 16 + (kind == K_BWD ? 128 : 0);
}
// The forward kinds send their results through a staging tile of their own, so that a stage can
// be refilled as soon as its tile is in registers; the fused backward writes its two results over
// the stage's inputs (a staging area would cost it two warps per CTA).
__host__ __device__ constexpr int lb_staging_bytes(int nch, int kind) { return kind == K_BWD ? 0 : 32 * nch * 16; }
// Prefix maps, per stage and lane: the affine map from the part's start to the lane's first
// element (two values of the compute type).
__host__ __device__ constexpr int lb_prefix_bytes(bool complex_type) { return complex_type ? 16 : 8; }
// Per worker: its `nt` tiles of two resident segments, the staging tile, the mbarriers, the
// prefix maps.
__host__ __device__ constexpr int lb_warp_smem(int nch, int nt, int kind, bool complex_type) {
    return 2 * nt * lb_stage_bytes(nch, kind) + lb_staging_bytes(nch, kind) + 128 + 2 * nt * 32 * lb_prefix_bytes(complex_type);
}
// Workspace of the look-back plan: control block, then the records of the three levels.
__host__ __device__ constexpr uint64_t lb_level_count(int64_t n) { return static_cast<uint64_t>((n + 31) / 32); }
__host__ __device__ constexpr uint64_t lb_records_per_row(int64_t segs) {
    return static_cast<uint64_t>(segs) + lb_level_count(segs) + lb_level_count(static_cast<int64_t>(lb_level_count(segs)));
}

__device__ __forceinline__ void st_relaxed_sys_u64(void *p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const void *p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// ---- records: an affine pair (A, B) in tagged words.  SYS = the record crosses GPUs.
template <bool SYS>
__device__ __forceinline__ void put_word(unsigned char *p, float v, uint32_t tag) {
    if (SYS) st_relaxed_sys_u64(p, tagged_word(v, tag));
    else st_relaxed_u64(p, tagged_word(v, tag));
}
template <bool SYS>
__device__ __forceinline__ bool get_word(const unsigned char *p, uint32_t tag, float &v) {
    const uint64_t w = SYS ? ld_relaxed_sys_u64(p) : ld_relaxed_u64(p);
    v = __uint_as_float(static_cast<uint32_t>(w));
    return static_cast<uint32_t>(w >> 32) == tag;
}
template <bool SYS>
__device__ __forceinline__ void put_pair(unsigned char *rec, float A, float B, uint32_t tag) {
    put_word<SYS>(rec, A, tag);
    put_word<SYS>(rec + 8, B, tag);
}
template <bool SYS>
__device__ __forceinline__ void put_pair(unsigned char *rec, float2 A, float2 B, uint32_t tag) {
    put_word<SYS>(rec, A.x, tag);
    put_word<SYS>(rec + 8, A.y, tag);
    put_word<SYS>(rec + 16, B.x, tag);
    put_word<SYS>(rec + 24, B.y, tag);
}
template <bool SYS>
__device__ __forceinline__ bool get_pair(const unsigned char *rec, uint32_t tag, float &A, float &B) {
    const bool a = get_word<SYS>(rec, tag, A);
    const bool b = get_word<SYS>(rec + 8, tag, B);
    return a && b;
}
template <bool SYS>
__device__ __forceinline__ bool get_pair(const unsigned char *rec, uint32_t tag, float2 &A, float2 &B) {
    const bool a = get_word<SYS>(rec, tag, A.x);
    const bool b = get_word<SYS>(rec + 8, tag, A.y);
    const bool c = get_word<SYS>(rec + 16, tag, B.x);
    const bool d = get_word<SYS>(rec + 24, tag, B.y);
    return a && b && c && d;
}

// Composes the `n` (<= 32) records base[0], base[stride], ... in that order: on return every
// lane holds (A, B) with  x -> A*x + B  = record n-1 after ... after record 0.  Lane i reads
// record i and polls until it carries `tag`; false when the bound expires.  The combine is a
// Kogge-Stone scan over the lanes with identity in the unused lanes: a fixed tree.
// `ahead` (real types, optional): this lane's two words loaded ahead of time; used if they carry
// the tag already.
template <class V, bool SYS>
__device__ __forceinline__ bool compose_window(const unsigned char *base, int64_t stride, int n, uint32_t tag, int lane,
                                               V &A, V &B, const uint64_t *ahead = nullptr) {
    V a = vone(V()), b = vzero(V());
    bool ok = lane >= n;
    if constexpr (sizeof(V) == 4) {
        if (ahead && !ok && static_cast<uint32_t>(ahead[0] >> 32) == tag && static_cast<uint32_t>(ahead[1] >> 32) == tag) {
            a = __uint_as_float(static_cast<uint32_t>(ahead[0]));
            b = __uint_as_float(static_cast<uint32_t>(ahead[1]));
            ok = true;
        }
    }
    bool all = false;
    for (uint32_t poll = 0; poll < LB_WAIT_POLLS; ++poll) {
        if (!ok) ok = get_pair<SYS>(base + lane * stride, tag, a, b);
        all = __all_sync(0xffffffffu, ok);
        if (all) break;
        if (poll > 8) __nanosleep(poll > 64 ? 200 : 40);
    }
    if (!all) {
        A = vone(V());
        B = vzero(V());
        return false;
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const V Ap = shfl_up(a, d), Bp = shfl_up(b, d);
        if (lane >= d) {
            b = vfma(a, Bp, b);
            a = vmul(a, Ap);
        }
    }
    A = shfl_idx(a, 31);
    B = shfl_idx(b, 31);
    return true;
}

// Reads up to three windows of records at once (lane i reads record i of each) and polls only
// for those still missing, so a look-back whose records are all there costs one round trip.
// Window w: n[w] records from base[w]; result (A[w], B[w]) as in compose_window.
// The words of a real-valued look-back (three windows of {A, B}), loaded ahead of time.
struct RecordWords {
    uint64_t w[6];
};
__device__ __forceinline__ RecordWords load_record_words(const unsigned char *const base[3], const int n[3], int lane) {
    RecordWords r;
#pragma unroll
    for (int w = 0; w < 3; ++w) {
        r.w[2 * w] = r.w[2 * w + 1] = 0;
        if (lane < n[w]) {
            r.w[2 * w] = ld_relaxed_u64(base[w] + lane * LB_RECORD_BYTES);
            r.w[2 * w + 1] = ld_relaxed_u64(base[w] + lane * LB_RECORD_BYTES + 8);
        }
    }
    return r;
}

template <class V>
__device__ __forceinline__ bool compose_three(const unsigned char *const base[3], const int n[3], uint32_t tag, int lane,
                                              V A[3], V B[3], const RecordWords *ahead = nullptr) {
    V a[3], b[3];
    bool ok[3];
#pragma unroll
    for (int w = 0; w < 3; ++w) {
        a[w] = vone(V());
        b[w] = vzero(V());
        ok[w] = lane >= n[w];
    }
    if constexpr (sizeof(V) == 4) {
        // words loaded before the aggregate pass of the next item: normally all of them are valid
        if (ahead) {
#pragma unroll
            for (int w = 0; w < 3; ++w) {
                if (!ok[w] && static_cast<uint32_t>(ahead->w[2 * w] >> 32) == tag &&
                    static_cast<uint32_t>(ahead->w[2 * w + 1] >> 32) == tag) {
                    a[w] = __uint_as_float(static_cast<uint32_t>(ahead->w[2 * w]));
                    b[w] = __uint_as_float(static_cast<uint32_t>(ahead->w[2 * w + 1]));
                    ok[w] = true;
                }
            }
        }
    }
    bool all = false;
    for (uint32_t poll = 0; poll < LB_WAIT_POLLS; ++poll) {
#pragma unroll
        for (int w = 0; w < 3; ++w)
            if (!ok[w]) ok[w] = get_pair<false>(base[w] + lane * LB_RECORD_BYTES, tag, a[w], b[w]);
        all = __all_sync(0xffffffffu, ok[0] && ok[1] && ok[2]);
        if (all) break;
        if (poll > 4) __nanosleep(poll > 64 ? 200 : 40);
    }
#pragma unroll
    for (int w = 0; w < 3; ++w) {
        if (n[w] > 0 && all) {
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const V Ap = shfl_up(a[w], d), Bp = shfl_up(b[w], d);
                if (lane >= d) {
                    b[w] = vfma(a[w], Bp, b[w]);
                    a[w] = vmul(a[w], Ap);
                }
            }
            A[w] = shfl_idx(a[w], 31);
            B[w] = shfl_idx(b[w], 31);
        } else {
            A[w] = vone(V());
            B[w] = vzero(V());
        }
    }
    return all;
}

// Bounded wait on an mbarrier of the team; ends early when a warp of the CTA has raised the
// abort flag (after a wait of its own has expired).
__device__ __forceinline__ bool team_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag) {
    if (mbar_test_wait(bar, parity)) return true;      // the usual case: the phase is over already
    for (uint32_t i = 0; i < LB_TEAM_POLLS; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
            : "memory");
        if (ok) return true;
        if ((i & 7u) == 7u && *abort_flag) return false;
    }
    return false;
}

// An affine pair in the team's shared memory (16 bytes per slot).
__device__ __forceinline__ void store_part(unsigned char *p, float A, float B) {
    volatile float *q = reinterpret_cast<volatile float *>(p);
    q[0] = A;
    q[1] = B;
}
__device__ __forceinline__ void store_part(unsigned char *p, float2 A, float2 B) {
    volatile float *q = reinterpret_cast<volatile float *>(p);
    q[0] = A.x;
    q[1] = A.y;
    q[2] = B.x;
    q[3] = B.y;
}
__device__ __forceinline__ void load_part(const unsigned char *p, float &A, float &B) {
    const volatile float *q = reinterpret_cast<const volatile float *>(p);
    A = q[0];
    B = q[1];
}
__device__ __forceinline__ void load_part(const unsigned char *p, float2 &A, float2 &B) {
    const volatile float *q = reinterpret_cast<const volatile float *>(p);
    A = make_float2(q[0], q[1]);
    B = make_float2(q[2], q[3]);
}

// A segment, and what a worker keeps about its part of one.
struct SegDesc {
    int64_t row;       // row of the segment
    int64_t pos0;      // position of its first element inside the row
    int64_t n;         // elements
    int32_t s;         // segment index in processing order
    int32_t nts;       // tiles
    bool valid;
};
template <class V>
struct PendingItem {
    ItemDesc d;
    V end_gate;            // backward: gate of the step right after the part
};
constexpr uint32_t LB_NO_ITEM = 0xffffffffu;

// KIND: K_SCAN (REVERSE selects the direction) or K_BWD.  Bulk loader, one segment per item.
// The CTA's last warp is the bookkeeper, the others are workers.  The CTA's segments are
// numbered k = 0, 1, 2, ... by all its warps alike; segment k uses the shared-memory buffers
// k & 1 (parts, incoming states) and the ticket slot k & 3, and the phases of their mbarriers
// follow from k.
template <class TR, int NCH, int KIND, bool REVERSE>
__global__ void __launch_bounds__(512, 1) lookback_kernel(const StreamParams p, const ShardParams sp) {
    using V = typename TR::V;
    using Raw = typename TR::Raw;
    constexpr int EPC = TR::EPC;
    constexpr int K = NCH * EPC;
    constexpr int TE = 32 * K;
    constexpr int TB = 32 * NCH * 16;
    constexpr bool BACK = (KIND == K_BWD);
    constexpr bool REV = REVERSE || BACK;
    constexpr int NIN = stream_nin(KIND);
    constexpr int NOUT = stream_nout(KIND);
    constexpr int STAGE_BYTES = lb_stage_bytes(NCH, KIND);
    constexpr int PREFIX_BYTES = lb_prefix_bytes(sizeof(V) == 8);
    const int NT = p.stages;                                  // tiles per worker and segment; 2 * NT stages per worker
    const int WARP_SMEM = lb_warp_smem(NCH, NT, KIND, sizeof(V) == 8);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    const int G = wpc - 1;                                    // workers
    const bool keeper = wib == G;
    unsigned char *wsm = smem_raw + static_cast<size_t>(wib) * WARP_SMEM;      // (workers only)
    constexpr bool STAGED = !BACK;                            // results leave through a staging tile
    constexpr int STAGING_BYTES = lb_staging_bytes(NCH, KIND);
    unsigned char *staging = wsm + 2 * NT * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(wsm + 2 * NT * STAGE_BYTES + STAGING_BYTES);
    unsigned char *lane_prefix = wsm + 2 * NT * STAGE_BYTES + STAGING_BYTES + 128;     // PREFIX_BYTES per stage and lane
    // the team's memory
    unsigned char *tsm = smem_raw + static_cast<size_t>(G) * WARP_SMEM;
    unsigned char *parts = tsm;                                              // [2][16] pairs: the workers' aggregates
    unsigned char *xin = tsm + 512;                                          // [2][16] values: the states entering the parts
    unsigned char *pdesc = tsm + 1024;                                       // [4][16] part descriptors of 32 bytes
    uint64_t *pub = reinterpret_cast<uint64_t *>(tsm + 832);                 // [2] the segment's aggregate is published
    uint64_t *xr = pub + 2;                                                  // [2] the incoming states are there
    uint64_t *dr = pub + 4;                                                  // [4] the part descriptors are there
    uint32_t *cnt = reinterpret_cast<uint32_t *>(tsm + 896);                 // [2] workers that have posted their part
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(tsm + 904);

    const int64_t W = static_cast<int64_t>(gridDim.x) * wpc;
    const int64_t T = p.T;
    const int64_t S = p.segs_per_row;
    const int64_t L = p.seg_elems;
    const unsigned char *gbase[3] = {static_cast<const unsigned char *>(p.in0), static_cast<const unsigned char *>(p.in1),
                                     static_cast<const unsigned char *>(p.in2)};
    unsigned char *obase[2] = {static_cast<unsigned char *>(p.out0), static_cast<unsigned char *>(p.out1)};
    const V *cin = static_cast<const V *>(p.carry_in);
    const V *hgate = static_cast<const V *>(p.halo_gate);
    const V *hstate = static_cast<const V *>(p.halo_state);

    // Tag of this launch's records: the launch epoch above fifteen one-bits.  Never zero, and never
    // equal to a carry tag of the chained plans (epoch above a segment number below 32767), which
    // may have left words in the same workspace.
    const uint32_t tag = (*reinterpret_cast<volatile uint32_t *>(p.ctrl + CTRL_EPOCH) << EPOCH_SHIFT) | 0x7fffu;
    const uint64_t S1 = lb_level_count(S), S2 = lb_level_count(static_cast<int64_t>(S1));
    const uint64_t per_row = static_cast<uint64_t>(S) + S1 + S2;
    unsigned char *records = p.records;

    // ---- time sharding
    const bool sharded = sp.world > 1;
    const int n_before = !sharded ? 0 : (REV ? sp.world - 1 - sp.rank : sp.rank);   // ranks earlier in processing order
    const int n_after = !sharded ? 0 : (REV ? sp.rank : sp.world - 1 - sp.rank);
    const uint32_t parity_slot = sp.call & 1u;
    unsigned char *xl = sharded ? sp.xchg[sp.rank] : nullptr;
    uint32_t status_bits = 0;

    if (lane == 0) {
        if (keeper) {
            for (int s = 0; s < 8; ++s) mbar_init(&pub[s], 1);       // pub[2], xr[2], dr[4]
            cnt[0] = 0;
            cnt[1] = 0;
            *abort_flag = 0;
        } else {
            for (int s = 0; s < 2 * NT; ++s) mbar_init(&bars[s], 1);
        }
        mbar_init_fence();
    }
    __syncthreads();

    // backward: the first gate of every row of this slice is the gate halo of the rank before
    if (BACK && sharded && sp.rank > 0) {
        const int64_t w = static_cast<int64_t>(blockIdx.x) * wpc + wib;
        unsigned char *peer = sp.xchg[sp.rank - 1];
        // the slot was last used two calls ago: the receiver must have finished that call
        bool ok = true;
        if (sp.call > 2) {
            ok = false;
            for (uint32_t poll = 0; poll < LB_WAIT_POLLS && !ok; ++poll) {
                ok = static_cast<int32_t>(static_cast<uint32_t>(ld_relaxed_sys_u64(xl + 8 * (sp.rank - 1))) - (sp.call - 2)) >= 0;
                if (!ok) __nanosleep(200);
            }
        }
        if (!ok) status_bits |= STATUS_LOOKBACK_TIMEOUT;
        for (int64_t r = w * 32 + lane; r < p.rows; r += W * 32) {
            const V g0 = TR::load_one(p.in0, r * T);
            unsigned char *slot = peer + xchg_halo_offset() + (static_cast<uint64_t>(parity_slot) * p.rows + r) * 16;
            if (ok) {
                if constexpr (sizeof(V) == 4) {
                    put_word<true>(slot, g0, sp.call);
                } else {
                    put_word<true>(slot, g0.x, sp.call);
                    put_word<true>(slot + 8, g0.y, sp.call);
                }
            }
        }
    }

    // ---- segments and parts
    auto describe_seg = [&](uint32_t q) -> SegDesc {
        SegDesc g;
        g.valid = q < static_cast<uint32_t>(p.items);
        g.row = 0; g.pos0 = 0; g.n = 0; g.s = 0; g.nts = 0;
        if (!g.valid) return g;
        // Tickets run over groups of rows, segment-major inside a group: the segment before this one
        // in its row was drawn a group's worth of tickets ago, so its aggregate (and those of all
        // earlier ones) is out when this one's look-back asks.  Unsharded, all rows are one group.
        // Sharded, a row's slice aggregate is due at the next rank as early as possible, and a
        // row is finished only a group's worth of segments after it was begun: groups of 16 rows,
        // 8 from eight ranks on, where every microsecond of lag per rank boundary is paid fourteen
        // times per step (measured on 1024 rows, a rank's slice of eight, forward / backward TB/s:
        // row-major 5.1 / 4.8, groups of 8 rows 5.5 / 5.3, 16 rows 5.5 / 5.4, 64 rows 5.6 / 5.5).
        const uint32_t rows_u = static_cast<uint32_t>(p.rows), ss = static_cast<uint32_t>(S);
        const uint32_t group = sp.world >= 8 ? LB_SHARDED_GROUP_ROWS / 2 : LB_SHARDED_GROUP_ROWS;
        const uint32_t R = sharded ? (rows_u < group ? rows_u : group) : rows_u;
        const uint32_t gi = q / (R * ss);
        const uint32_t left_rows = rows_u - gi * R;
        const uint32_t Rg = left_rows < R ? left_rows : R;
        const uint32_t w = q - gi * R * ss;
        const uint32_t sq = w / Rg;
        g.s = static_cast<int32_t>(sq);
        g.row = gi * R + (w - sq * Rg);
        const int64_t from_start = REV ? S - 1 - g.s : g.s;      // segments are aligned to the row start
        g.pos0 = from_start * L;
        const int64_t left = T - g.pos0;
        g.n = left < L ? left : L;
        g.nts = static_cast<int32_t>((g.n + TE - 1) / TE);
        return g;
    };
    // worker `g` takes the tiles g*NT, ..., g*NT + NT - 1 of the segment in processing order
    auto part_of = [&](const SegDesc &sg, int g) -> ItemDesc {
        ItemDesc d;
        d.valid = sg.valid;
        d.row0 = sg.row;
        d.s_log = sg.s;
        d.pos0 = sg.pos0;
        d.e_begin = sg.row * T + sg.pos0;
        d.n = 0;
        d.nt = 0;
        if (!sg.valid) return d;
        int c = sg.nts - g * NT;
        c = c < 0 ? 0 : (c > NT ? NT : c);
        if (c == 0) return d;
        const int m_lo = REV ? sg.nts - g * NT - c : g * NT;     // first tile of the part in memory order
        d.nt = c;
        d.pos0 = sg.pos0 + static_cast<int64_t>(m_lo) * TE;
        d.e_begin = sg.row * T + d.pos0;
        const int64_t left = sg.n - static_cast<int64_t>(m_lo) * TE;
        const int64_t full = static_cast<int64_t>(c) * TE;
        d.n = left < full ? left : full;
        return d;
    };
    auto tile_of_step = [&](const ItemDesc &d, int i) -> int { return REV ? d.nt - 1 - i : i; };
    auto tile_valid = [&](const ItemDesc &d, int t) -> int {
        const int64_t left = d.n - static_cast<int64_t>(t) * TE;
        return left < TE ? static_cast<int>(left) : TE;
    };

    // The map from the slice's start to the start of segment `s` of a row, from the records of
    // the segments of its block, the blocks of its super-block and the super-blocks before it
    // (fixed order: super-blocks, then blocks, then segments).  false when a wait expires.
    auto local_prefix = [&](unsigned char *row_rec, int s, V &preA, V &preB, const RecordWords *ahead) -> bool {
        preA = vone(V());
        preB = vzero(V());
        if (s == 0) return true;
        const int n2 = s >> 10;
        const unsigned char *base[3] = {
            row_rec + (static_cast<uint64_t>(s >> 5) << 5) * LB_RECORD_BYTES,
            row_rec + (static_cast<uint64_t>(S) + (static_cast<uint64_t>(s >> 10) << 5)) * LB_RECORD_BYTES,
            row_rec + (static_cast<uint64_t>(S) + S1) * LB_RECORD_BYTES};
        const int n[3] = {s & 31, (s >> 5) & 31, n2 < 32 ? n2 : 32};
        V Aw[3], Bw[3];
        bool ok = compose_three<V>(base, n, tag, lane, Aw, Bw, ahead);
        // further super-blocks of very long rows, 32 at a time, in order
        V A2 = Aw[2], B2 = Bw[2];
        for (int w0 = 32; w0 < n2 && ok; w0 += 32) {
            V Ax, Bx;
            const int nn = n2 - w0 < 32 ? n2 - w0 : 32;
            ok = compose_window<V, false>(row_rec + (static_cast<uint64_t>(S) + S1 + w0) * LB_RECORD_BYTES, LB_RECORD_BYTES, nn,
                                          tag, lane, Ax, Bx);
            B2 = vfma(Ax, B2, Bx);
            A2 = vmul(Ax, A2);
        }
        preA = A2;
        preB = B2;
        preB = vfma(Aw[1], preB, Bw[1]);
        preA = vmul(Aw[1], preA);
        preB = vfma(Aw[0], preB, Bw[0]);
        preA = vmul(Aw[0], preA);
        return ok;
    };

    // the records a look-back of segment `s` reads first, loaded ahead of time (real types)
    auto load_ahead = [&](unsigned char *row_rec, int s) -> RecordWords {
        const int n2 = s >> 10;
        const unsigned char *base[3] = {
            row_rec + (static_cast<uint64_t>(s >> 5) << 5) * LB_RECORD_BYTES,
            row_rec + (static_cast<uint64_t>(S) + (static_cast<uint64_t>(s >> 10) << 5)) * LB_RECORD_BYTES,
            row_rec + (static_cast<uint64_t>(S) + S1) * LB_RECORD_BYTES};
        const int n[3] = {s & 31, (s >> 5) & 31, n2 < 32 ? n2 : 32};
        return load_record_words(base, n, lane);
    };

    bool failed = false;
    // A wait that expires ends this warp's work: the status bit is set, the abort flag tells the
    // other warps of the CTA, whose waits on this warp then end at once.  Every warp gives up at
    // its first expired wait, so a launch whose partner rank never shows up ends after about one
    // bound, not one bound per item.
    auto give_up = [&](uint32_t bit) {
        status_bits |= bit;
        failed = true;
        if (lane == 0) *abort_flag = 1;
    };
    // the parts of buffer `b`, composed in worker order: inclusive in every lane (identity
    // beyond the last worker, so lane 31 holds the whole segment)
    auto compose_parts = [&](int b, V &a, V &bb) {
        a = vone(V());
        bb = vzero(V());
        if (lane < G) load_part(parts + (b * 16 + lane) * 16, a, bb);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const V Ap = shfl_up(a, d), Bp = shfl_up(bb, d);
            if (lane >= d) {
                bb = vfma(a, Bp, bb);
                a = vmul(a, Ap);
            }
        }
    };

    if (!keeper) {
        // =====================================================================================
        // Worker.
        const int g = wib;
        uint32_t phase_bits = 0;       // bit s: parity to wait for on stage s

        // step i of a part in slot `slot` lives in stage slot * NT + i.  Lane 0 arms the stage's
        // mbarrier, then one lane per stream issues its copy (and one more the 16 bytes of saved
        // states just below the tile).
        auto issue = [&](const ItemDesc &d, int slot, int i) {
            const int t = tile_of_step(d, i);
            const int stage = slot * NT + i;
            const uint32_t bytes = static_cast<uint32_t>(tile_valid(d, t)) * TR::ESIZE;
            const int64_t goff = (d.e_begin + static_cast<int64_t>(t) * TE) * TR::ESIZE;
            const bool halo = BACK && goff > 0;
            unsigned char *dst = wsm + stage * STAGE_BYTES;
            if (lane == 0) mbar_expect_tx(&bars[stage], bytes * NIN + (halo ? 16u : 0u));
            __syncwarp();
            if (lane < NIN) bulk_g2s(dst + lane * TB, gbase[lane] + goff, bytes, &bars[stage]);
            if (lane == NIN && halo) bulk_g2s(dst + NIN * TB, gbase[2] + goff - 16, 16, &bars[stage]);
        };
        // this worker's part of the CTA's k-th segment, once the bookkeeper has posted it
        // (32 bytes per worker: e_begin, pos0, n, nt, row, s; row < 0: no segment)
        auto take_part = [&](uint32_t k, SegDesc &sg, ItemDesc &d) {
            sg.valid = false;
            sg.row = 0; sg.pos0 = 0; sg.n = 0; sg.s = 0; sg.nts = 0;
            d.valid = false;
            d.e_begin = 0; d.row0 = 0; d.pos0 = 0; d.n = 0; d.s_log = 0; d.nt = 0;
            if (!__all_sync(0xffffffffu, team_wait(&dr[k & 3u], (k >> 2) & 1u, abort_flag))) {
                if (!*abort_flag) give_up(STATUS_LOOKBACK_TIMEOUT);
                failed = true;
                return;
            }
            const unsigned char *pd = pdesc + ((k & 3u) * 16 + g) * 32;
            const longlong2 w0 = *reinterpret_cast<const longlong2 *>(pd);
            const int4 w1 = *reinterpret_cast<const int4 *>(pd + 16);
            if (w1.z < 0) return;
            sg.valid = true;
            sg.row = w1.z;
            sg.s = w1.w;
            d.valid = true;
            d.e_begin = w0.x;
            d.pos0 = w0.y;
            d.n = w1.x;
            d.nt = w1.y;
            d.row0 = w1.z;
            d.s_log = w1.w;
        };
        // backward: the gate of the step right after a part, loaded when the part is known (the
        // load's latency hides behind the scan pass that runs meanwhile)
        auto end_gate_raw = [&](const ItemDesc &d) -> Raw {
            Raw r = 0;
            if (BACK && d.valid && d.nt > 0 && d.pos0 + d.n < T) r = TR::load_raw(p.in0, d.e_begin + d.n);
            return r;
        };
        // ... and decoded, or taken from the halos, when the part's aggregate pass starts
        auto end_gate = [&](const ItemDesc &d, Raw raw, bool &ok) -> V {
            V gt = vone(V());
            if (!BACK || d.nt == 0) return gt;
            if (d.pos0 + d.n < T) return TR::decode(raw);
            if (sharded && sp.rank + 1 < sp.world) {
                // first gate of the next rank's slice, stored into this rank's exchange buffer
                const unsigned char *slot = xl + xchg_halo_offset() + (static_cast<uint64_t>(parity_slot) * p.rows + d.row0) * 16;
                bool got = false;
                for (uint32_t poll = 0; poll < LB_WAIT_POLLS && !got; ++poll) {
                    if constexpr (sizeof(V) == 4) {
                        got = get_word<true>(slot, sp.call, gt);
                    } else {
                        const bool a = get_word<true>(slot, sp.call, gt.x);
                        const bool b = get_word<true>(slot + 8, sp.call, gt.y);
                        got = a && b;
                    }
                    if (!got) __nanosleep(100);
                }
                if (!got) {
                    ok = false;
                    gt = vone(V());
                }
                return gt;
            }
            if (hgate) gt = hgate[d.row0];
            return gt;
        };

        // One tile from its stage into registers, ready for the two passes: a[] = the gates that
        // multiply the state entering each element (shifted by one step for the backward), b[] = the
        // additive terms; beyond the row's end the identity.
        auto fetch = [&](const PendingItem<V> &it, int slot, int i, V *a, V *b, V &next_gate, int &nvalid) {
            const int t = tile_of_step(it.d, i);
            nvalid = tile_valid(it.d, t);
            const unsigned char *stg = wsm + (slot * NT + i) * STAGE_BYTES;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                TR::unpack(*reinterpret_cast<const uint4 *>(stg + 0 * TB + (lane * NCH + c) * 16), &a[c * EPC]);
                TR::unpack(*reinterpret_cast<const uint4 *>(stg + 1 * TB + (lane * NCH + c) * 16), &b[c * EPC]);
            }
            if (BACK) {
                const V g0 = a[0];
                V up = shfl_down(g0, 1);
                if (lane == 31) up = next_gate;
#pragma unroll
                for (int j = 0; j < K - 1; ++j) a[j] = vconj(a[j + 1]);
                a[K - 1] = vconj(up);
                next_gate = shfl_idx(g0, 0);
            }
            if (nvalid < TE) {
                const int jv = nvalid - lane * K;
                const V gate_end = BACK ? vconj(it.end_gate) : vone(V());
#pragma unroll
                for (int j = 0; j < K; ++j) {
                    if (j >= jv) {
                        a[j] = vone(V());
                        b[j] = vzero(V());
                    } else if (BACK && j + 1 >= jv) {
                        a[j] = gate_end;
                    }
                }
            }
        };

        // ---------------- aggregate pass of this worker's part of segment `kk` (in `slot`): lane
        // prefixes, the part's aggregate into the team's memory; the worker that posts last
        // publishes the segment
        auto aggregate = [&](PendingItem<V> &it, const SegDesc &sg, int slot, uint32_t kk, Raw gate_raw) {
            bool waits_ok = true;
            it.end_gate = end_gate(it.d, gate_raw, waits_ok);
            V segA = vone(V()), segB = vzero(V());      // map from the part's start to the current tile's start
            V next_gate = it.end_gate;
            for (int i = 0; i < it.d.nt; ++i) {
                const int stage = slot * NT + i;
                bool ok = mbar_wait_bounded_suspended(&bars[stage], (phase_bits >> stage) & 1u, LOAD_WAIT_POLLS, 2000);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    give_up(STATUS_LOAD_TIMEOUT);
                    return;
                }
                phase_bits ^= 1u << stage;
                V a[K], b[K];
                int nvalid;
                fetch(it, slot, i, a, b, next_gate, nvalid);
                V A, B;
                {
                    constexpr int JF = REV ? K - 1 : 0;
                    A = a[JF];
                    B = b[JF];
#pragma unroll
                    for (int q = 1; q < K; ++q) {
                        const int j = REV ? K - 1 - q : q;
                        B = vfma(a[j], B, b[j]);
                        A = vmul(A, a[j]);
                    }
                }
                // inclusive Kogge-Stone over the lanes in processing order; the map that enters the
                // tile (segA, segB) goes in through the first lane
                const int ll = REV ? 31 - lane : lane;
                if (ll == 0) {
                    B = vfma(A, segB, B);
                    A = vmul(A, segA);
                }
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const V Ap = REV ? shfl_down(A, d) : shfl_up(A, d);
                    const V Bp = REV ? shfl_down(B, d) : shfl_up(B, d);
                    if (ll >= d) {
                        B = vfma(A, Bp, B);
                        A = vmul(A, Ap);
                    }
                }
                // map from the part's start to this lane's first element
                V pA = REV ? shfl_down(A, 1) : shfl_up(A, 1);
                V pB = REV ? shfl_down(B, 1) : shfl_up(B, 1);
                if (ll == 0) {
                    pA = segA;
                    pB = segB;
                }
                if constexpr (sizeof(V) == 4) {
                    *reinterpret_cast<float2 *>(lane_prefix + (stage * 32 + lane) * PREFIX_BYTES) = make_float2(pA, pB);
                } else {
                    *reinterpret_cast<float4 *>(lane_prefix + (stage * 32 + lane) * PREFIX_BYTES) = make_float4(pA.x, pA.y, pB.x, pB.y);
                }
                segA = shfl_idx(A, REV ? 0 : 31);
                segB = shfl_idx(B, REV ? 0 : 31);
            }
            // post the part; the worker that finds all others posted goes on for the segment
            const int b = static_cast<int>(kk & 1u);
            uint32_t posted = 0;
            if (lane == 0) {
                store_part(parts + (b * 16 + g) * 16, segA, segB);
                __threadfence_block();
                posted = atomicAdd(&cnt[b], 1u);
            }
            const bool last = __shfl_sync(0xffffffffu, posted, 0) == static_cast<uint32_t>(G - 1);
            if (last) {
                if (lane == 0) {
                    cnt[b] = 0;
                    __threadfence_block();
                }
                __syncwarp();
                V ta, tb;
                compose_parts(b, ta, tb);
                const V totA = shfl_idx(ta, 31), totB = shfl_idx(tb, 31);
                unsigned char *row_rec = records + static_cast<uint64_t>(sg.row) * per_row * LB_RECORD_BYTES;
                const int s = sg.s;
                if (lane == 0) {
                    put_pair<false>(row_rec + static_cast<uint64_t>(s) * LB_RECORD_BYTES, totA, totB, tag);
                    mbar_arrive(&pub[b]);
                }
                // Closing duties.  The last segment of a block publishes the block's aggregate (this
                // segment after the 31 before it), the last block of a super-block the super-block's.
                // They wait only for aggregates of segments drawn earlier, which nobody holds back; the
                // records are there long before the look-backs that read them.  Only full blocks and
                // super-blocks are ever read.
                if ((s & 31) == 31) {
                    V A0, B0;
                    bool ok = compose_window<V, false>(row_rec + static_cast<uint64_t>(s - 31) * LB_RECORD_BYTES, LB_RECORD_BYTES, 31,
                                                       tag, lane, A0, B0);
                    const V Ab = vmul(totA, A0), Bb = vfma(totA, B0, totB);
                    if (ok && lane == 0) put_pair<false>(row_rec + (static_cast<uint64_t>(S) + (s >> 5)) * LB_RECORD_BYTES, Ab, Bb, tag);
                    if (ok && ((s >> 5) & 31) == 31) {
                        V A1, B1;
                        ok = compose_window<V, false>(row_rec + (static_cast<uint64_t>(S) + (s >> 5) - 31) * LB_RECORD_BYTES,
                                                      LB_RECORD_BYTES, 31, tag, lane, A1, B1);
                        if (ok && lane == 0)
                            put_pair<false>(row_rec + (static_cast<uint64_t>(S) + S1 + (s >> 10)) * LB_RECORD_BYTES, vmul(Ab, A1),
                                            vfma(Ab, B1, Bb), tag);
                    }
                    if (!ok) waits_ok = false;
                }
                // The slice of the row ends with this segment: the slice's aggregate goes to the ranks that
                // come later in processing order, as early as possible (they all wait for it).
                if (sharded && s == S - 1 && n_after > 0 && waits_ok) {
                    V preA, preB;
                    bool ok = local_prefix(row_rec, s, preA, preB, nullptr);
                    const V Ps = vmul(totA, preA), Ss = vfma(totA, preB, totB);
                    if (ok && lane < n_after) {
                        const int target = REV ? sp.rank - 1 - lane : sp.rank + 1 + lane;
                        // the slot was last used two calls ago: the receiver must have finished that call
                        ok = sp.call <= 2;
                        for (uint32_t poll = 0; poll < LB_WAIT_POLLS && !ok; ++poll) {
                            ok = static_cast<int32_t>(static_cast<uint32_t>(ld_relaxed_sys_u64(xl + 8 * target)) - (sp.call - 2)) >= 0;
                            if (!ok) __nanosleep(200);
                        }
                        if (ok) {
                            unsigned char *slot_rec = sp.xchg[target] + xchg_carry_offset(p.rows) +
                                                      ((static_cast<uint64_t>(parity_slot) * sp.world + sp.rank) * p.rows + sg.row) * LB_RECORD_BYTES;
                            put_pair<true>(slot_rec, Ps, Ss, sp.call);
                        }
                    }
                    if (!__all_sync(0xffffffffu, ok)) waits_ok = false;
                }
            }
            if (!waits_ok) give_up(STATUS_LOOKBACK_TIMEOUT);
        };

        uint32_t k = 0;
        SegDesc sc, sn;
        PendingItem<V> cur, nxt;
        take_part(0, sc, cur.d);
        sn = sc;
        sn.valid = false;
        cur.end_gate = vone(V());
        nxt = cur;
        nxt.d.valid = false;
        nxt.d.nt = 0;
        int cur_slot = 0;
        Raw nxt_gate_raw = 0;
        if (sc.valid && !failed) {
            for (int i = 0; i < cur.d.nt; ++i) issue(cur.d, 0, i);
            const Raw g_raw = end_gate_raw(cur.d);
            take_part(1, sn, nxt.d);
            if (sn.valid) {
                for (int i = 0; i < nxt.d.nt; ++i) issue(nxt.d, 1, i);
            }
            nxt_gate_raw = end_gate_raw(nxt.d);
            if (!failed) aggregate(cur, sc, 0, 0, g_raw);
        }

        while (sc.valid && !failed) {
            const int nxt_slot = cur_slot ^ 1;
            const int64_t row = sc.row;

            // ---------------- aggregate pass of the segment after this one
            if (sn.valid) aggregate(nxt, sn, nxt_slot, k + 1, nxt_gate_raw);
            if (failed) break;

            // ---------------- the state entering this worker's part, from the bookkeeper
            if (!__all_sync(0xffffffffu, team_wait(&xr[k & 1u], (k >> 1) & 1u, abort_flag))) {
                if (!*abort_flag) give_up(STATUS_LOOKBACK_TIMEOUT);
                break;
            }
            const V x_in = *reinterpret_cast<const V *>(xin + ((k & 1u) * 16 + g) * 8);
            // the segment after the next: its tiles refill the stages as they drain (the bookkeeper
            // drew its ticket right after this segment's look-back, which is over by now)
            SegDesc sa = sn;
            sa.valid = false;
            PendingItem<V> aft;
            aft.d = nxt.d;
            aft.d.valid = false;
            aft.d.nt = 0;
            if (sn.valid) take_part(k + 2, sa, aft.d);
            if (failed) break;
            aft.end_gate = vone(V());
            const Raw aft_gate_raw = end_gate_raw(aft.d);
            const int aft_nt = sa.valid ? aft.d.nt : 0;

            // ---------------- scan pass from shared memory
            {
                V next_gate = cur.end_gate;
                const int nt = cur.d.nt;
                for (int i = 0; i < nt; ++i) {
                    V a[K], b[K];
                    int nvalid;
                    fetch(cur, cur_slot, i, a, b, next_gate, nvalid);
                    const int t = tile_of_step(cur.d, i);
                    const int64_t toff = static_cast<int64_t>(t) * TE;
                    const int stage = cur_slot * NT + i;
                    unsigned char *stg = wsm + stage * STAGE_BYTES;
                    V xp[BACK ? K : 1];
                    V x_below = vzero(V());
                    if (BACK) {
#pragma unroll
                        for (int c = 0; c < NCH; ++c)
                            TR::unpack(*reinterpret_cast<const uint4 *>(stg + 2 * TB + (lane * NCH + c) * 16), &xp[c * EPC]);
                        if (cur.d.pos0 + toff != 0) {
                            V hv[EPC];
                            TR::unpack(*reinterpret_cast<const uint4 *>(stg + NIN * TB), hv);
                            x_below = hv[EPC - 1];
                        } else if (hstate) {
                            x_below = hstate[row];
                        }
                    }
                    // the state entering this lane's first element
                    V x;
                    if constexpr (sizeof(V) == 4) {
                        const float2 pf = *reinterpret_cast<const float2 *>(lane_prefix + (stage * 32 + lane) * PREFIX_BYTES);
                        x = vfma(pf.x, x_in, pf.y);
                    } else {
                        const float4 pf = *reinterpret_cast<const float4 *>(lane_prefix + (stage * 32 + lane) * PREFIX_BYTES);
                        x = vfma(make_float2(pf.x, pf.y), x_in, make_float2(pf.z, pf.w));
                    }
                    if constexpr (STAGED) {
                        // the tile is in registers: its stage takes the matching tile of the segment
                        // after the next
                        __syncwarp();
                        fence_async_smem();
                        if (i < aft_nt) issue(aft.d, cur_slot, i);
                    }
#pragma unroll
                    for (int q = 0; q < K; ++q) {
                        const int j = REV ? K - 1 - q : q;
                        x = vfma(a[j], x, b[j]);
                        b[j] = x;
                    }
                    if (BACK) {
                        // d_gates[t] = conj(x[t-1]) * g[t]
                        V dn = shfl_up(xp[K - 1], 1);
                        if (lane == 0) dn = x_below;
#pragma unroll
                        for (int j = K - 1; j >= 1; --j) a[j] = vmul(vconj(xp[j - 1]), b[j]);
                        a[0] = vmul(vconj(dn), b[0]);
                    }
                    if constexpr (STAGED) {
                        // results into the staging tile (once the store before has read it), then out
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
#pragma unroll
                        for (int c = 0; c < NCH; ++c)
                            *reinterpret_cast<uint4 *>(staging + (lane * NCH + c) * 16) = TR::pack(&b[c * EPC]);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            bulk_s2g(obase[0] + (cur.d.e_begin + toff) * TR::ESIZE, staging, static_cast<uint32_t>(nvalid) * TR::ESIZE);
                            bulk_commit();
                        }
                    } else {
                        // results over the inputs of the stage, then out by bulk copies
                        __syncwarp();
#pragma unroll
                        for (int c = 0; c < NCH; ++c) {
                            *reinterpret_cast<uint4 *>(stg + 1 * TB + (lane * NCH + c) * 16) = TR::pack(&b[c * EPC]);
                            if (NOUT > 1) *reinterpret_cast<uint4 *>(stg + 2 * TB + (lane * NCH + c) * 16) = TR::pack(&a[c * EPC]);
                        }
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t bytes = static_cast<uint32_t>(nvalid) * TR::ESIZE;
                            const int64_t goff = (cur.d.e_begin + toff) * TR::ESIZE;
                            bulk_s2g(obase[0] + goff, stg + 1 * TB, bytes);
                            if (NOUT > 1) bulk_s2g(obase[1] + goff, stg + 2 * TB, bytes);
                            bulk_commit();
                            // the store of the stage before this one has read its data: refill that stage
                            if (i > 0) bulk_wait_read<1>();
                        }
                        __syncwarp();
                        if (i > 0 && i - 1 < aft_nt) issue(aft.d, cur_slot, i - 1);
                    }
                }
                if constexpr (STAGED) {
                    // stages beyond this part's tiles
                    for (int i = nt; i < aft_nt; ++i) issue(aft.d, cur_slot, i);
                } else {
                    if (lane == 0) bulk_wait_read<0>();
                    __syncwarp();
                    for (int i = nt > 0 ? nt - 1 : 0; i < aft_nt; ++i) issue(aft.d, cur_slot, i);
                }
            }
            if (failed) break;
            cur = nxt;
            sc = sn;
            nxt = aft;
            sn = sa;
            nxt_gate_raw = aft_gate_raw;
            cur_slot = nxt_slot;
            ++k;
        }
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
    } else {
        // =====================================================================================
        // Bookkeeper: tickets and look-backs.
        auto draw = [&]() -> uint32_t {
            uint32_t t = 0;
            if (lane == 0) t = atomicAdd(p.ctrl + CTRL_TICKET, 1u);
            return __shfl_sync(0xffffffffu, t, 0);
        };
        // the parts of segment `q` (the CTA's k-th), one descriptor per worker
        auto post_ticket = [&](uint32_t k, uint32_t q) {
            const SegDesc sg = describe_seg(q);
            const ItemDesc d = part_of(sg, lane < G ? lane : 0);
            if (lane < G) {
                unsigned char *pd = pdesc + ((k & 3u) * 16 + lane) * 32;
                *reinterpret_cast<longlong2 *>(pd) = make_longlong2(d.e_begin, d.pos0);
                *reinterpret_cast<int4 *>(pd + 16) = make_int4(static_cast<int>(d.n), d.nt, sg.valid ? static_cast<int>(sg.row) : -1, sg.s);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&dr[k & 3u]);
            // the segment's inputs on their way into L2 already: the workers ask for their tiles a
            // scan pass later and need them right after it
            if (sg.valid && lane < NIN)
                bulk_prefetch_l2(gbase[lane] + (sg.row * T + sg.pos0) * TR::ESIZE, static_cast<uint32_t>(sg.n * TR::ESIZE));
        };
        uint32_t q_cur = draw();
        if (q_cur >= static_cast<uint32_t>(p.items)) q_cur = LB_NO_ITEM;
        post_ticket(0, q_cur);
        uint32_t q_nxt = LB_NO_ITEM;
        if (q_cur != LB_NO_ITEM) {
            q_nxt = draw();
            if (q_nxt >= static_cast<uint32_t>(p.items)) q_nxt = LB_NO_ITEM;
        }
        post_ticket(1, q_nxt);

        RecordWords ahead;
        for (int w = 0; w < 6; ++w) ahead.w[w] = 0;
        bool have_ahead = false;
        uint64_t xahead[2] = {0, 0};                  // time sharding: the earlier ranks' slice aggregates of the next segment's row
        // lane i reads the aggregate of the i-th rank in processing order
        const int xfirst = REV ? sp.world - 1 : 0;
        const int64_t xstep = (REV ? -1 : 1) * static_cast<int64_t>(p.rows) * LB_RECORD_BYTES;
        auto xbase = [&](int64_t row) -> const unsigned char * {
            return xl + xchg_carry_offset(p.rows) + ((static_cast<uint64_t>(parity_slot) * sp.world + xfirst) * p.rows + row) * LB_RECORD_BYTES;
        };
        for (uint32_t k = 0; q_cur != LB_NO_ITEM && !failed; ++k) {
            const SegDesc sg = describe_seg(q_cur);
            const int b = static_cast<int>(k & 1u);
            if (!__all_sync(0xffffffffu, team_wait(&pub[b], (k >> 1) & 1u, abort_flag))) {
                if (!*abort_flag) give_up(STATUS_LOOKBACK_TIMEOUT);
                break;
            }
            // the map from the segment's start to the start of every worker's part
            V pa, pb;
            compose_parts(b, pa, pb);
            pa = shfl_up(pa, 1);
            pb = shfl_up(pb, 1);
            if (lane == 0) {
                pa = vone(V());
                pb = vzero(V());
            }
            // ---------------- look back
            const int64_t row = sg.row;
            const int s = sg.s;
            unsigned char *row_rec = records + static_cast<uint64_t>(row) * per_row * LB_RECORD_BYTES;
            V preA, preB;                                  // map from the slice's start to the segment's start
            bool lb_ok = local_prefix(row_rec, s, preA, preB, have_ahead ? &ahead : nullptr);
            // state entering the slice: the caller's, or the fold of the earlier ranks' aggregates
            V x_slice = cin ? cin[row] : vzero(V());
            if (n_before > 0 && lb_ok) {
                V Ar, Br;
                lb_ok = compose_window<V, true>(xbase(row), xstep, n_before, sp.call, lane, Ar, Br, have_ahead ? xahead : nullptr);
                x_slice = vfma(Ar, x_slice, Br);
            }
            // forward: the state entering the slice is what the backward needs below its first step
            if (!REV && s == 0 && sp.carry_save && lane == 0) static_cast<V *>(sp.carry_save)[row] = x_slice;
            if (!lb_ok) {
                give_up(STATUS_LOOKBACK_TIMEOUT);
                break;
            }
            // The ticket of the segment after the next is drawn only now, after the look-back: from
            // this draw to the publication of that segment's aggregate nothing waits for a look-back,
            // so a drawn segment is never held back by this warp waiting for other CTAs.  (Drawn
            // earlier, such waits chained up across CTAs.)  The number arrives while the states go
            // out and the next look-back's records are asked for.
            uint32_t raw_aft = 0;
            if (q_nxt != LB_NO_ITEM && lane == 0) raw_aft = atomicAdd(p.ctrl + CTRL_TICKET, 1u);
            const V x_seg = vfma(preA, x_slice, preB);
            if (lane < G) *reinterpret_cast<V *>(xin + (b * 16 + lane) * 8) = vfma(pa, x_seg, pb);
            __syncwarp();
            if (lane == 0) mbar_arrive(&xr[b]);
            // real types: the records the next segment's look-back will read, loaded now and used
            // once that segment's aggregate is out (what is missing then is polled for)
            have_ahead = false;
            if constexpr (sizeof(V) == 4) {
                if (q_nxt != LB_NO_ITEM) {
                    const SegDesc sx = describe_seg(q_nxt);
                    ahead = load_ahead(records + static_cast<uint64_t>(sx.row) * per_row * LB_RECORD_BYTES, sx.s);
                    if (lane < n_before) {
                        const unsigned char *xb = xbase(sx.row) + lane * xstep;
                        xahead[0] = ld_relaxed_sys_u64(xb);
                        xahead[1] = ld_relaxed_sys_u64(xb + 8);
                    }
                    have_ahead = true;
                }
            }
            uint32_t q_aft = LB_NO_ITEM;
            if (q_nxt != LB_NO_ITEM) {
                q_aft = __shfl_sync(0xffffffffu, raw_aft, 0);
                if (q_aft >= static_cast<uint32_t>(p.items)) q_aft = LB_NO_ITEM;
            }
            post_ticket(k + 2, q_aft);
            q_cur = q_nxt;
            q_nxt = q_aft;
        }
    }

    // a rank that leaves tells the others: its reads of this call's exchange slots are over
    if (sharded) {
        uint32_t last = 0;
        if (lane == 0) {
            __threadfence();
            last = (atomicAdd(p.ctrl + CTRL_DONE + 8, 1u) == static_cast<uint32_t>(W - 1)) ? 1u : 0u;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            if (lane < sp.world) st_relaxed_sys_u64(sp.xchg[lane] + 8 * sp.rank, sp.call);
            if (lane == 0) p.ctrl[CTRL_DONE + 8] = 0;
            __threadfence_system();
        }
    }
    leave_kernel(p, W, status_bits, lane);
}

}  // namespace ascan

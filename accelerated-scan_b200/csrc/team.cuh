// Warp-team scan kernel: for matrices with fewer rows than warps.
//
// A single warp streams a row at a few GB/s because the steps of a tile depend on each
// other; with fewer rows than warps the chained stream kernel therefore cannot fill the
// memory system.  Here G consecutive warps of a CTA form a TEAM that works on one item (a
// segment of a row) together:
//   * the tiles of the item are dealt round-robin to the team's warps (warp g takes the
//     tiles g, g+G, ... in processing order), each warp with its own shared-memory ring fed
//     by bulk asynchronous copies, exactly as in the stream kernel;
//   * everything in a tile that does not need the incoming state -- loading, the lane
//     aggregates, the Kogge-Stone combine across lanes -- runs as soon as the data is there;
//   * the incoming state then arrives from the warp that owns the tile before, through a
//     sequence-numbered mailbox in shared memory; the warp immediately forwards
//     A_tile*x_in + B_tile to the next warp and only afterwards finishes its own tile.
//     The serial part per tile is one mailbox hop, so a row advances G times faster.
// Items (coarse and fine segments, segment-major tickets, per-row tagged carry records
// between segments, launch epoch) are those of the stream kernel; the team leader draws
// the tickets and posts them to its team.  The team meets at a named barrier after every
// item.  All waits are bounded; a warp that gives up raises the team's abort flag.
//
// Kinds: forward scan (optionally reversed) and the fused backward.  Rows are one item or
// split into segments (never grouped), the bulk loader is required.
#pragma once

#include "stream.cuh"

namespace ascan {

constexpr int TEAM_SMEM_BYTES = 384;          // per team: 16 mailboxes of 16 bytes, ticket ring, abort flag
constexpr uint32_t MAIL_WAIT_POLLS = 1u << 24;

__host__ __device__ constexpr int team_stage_bytes(int nch, int kind) {
    return stream_nin(kind) * 32 * nch * 16 + ((kind == K_BWD || kind == K_REDUCE_BWD) ? 128 : 0);
}
__host__ __device__ constexpr int team_warp_smem(int nch, int stages, int kind) {
    const int tb = 32 * nch * 16;
    return stages * team_stage_bytes(nch, kind) + 2 * stream_nout(kind) * tb + 128;
}

// (the forward kinds run with up to 16 warps per CTA, the backward kinds with 12)
template <class TR, int NCH, int KIND, bool REVERSE>
__global__ void __launch_bounds__((KIND == K_BWD || KIND == K_REDUCE_BWD) ? 384 : 512, 1) team_kernel(const StreamParams p) {
    using V = typename TR::V;
    constexpr int EPC = TR::EPC;
    constexpr int K = NCH * EPC;
    constexpr int TE = 32 * K;
    constexpr int TB = 32 * NCH * 16;
    constexpr bool BACK = (KIND == K_BWD || KIND == K_REDUCE_BWD);     // gates shifted by one step
    constexpr bool FULL_BWD = (KIND == K_BWD);                          // ... and the d_gates epilogue
    constexpr bool REDUCE = (KIND == K_REDUCE || KIND == K_REDUCE_BWD); // carry only (real dtypes)
    constexpr bool REV = REVERSE || BACK;
    static_assert(!REDUCE || sizeof(typename TR::V) == 4, "team reductions carry two values in two 64-bit words");
    constexpr int NIN = stream_nin(KIND);
    constexpr int NOUT = stream_nout(KIND);
    constexpr int STAGE_BYTES = team_stage_bytes(NCH, KIND);
    const int NSTG = p.stages;
    const int WARP_SMEM = team_warp_smem(NCH, p.stages, KIND);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    const int G = p.team_size;
    const int g = wib % G;                 // position in the team
    const int team = wib / G;              // team inside the CTA
    const bool leader = (g == 0);
    unsigned char *wsm = smem_raw + static_cast<size_t>(wib) * WARP_SMEM;
    unsigned char *stage_base = wsm;
    unsigned char *out_base = wsm + NSTG * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(out_base + 2 * NOUT * TB);
    unsigned char *tsm = smem_raw + static_cast<size_t>(wpc) * WARP_SMEM + team * TEAM_SMEM_BYTES;
    volatile uint32_t *mail_seq = reinterpret_cast<volatile uint32_t *>(tsm);          // [g*4]
    volatile float *mail_val = reinterpret_cast<volatile float *>(tsm);                // [g*4 + 2], [g*4 + 3]
    volatile unsigned long long *mail_word = reinterpret_cast<volatile unsigned long long *>(tsm);   // [g*2], real types
    volatile unsigned long long *tix = reinterpret_cast<volatile unsigned long long *>(tsm + 256);   // ring of 4
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(tsm + 288);

    const int64_t W = static_cast<int64_t>(gridDim.x) * wpc;
    const int64_t T = p.T;
    const bool split = p.segs_per_row > 1;
    const unsigned char *gbase[3] = {static_cast<const unsigned char *>(p.in0), static_cast<const unsigned char *>(p.in1),
                                     static_cast<const unsigned char *>(p.in2)};
    unsigned char *obase[2] = {static_cast<unsigned char *>(p.out0), static_cast<unsigned char *>(p.out1)};
    const V *cin = static_cast<const V *>(p.carry_in);
    const V *hgate = static_cast<const V *>(p.halo_gate);
    const V *hstate = static_cast<const V *>(p.halo_state);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(p.ctrl + CTRL_EPOCH) << EPOCH_SHIFT;

    auto team_barrier = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(G * 32) : "memory"); };

    if (lane == 0) {
        for (int s = 0; s < NSTG; ++s) mbar_init(&bars[s], 1);
        mbar_init_fence();
        if (leader) {
            for (int i = 0; i < TEAM_SMEM_BYTES / 4; ++i) reinterpret_cast<volatile uint32_t *>(tsm)[i] = 0;
        }
    }
    __syncwarp();
    team_barrier();

    // ---- tickets: the leader draws, everybody learns the number through the ticket ring
    bool failed = false;
    uint32_t status_bits = 0;
    auto draw = [&]() -> uint32_t {
        uint32_t t = 0;
        if (leader && lane == 0) t = atomicAdd(p.ctrl + CTRL_TICKET, 1u);
        return t;
    };
    auto resolve = [&](uint32_t raw, uint32_t n) -> int64_t {
        // n = running number of the item inside the team; ring entry {n+1, ticket}
        unsigned long long word = 0;
        if (leader) {
            const uint32_t q = __shfl_sync(0xffffffffu, raw, 0);
            word = (static_cast<unsigned long long>(q) << 32) | (n + 1u);
            if (lane == 0) tix[n & 3u] = word;
        } else {
            bool got = false;
            for (uint32_t poll = 0; poll < MAIL_WAIT_POLLS; ++poll) {
                word = tix[n & 3u];
                if (static_cast<uint32_t>(word) == n + 1u) {
                    got = true;
                    break;
                }
                if (*abort_flag) break;
                if (poll > 64) __nanosleep(40);
            }
            if (!got) {
                failed = true;
                status_bits |= STATUS_LOOKBACK_TIMEOUT;
                *abort_flag = 1;
                return p.items;          // an invalid item: the warp winds down
            }
        }
        return static_cast<int64_t>(word >> 32);
    };
    auto describe = [&](int64_t q) -> ItemDesc {
        ItemDesc d;
        d.valid = q < p.items;
        d.e_begin = 0; d.row0 = 0; d.pos0 = 0; d.s_log = 0; d.n = 0; d.nt = 0;
        if (!d.valid) return d;
        if (!split) {
            d.row0 = q;
            d.e_begin = q * T;
            d.n = T;
        } else {
            const uint32_t qq = static_cast<uint32_t>(q), rg = static_cast<uint32_t>(p.row_groups);
            const uint32_t sl = qq / rg;
            d.s_log = static_cast<int32_t>(sl);
            d.row0 = qq - sl * rg;
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
    // bulk loader: the tile of every stream; for the backward also the 16-byte chunk of saved
    // states just below the tile and the 16-byte chunk of gates just above it (both aligned,
    // because tiles start and end on 16 bytes)
    auto issue = [&](const ItemDesc &d, int t, int s) {
        const int valid = tile_valid(d, t);
        const uint32_t bytes = static_cast<uint32_t>(valid) * TR::ESIZE;
        const int64_t goff = (d.e_begin + static_cast<int64_t>(t) * TE) * TR::ESIZE;
        const bool below = FULL_BWD && goff > 0;
        const bool above = BACK && (d.pos0 + static_cast<int64_t>(t) * TE + valid < T);
        mbar_expect_tx(&bars[s], bytes * NIN + (below ? 16u : 0u) + (above ? 16u : 0u));
        unsigned char *dst = stage_base + s * STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < NIN; ++k) bulk_g2s(dst + k * TB, gbase[k] + goff, bytes, &bars[s]);
        if (below) bulk_g2s(dst + NIN * TB, gbase[FULL_BWD ? 2 : 0] + goff - 16, 16, &bars[s]);
        if (above) bulk_g2s(dst + NIN * TB + 16, gbase[0] + goff + bytes, 16, &bars[s]);
    };

    uint32_t n_item = 0;          // running number of the current item inside the team
    uint32_t step_base = 0;       // tiles of all earlier items: mailbox sequence numbers continue across items
    ItemDesc cur = describe(resolve(draw(), n_item));
    uint32_t raw_next = draw();
    bool nxt_ready = false;
    ItemDesc nxt = cur;
    auto need_next = [&]() {
        if (!nxt_ready) {
            nxt = describe(cur.valid ? resolve(raw_next, n_item + 1) : p.items);
            nxt_ready = true;
        }
    };

    // producer cursor over this warp's tiles (g, g+G, ...) of the current and the next item
    bool prod_in_next = false;
    int p_i = g;
    int in_flight = 0;
    int ps = 0;
    auto produce = [&]() {
        while (in_flight < NSTG) {
            if (!prod_in_next) {
                if (p_i < cur.nt) {
                    if (lane == 0) issue(cur, tile_of_step(cur, p_i), ps);
                } else {
                    need_next();
                    if (!nxt.valid) break;
                    prod_in_next = true;
                    p_i = g;
                    continue;
                }
            } else {
                if (p_i < nxt.nt) {
                    if (lane == 0) issue(nxt, tile_of_step(nxt, p_i), ps);
                } else {
                    break;
                }
            }
            p_i += G;
            ++in_flight;
            if (++ps == NSTG) ps = 0;
        }
    };
    // everybody has the first ticket (or the team gives up together)
    team_barrier();
    if (*abort_flag) failed = true;
    if (cur.valid && !failed) produce();

    int cs = 0;
    uint32_t parity = 0;
    uint32_t step_count = 0;

    // what the first tile of an item needs from outside: the state published by the previous
    // segment of the row (fetched early, checked late, as in the stream kernel)
    // (reduce kinds are real: slot 0 = state in w0, slot 1 = unit response in w1)
    auto fetch_state = [&](const ItemDesc &d) -> TaggedWords {
        TaggedWords wds;
        wds.w0 = 0;
        wds.w1 = 0;
        if (d.valid && leader && split && d.s_log > 0) {
            const unsigned char *rec = p.records + d.row0 * CARRY_RECORD_BYTES;
            if constexpr (REDUCE) {
                wds.w0 = ld_relaxed_u64(rec);
                wds.w1 = ld_relaxed_u64(rec + 16);
            } else {
                wds = fetch_tagged(rec, 0, sizeof(V) > 4);
            }
        }
        return wds;
    };
    TaggedWords head = fetch_state(cur);

    while (cur.valid && !failed) {
        // ---------------- item prologue (only the leader's first tile uses the incoming state)
        V item_x_in = vzero(V());
        V item_x2_in = vone(V());          // reduce kinds: unit response entering the item
        if (leader) {
            if (split && cur.s_log > 0) {
                const unsigned char *rec = p.records + cur.row0 * CARRY_RECORD_BYTES;
                const uint32_t want = epoch | static_cast<uint32_t>(cur.s_log);
                bool got;
                if constexpr (REDUCE) {
                    TaggedWords t0, t1;
                    t0.w0 = head.w0; t0.w1 = 0; t1.w0 = head.w1; t1.w1 = 0;
                    got = decode_tagged(t0, want, item_x_in);
                    got = decode_tagged(t1, want, item_x2_in) && got;
                } else {
                    got = decode_tagged(head, want, item_x_in);
                }
                for (uint32_t poll = 0; !got && poll < CARRY_WAIT_POLLS; ++poll) {
                    __nanosleep(64);
                    got = read_tagged(rec, 0, want, item_x_in);
                    if (REDUCE) got = read_tagged(rec, 1, want, item_x2_in) && got;
                }
                if (!got) {
                    status_bits |= STATUS_LOOKBACK_TIMEOUT;
                    item_x_in = vzero(V());
                    item_x2_in = vzero(V());
                }
            } else if (cin) {
                item_x_in = cin[cur.row0];
            }
        }
        // gate of the step after the row (backward): the caller's halo, or one
        const V row_end_gate = (BACK && hgate) ? hgate[cur.row0] : vone(V());
        V item_x_out = vzero(V()), item_x2_out = vzero(V());
        bool fetched_next = false;
        TaggedWords head_next = head;

        for (int i = g; i < cur.nt; i += G) {
            const int t = tile_of_step(cur, i);
            const int64_t toff = static_cast<int64_t>(t) * TE;
            const int nvalid = tile_valid(cur, t);
            const int64_t pos = cur.pos0 + toff;                 // position of the tile in its row
            const unsigned char *stg = stage_base + cs * STAGE_BYTES;
            V x_row_start = vzero(V());
            if (FULL_BWD && pos == 0 && hstate) x_row_start = hstate[cur.row0];
            if (i + G >= cur.nt) {
                // this warp's last tile of the item: look at the next item now
                need_next();
                head_next = fetch_state(nxt);
                fetched_next = true;
            }

            bool ok = mbar_wait_bounded(&bars[cs], parity, LOAD_WAIT_POLLS);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                failed = true;
                status_bits |= STATUS_LOAD_TIMEOUT;
                *abort_flag = 1;
                break;
            }

            // ---- shared -> registers
            V a[K], b[K];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                TR::unpack(*reinterpret_cast<const uint4 *>(stg + 0 * TB + (lane * NCH + c) * 16), &a[c * EPC]);
                TR::unpack(*reinterpret_cast<const uint4 *>(stg + 1 * TB + (lane * NCH + c) * 16), &b[c * EPC]);
            }
            V xp[FULL_BWD ? K : 1];
            V x_below = vzero(V()), gate_above = row_end_gate;
            if (BACK) {
                V hv[EPC];
                if (FULL_BWD) {
#pragma unroll
                    for (int c = 0; c < NCH; ++c)
                        TR::unpack(*reinterpret_cast<const uint4 *>(stg + 2 * TB + (lane * NCH + c) * 16), &xp[c * EPC]);
                    if (pos != 0) {
                        TR::unpack(*reinterpret_cast<const uint4 *>(stg + NIN * TB), hv);
                        x_below = hv[EPC - 1];
                    }
                }
                if (pos + nvalid < T) {
                    TR::unpack(*reinterpret_cast<const uint4 *>(stg + NIN * TB + 16), hv);
                    gate_above = hv[0];
                }
            }
            __syncwarp();
            --in_flight;
            if (++cs == NSTG) {
                cs = 0;
                parity ^= 1u;
            }
            if (lane == 0) fence_async_smem();
            produce();

            // ---- backward: gates shifted by one step inside registers
            if (BACK) {
                V up = shfl_down(a[0], 1);
                if (lane == 31) up = gate_above;
#pragma unroll
                for (int j = 0; j < K - 1; ++j) a[j] = vconj(a[j + 1]);
                a[K - 1] = vconj(up);
            }
            // ---- the ragged last tile of a row: identity beyond the row's end
            const int jv = nvalid - lane * K;
            if (nvalid < TE) {
                const V gate_end = vconj(row_end_gate);
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

            // ---- pass 1: lane aggregate (two half chains in packed fp32x2 for real types)
            constexpr bool PACKED = sizeof(V) == 4 && (K % 2 == 0);
            constexpr int H = K / 2;
            V A, B, A0h = vone(V()), B0h = vzero(V());
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
            // ---- Kogge-Stone inclusive combine across lanes, independent of the incoming state
            const int ll = REV ? 31 - lane : lane;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const V Ap = REV ? shfl_down(A, d) : shfl_up(A, d);
                const V Bp = REV ? shfl_down(B, d) : shfl_up(B, d);
                if (ll >= d) {
                    B = vfma(A, Bp, B);
                    A = vmul(A, Ap);
                }
            }
            V Ae = REV ? shfl_down(A, 1) : shfl_up(A, 1);
            V Be = REV ? shfl_down(B, 1) : shfl_up(B, 1);
            if (ll == 0) {
                Ae = vone(V());
                Be = vzero(V());
            }
            const V At = shfl_idx(A, REV ? 0 : 31), Bt = shfl_idx(B, REV ? 0 : 31);

            // ---- the incoming state: from the item (first tile) or from the warp before
            // A real value travels with its sequence number in one 64-bit shared-memory word
            // (a single store, a single load: nothing to order); a complex value is written
            // first, fenced, and then announced by the sequence number.
            V x_in = item_x_in;
            V x2_in = item_x2_in;
            if (i > 0) {
                const int from = (g + G - 1) % G;
                const uint32_t want = step_base + static_cast<uint32_t>(i);
                bool got = false;
                unsigned long long word = 0;
                for (uint32_t poll = 0; poll < MAIL_WAIT_POLLS; ++poll) {
                    if constexpr (sizeof(V) == 4) {
                        word = mail_word[from * 2];
                        got = static_cast<uint32_t>(word >> 32) == want;
                    } else {
                        got = mail_seq[from * 4] == want;
                    }
                    if (got) break;
                    if ((poll & 63u) == 63u) {
                        if (*abort_flag) break;
                        if (poll > 4096) __nanosleep(40);
                    }
                }
                got = __all_sync(0xffffffffu, got);
                if (!got) {
                    failed = true;
                    status_bits |= STATUS_LOOKBACK_TIMEOUT;
                    *abort_flag = 1;
                    break;
                }
                if constexpr (sizeof(V) == 4) {
                    x_in = __uint_as_float(static_cast<uint32_t>(word));
                    if constexpr (REDUCE) {
                        // the second word was stored before the first: it is there once the first is
                        x2_in = __uint_as_float(static_cast<uint32_t>(mail_word[from * 2 + 1]));
                    }
                } else {
                    x_in.x = mail_val[from * 4 + 2];
                    x_in.y = mail_val[from * 4 + 3];
                }
            }
            const V x_out = vfma(At, x_in, Bt);
            const V x2_out = REDUCE ? vmul(At, x2_in) : vzero(V());
            if (i + 1 < cur.nt) {
                // forward it at once: the next warp only waits for this hop
                if (lane == 0) {
                    const uint32_t seq = step_base + static_cast<uint32_t>(i) + 1u;
                    if constexpr (sizeof(V) == 4) {
                        if constexpr (REDUCE) {
                            mail_word[g * 2 + 1] = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(x2_out);
                            __threadfence_block();
                        }
                        mail_word[g * 2] = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(x_out);
                    } else {
                        mail_val[g * 4 + 2] = x_out.x;
                        mail_val[g * 4 + 3] = x_out.y;
                        __threadfence_block();
                        mail_seq[g * 4] = seq;
                    }
                }
            } else {
                item_x_out = x_out;
                item_x2_out = x2_out;
            }
            if constexpr (REDUCE) {
                ++step_count;
                continue;          // carries only: nothing to write for this tile
            }

            // ---- pass 2: the recurrence from the lane's incoming state
            V x = vfma(Ae, x_in, Be);
            if constexpr (PACKED) {
                auto J = [](int q) { return REV ? K - 1 - q : q; };
                float2 Xv = make_float2(x, fmaf(A0h, x, B0h));
#pragma unroll
                for (int q = 0; q < H; ++q) {
                    const float2 av = make_float2(a[J(q)], a[J(H + q)]);
                    const float2 bv = make_float2(b[J(q)], b[J(H + q)]);
                    Xv = __ffma2_rn(av, Xv, bv);
                    b[J(q)] = Xv.x;
                    b[J(H + q)] = Xv.y;
                }
            } else {
#pragma unroll
                for (int q = 0; q < K; ++q) {
                    const int j = REV ? K - 1 - q : q;
                    x = vfma(a[j], x, b[j]);
                    b[j] = x;
                }
            }
            if (FULL_BWD) {
                // d_gates[t] = conj(x[t-1]) * g[t]
                V dn = shfl_up(xp[K - 1], 1);
                if (lane == 0) dn = (pos != 0) ? x_below : x_row_start;
#pragma unroll
                for (int j = 1; j < K; ++j) a[j] = vmul(vconj(xp[j - 1]), b[j]);
                a[0] = vmul(vconj(dn), b[0]);
            }
            // ---- registers -> staging -> global
            unsigned char *ob = out_base + static_cast<int>(step_count & 1u) * NOUT * TB;
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                *reinterpret_cast<uint4 *>(ob + (lane * NCH + c) * 16) = TR::pack(&b[c * EPC]);
                if (NOUT > 1) *reinterpret_cast<uint4 *>(ob + TB + (lane * NCH + c) * 16) = TR::pack(&a[c * EPC]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                const uint32_t bytes = static_cast<uint32_t>(nvalid) * TR::ESIZE;
                const int64_t goff = (cur.e_begin + toff) * TR::ESIZE;
#pragma unroll
                for (int k = 0; k < NOUT; ++k) bulk_s2g(obase[k] + goff, ob + k * TB, bytes);
                bulk_commit();
            }
            ++step_count;
        }

        // ---------------- item epilogue
        if (!failed) {
            // the warp that owned the last tile holds the state leaving the segment
            if ((cur.nt - 1) % G == g && lane == 0) {
                if (split && cur.s_log + 1 < p.segs_per_row) {
                    unsigned char *rec = p.records + cur.row0 * CARRY_RECORD_BYTES;
                    const uint32_t tag = epoch | static_cast<uint32_t>(cur.s_log + 1);
                    publish_tagged(rec, 0, item_x_out, tag);
                    if (REDUCE) publish_tagged(rec, 1, item_x2_out, tag);
                } else if (REDUCE) {
                    // the item closes its row: the running state is the row's carry
                    V *cout = static_cast<V *>(p.carry_out);
                    cout[2 * cur.row0] = item_x2_out;
                    cout[2 * cur.row0 + 1] = item_x_out;
                }
            }
            if (!fetched_next) {
                need_next();
                head_next = fetch_state(nxt);
            }
        }
        team_barrier();
        if (*abort_flag) {
            failed = true;
            break;
        }
        step_base += static_cast<uint32_t>(cur.nt);
        ++n_item;
        head = head_next;
        cur = nxt;
        raw_next = cur.valid ? draw() : 0u;
        nxt_ready = false;
        if (prod_in_next) {
            prod_in_next = false;
        } else {
            p_i = g;
        }
        if (cur.valid) produce();
    }

    if (lane == 0) bulk_wait_read<0>();
    __syncwarp();
    leave_kernel(p, W, status_bits, lane);
}

}  // namespace ascan

// Row-stream scan kernel: every warp owns a contiguous group of whole rows and
// streams it tile by tile through its own shared-memory ring.
//
//   * The rows x T matrix is treated as one flat array.  A warp's share is a flat
//     range that starts and ends on row boundaries; tiles are fixed-size pieces of
//     that range and may straddle rows.  A row boundary inside a tile is handled by
//     forcing the gate of the row's first processed element to zero, which resets
//     the running state without any special tile shapes (so any T works).
//   * Bulk loader: one lane issues 1-D bulk asynchronous copies (global -> shared,
//     mbarrier completion, no multicast) STAGES tiles ahead; results leave through
//     bulk asynchronous stores from a double-buffered shared staging area.  Each lane
//     owns NCH consecutive 16-byte chunks of a tile; with NCH odd the 16-byte shared
//     accesses of a quarter-warp fall in distinct bank groups.
//   * Plain loader: the same arithmetic fed by element-wise loads/stores, for data
//     that is not 16-byte aligned.
//   * Per tile: sequential pass over the lane's elements for the lane aggregate
//     (A, B) of x -> A*x + B, Kogge-Stone combine across lanes by shuffles, then a
//     second sequential pass from the lane's incoming state.  The state crossing
//     tiles is one register per warp; no block-level barrier exists in the loop.
//
// Kinds: forward scan (optionally reversed), fused backward (reverse scan over the
// gates shifted by one step plus the d_gates epilogue; the shifted operands come
// from neighbouring lanes by shuffle, the tile halo from one scalar), and the two
// carry-only reductions used by time-sharded callers.
#pragma once

#include "common.cuh"

namespace ascan {

enum : int { K_SCAN = 0, K_BWD = 1, K_REDUCE = 2, K_REDUCE_BWD = 3 };

struct RowStreamParams {
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
    int64_t rows_per_item, items;
    uint32_t *status;        // device status word, or null
    int32_t stages;          // shared-memory stages per warp (bulk loader)
};

__host__ __device__ constexpr int rowstream_nin(int kind) { return kind == K_BWD ? 3 : 2; }
__host__ __device__ constexpr int rowstream_nout(int kind) { return kind == K_SCAN ? 1 : (kind == K_BWD ? 2 : 0); }
__host__ __device__ constexpr int rowstream_warp_smem(int nch, int stages, int kind, bool bulk) {
    const int tb = 32 * nch * 16;
    const int nstg = bulk ? stages : 1;
    const int outbufs = bulk ? 2 : 1;
    return nstg * rowstream_nin(kind) * tb + outbufs * rowstream_nout(kind) * tb + 128;
}

constexpr uint32_t LOAD_WAIT_POLLS = 1u << 22;

template <class TR, int NCH, int KIND, bool REVERSE, bool BULK>
__global__ void __launch_bounds__(384, 1) rowstream_kernel(const RowStreamParams p) {
    using V = typename TR::V;
    using Raw = typename TR::Raw;
    constexpr int EPC = TR::EPC;
    constexpr int K = NCH * EPC;          // elements per lane per tile
    constexpr int TE = 32 * K;            // elements per tile
    constexpr int TB = 32 * NCH * 16;     // bytes per tile per stream
    constexpr bool BACK = (KIND == K_BWD || KIND == K_REDUCE_BWD);
    constexpr bool REV = REVERSE || BACK;
    constexpr bool REDUCE = (KIND == K_REDUCE || KIND == K_REDUCE_BWD);
    constexpr int NIN = rowstream_nin(KIND);
    constexpr int NOUT = rowstream_nout(KIND);
    constexpr int OUTBUFS = BULK ? 2 : 1;
    const int NSTG = BULK ? p.stages : 1;
    const int WARP_SMEM = rowstream_warp_smem(NCH, p.stages, KIND, BULK);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    unsigned char *wsm = smem_raw + static_cast<size_t>(wib) * WARP_SMEM;
    unsigned char *stage_base = wsm;
    unsigned char *out_base = wsm + NSTG * NIN * TB;
    uint64_t *bars = reinterpret_cast<uint64_t *>(out_base + OUTBUFS * NOUT * TB);

    // contiguous share of the items for this warp
    const int64_t w = static_cast<int64_t>(blockIdx.x) * wpc + wib;
    const int64_t W = static_cast<int64_t>(gridDim.x) * wpc;
    const int64_t i0 = (p.items * w) / W, i1 = (p.items * (w + 1)) / W;
    int64_t r0 = i0 * p.rows_per_item, r1 = i1 * p.rows_per_item;
    if (r0 > p.rows) r0 = p.rows;
    if (r1 > p.rows) r1 = p.rows;
    if (r0 >= r1) return;
    const int64_t T = p.T;
    const int64_t e_begin = r0 * T;
    const int64_t n = (r1 - r0) * T;
    const int64_t nt = (n + TE - 1) / TE;

    const unsigned char *gin[3] = {static_cast<const unsigned char *>(p.in0) + e_begin * TR::ESIZE,
                                   static_cast<const unsigned char *>(p.in1) + e_begin * TR::ESIZE,
                                   NIN > 2 ? static_cast<const unsigned char *>(p.in2) + e_begin * TR::ESIZE : nullptr};
    unsigned char *gout[2] = {NOUT > 0 ? static_cast<unsigned char *>(p.out0) + e_begin * TR::ESIZE : nullptr,
                              NOUT > 1 ? static_cast<unsigned char *>(p.out1) + e_begin * TR::ESIZE : nullptr};
    const V *cin = static_cast<const V *>(p.carry_in);
    const V *hgate = static_cast<const V *>(p.halo_gate);
    const V *hstate = static_cast<const V *>(p.halo_state);

    auto tile_of_step = [&](int64_t i) -> int64_t { return REV ? nt - 1 - i : i; };
    auto tile_valid = [&](int64_t t) -> int {
        const int64_t left = n - t * TE;
        return left < TE ? static_cast<int>(left) : TE;
    };

    // bulk loader: lane 0 arms the stage's mbarrier and issues one copy per stream
    auto issue = [&](int64_t t, int s) {
        const uint32_t bytes = static_cast<uint32_t>(tile_valid(t)) * TR::ESIZE;
        mbar_expect_tx(&bars[s], bytes * NIN);
#pragma unroll
        for (int k = 0; k < NIN; ++k)
            bulk_g2s(stage_base + (s * NIN + k) * TB, gin[k] + t * TB, bytes, &bars[s]);
    };

    if (BULK) {
        if (lane == 0) {
            for (int s = 0; s < NSTG; ++s) mbar_init(&bars[s], 1);
            mbar_init_fence();
        }
        __syncwarp();
        if (lane == 0) {
            for (int s = 0; s < NSTG; ++s)
                if (s < nt) issue(tile_of_step(s), s);
        }
    }

    // running position of the tile start: ts_mod = (tile start) mod T, row_ts = its row
    int64_t ts_mod, row_ts;
    {
        const int64_t off = tile_of_step(0) * TE;
        ts_mod = off % T;
        row_ts = r0 + off / T;
    }

    V x_carry = vzero(V());    // state entering the tile
    V x2_carry = vzero(V());   // reduce kinds: response to a unit incoming state
    V next_gate = vone(V());   // backward kinds: gate of the first element of the tile above
    bool failed = false;
    int s = 0;                 // ring stage of the current tile
    uint32_t parity = 0;       // mbarrier phase parity of that stage

    for (int64_t i = 0; i < nt; ++i) {
        const int64_t t = tile_of_step(i);
        const int64_t toff = t * TE;
        const int nvalid = tile_valid(t);
        const unsigned char *stg = stage_base + s * NIN * TB;

        // backward: the state just below the tile, needed by lane 0 for d_gates
        V x_halo = vzero(V());
        if (KIND == K_BWD) {
            if (ts_mod != 0) x_halo = TR::load_one(p.in2, e_begin + toff - 1);
        }

        if (BULK) {
            bool ok = mbar_wait_bounded(&bars[s], parity, LOAD_WAIT_POLLS);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                failed = true;
                break;
            }
        } else {
            // plain loader: element-wise copy of the valid part of the tile
            __syncwarp();
#pragma unroll
            for (int k = 0; k < NIN; ++k) {
                const Raw *src = reinterpret_cast<const Raw *>(gin[k]) + toff;
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
            const uint4 qb = *reinterpret_cast<const uint4 *>(stg + 1 * TB + (lane * NCH + c) * 16);
            TR::unpack(qa, &a[c * EPC]);
            TR::unpack(qb, &b[c * EPC]);
        }
        V xp[KIND == K_BWD ? K : 1];
        if (KIND == K_BWD) {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const uint4 qx = *reinterpret_cast<const uint4 *>(stg + 2 * TB + (lane * NCH + c) * 16);
                TR::unpack(qx, &xp[c * EPC]);
            }
        }
        if (BULK) {
            __syncwarp();
            if (lane == 0 && i + NSTG < nt) {
                fence_async_smem();
                issue(tile_of_step(i + NSTG), s);
            }
        }

        // ---- backward kinds: shift the operands by one step inside registers
        if (BACK) {
            const V g0 = a[0];
            V up = shfl_down(g0, 1);
            if (lane == 31) up = next_gate;
#pragma unroll
            for (int j = 0; j < K - 1; ++j) a[j] = vconj(a[j + 1]);
            a[K - 1] = vconj(up);
            next_gate = shfl_idx(g0, 0);
        }
        if (KIND == K_BWD) {
            V dn = shfl_up(xp[K - 1], 1);
            if (lane == 0) dn = x_halo;
#pragma unroll
            for (int j = K - 1; j > 0; --j) xp[j] = xp[j - 1];
            xp[0] = dn;
        }

        // ---- row boundaries and the ragged last tile
        V b2[REDUCE ? K : 1];
        if (REDUCE) {
#pragma unroll
            for (int j = 0; j < K; ++j) b2[j] = vzero(V());
        }
        const bool has_boundary = (ts_mod == 0) || (ts_mod + nvalid >= T);
        const bool slow = has_boundary || (nvalid < TE);
        if (slow) {
#pragma unroll
            for (int j = 0; j < K; ++j) {
                const int o = lane * K + j;
                const int64_t pos = ts_mod + o;
                int64_t q, rem;
                if (T > TE) {
                    q = pos >= T ? 1 : 0;
                    rem = pos - (q ? T : 0);
                } else {
                    const int pi = static_cast<int>(pos), ti = static_cast<int>(T);
                    q = pi / ti;
                    rem = pi - static_cast<int>(q) * ti;
                }
                const bool is_start = (rem == 0);
                const bool is_end = (rem == T - 1);
                const bool first = REV ? is_end : is_start;
                const int64_t row = row_ts + q;
                if (o >= nvalid) {
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
                    if (KIND == K_BWD) {
                        if (is_start) xp[j] = hstate ? hstate[row] : vzero(V());
                    }
                }
            }
        }

        // ---- pass 1: lane aggregate in processing order
        constexpr int JF = REV ? K - 1 : 0;
        V A = a[JF], B = b[JF];
        V B2 = REDUCE ? b2[JF] : vzero(V());
#pragma unroll
        for (int q = 1; q < K; ++q) {
            const int j = REV ? K - 1 - q : q;
            B = vfma(a[j], B, b[j]);
            if (REDUCE) B2 = vfma(a[j], B2, b2[j]);
            A = vmul(A, a[j]);
        }
        // the warp's incoming state enters through the first lane in processing order
        const int ll = REV ? 31 - lane : lane;
        if (ll == 0) {
            B = vfma(A, x_carry, B);
            if (REDUCE) B2 = vfma(A, x2_carry, B2);
        }
        // ---- Kogge-Stone inclusive combine across lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const V Ap = REV ? shfl_down(A, d) : shfl_up(A, d);
            const V Bp = REV ? shfl_down(B, d) : shfl_up(B, d);
            V B2p = vzero(V());
            if (REDUCE) B2p = REV ? shfl_down(B2, d) : shfl_up(B2, d);
            if (ll >= d) {
                B = vfma(A, Bp, B);
                if (REDUCE) B2 = vfma(A, B2p, B2);
                if (d < 16) A = vmul(A, Ap);
            }
        }
        // state entering this lane = inclusive result of the previous lane
        V x = REV ? shfl_down(B, 1) : shfl_up(B, 1);
        if (ll == 0) x = x_carry;
        V x2 = vzero(V());
        if (REDUCE) {
            x2 = REV ? shfl_down(B2, 1) : shfl_up(B2, 1);
            if (ll == 0) x2 = x2_carry;
        }
        x_carry = shfl_idx(B, REV ? 0 : 31);
        if (REDUCE) x2_carry = shfl_idx(B2, REV ? 0 : 31);

        if (!REDUCE) {
            // ---- pass 2: the recurrence itself from the lane's incoming state
#pragma unroll
            for (int q = 0; q < K; ++q) {
                const int j = REV ? K - 1 - q : q;
                x = vfma(a[j], x, b[j]);
                b[j] = x;
                if (KIND == K_BWD) a[j] = vmul(vconj(xp[j]), x);
            }
            // ---- registers -> staging -> global
            if (BULK) {
                unsigned char *ob = out_base + static_cast<int>(i & 1) * NOUT * TB;
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
#pragma unroll
                    for (int k = 0; k < NOUT; ++k) bulk_s2g(gout[k] + t * TB, ob + k * TB, bytes);
                    bulk_commit();
                }
            } else {
                unsigned char *ob = out_base;
                __syncwarp();
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    *reinterpret_cast<uint4 *>(ob + (lane * NCH + c) * 16) = TR::pack(&b[c * EPC]);
                    if (NOUT > 1) *reinterpret_cast<uint4 *>(ob + TB + (lane * NCH + c) * 16) = TR::pack(&a[c * EPC]);
                }
                __syncwarp();
#pragma unroll
                for (int k = 0; k < NOUT; ++k) {
                    const Raw *src = reinterpret_cast<const Raw *>(ob + k * TB);
                    Raw *dst = reinterpret_cast<Raw *>(gout[k]) + toff;
                    for (int idx = lane; idx < nvalid; idx += 32) dst[idx] = src[idx];
                }
            }
        } else if (has_boundary) {
            // reduce kinds: only tiles that finish a row need the element states
            V *cout = static_cast<V *>(p.carry_out);
#pragma unroll
            for (int q = 0; q < K; ++q) {
                const int j = REV ? K - 1 - q : q;
                x = vfma(a[j], x, b[j]);
                x2 = vfma(a[j], x2, b2[j]);
                const int o = lane * K + j;
                const int64_t pos = ts_mod + o;
                int64_t qq, rem;
                if (T > TE) {
                    qq = pos >= T ? 1 : 0;
                    rem = pos - (qq ? T : 0);
                } else {
                    const int pi = static_cast<int>(pos), ti = static_cast<int>(T);
                    qq = pi / ti;
                    rem = pi - static_cast<int>(qq) * ti;
                }
                const bool last = REV ? (rem == 0) : (rem == T - 1);
                if (last && o < nvalid) {
                    const int64_t row = row_ts + qq;
                    cout[2 * row] = x2;
                    cout[2 * row + 1] = x;
                }
            }
        }

        // ---- advance the ring and the running tile position
        if (BULK) {
            if (++s == NSTG) {
                s = 0;
                parity ^= 1u;
            }
        }
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

    if (BULK) {
        if (lane == 0) bulk_wait_read<0>();
        if (failed && lane == 0 && p.status) atomicOr(p.status, STATUS_LOAD_TIMEOUT);
        __syncwarp();
    }
}

}  // namespace ascan

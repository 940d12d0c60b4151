// extern "C" entry points of the library (declared in include/ascan_b200.h):
// argument validation, planning, kernel dispatch, launch-error reporting.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "../../include/ascan_b200.h"
#include "launch.h"
#include "planner.h"
#include "lookback.cuh"
#include "stream.cuh"

namespace ascan {

static int cached_sm_count(int *out) {
    static std::atomic<int> counts[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (dev >= 0 && dev < 64) {
        const int c = counts[dev].load(std::memory_order_relaxed);
        if (c > 0) {
            *out = c;
            return ASCAN_OK;
        }
    }
    int n = 0, major = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (major != 10 || n < 1) return ASCAN_ERR_DEVICE;   // built for sm_100a only
    if (dev >= 0 && dev < 64) counts[dev].store(n, std::memory_order_relaxed);
    *out = n;
    return ASCAN_OK;
}

// ---- options (ascan_set_option): process-wide, read on every call, never from the environment
static std::atomic<int> g_opt_stages{2}, g_opt_wpc{0}, g_opt_lookback_tiles{0}, g_opt_disable_plans{0};
static std::atomic<int> g_opt_drop_carry{0}, g_opt_epoch_bits{17}, g_opt_items_per_warp{4}, g_opt_static_below{8};
static std::atomic<uint32_t> g_opt_generation{0};

static PlanTuning current_tuning() {
    PlanTuning t;
    t.stages = g_opt_stages.load(std::memory_order_relaxed);
    t.warps_per_cta = g_opt_wpc.load(std::memory_order_relaxed);
    t.lookback_tiles = g_opt_lookback_tiles.load(std::memory_order_relaxed);
    t.disable_plans = g_opt_disable_plans.load(std::memory_order_relaxed);
    t.items_per_warp = g_opt_items_per_warp.load(std::memory_order_relaxed);
    t.static_below = g_opt_static_below.load(std::memory_order_relaxed);
    return t;
}

// ---- plan memo: the last few plans of this thread.  make_plan is pure arithmetic on its
// input, so an equal key means an equal plan; options changes bump the generation.
struct PlanKey {
    int64_t rows, seqlen;
    int dtype, kind, sm_count;
    uint32_t flags, generation;
    bool operator==(const PlanKey &o) const {
        return rows == o.rows && seqlen == o.seqlen && dtype == o.dtype && kind == o.kind && sm_count == o.sm_count &&
               flags == o.flags && generation == o.generation;
    }
};
struct PlanMemo {
    static constexpr int N = 8;
    PlanKey key[N];
    ascan_plan plan[N];
    int rc[N];
    int used = 0, next = 0;
};
static int make_plan_cached(const PlanInput &in, ascan_plan *pl) {
    thread_local PlanMemo memo;
    PlanKey k;
    k.rows = in.rows;
    k.seqlen = in.seqlen;
    k.dtype = in.dtype;
    k.kind = in.kind;
    k.sm_count = in.sm_count;
    k.flags = (in.reverse ? 1u : 0u) | (in.aligned ? 2u : 0u) | (in.workspace ? 4u : 0u) | (in.allow_lookback ? 8u : 0u) |
              (in.allow_team ? 16u : 0u) | (in.three_chunks ? 32u : 0u) | (in.force_lookback ? 64u : 0u) |
              (in.allow_grid ? 128u : 0u);
    k.generation = g_opt_generation.load(std::memory_order_relaxed);
    for (int i = 0; i < memo.used; ++i) {
        if (memo.key[i] == k) {
            *pl = memo.plan[i];
            return memo.rc[i];
        }
    }
    const int rc = make_plan(in, pl);
    const int slot = memo.next;
    memo.key[slot] = k;
    memo.plan[slot] = *pl;
    memo.rc[slot] = rc;
    memo.next = (slot + 1) % PlanMemo::N;
    if (memo.used < PlanMemo::N) ++memo.used;
    return rc;
}

static int launch_by_dtype(int dtype, int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl,
                           cudaStream_t st, const ShardParams *sp = nullptr) {
    switch (dtype) {
        case ASCAN_F32: return launch_f32(variant, kind, reverse, p, pl, st, sp);
        case ASCAN_BF16: return launch_bf16(variant, kind, reverse, p, pl, st, sp);
        case ASCAN_F16: return launch_f16(variant, kind, reverse, p, pl, st, sp);
        case ASCAN_C64: return launch_c64(variant, kind, reverse, p, pl, st, sp);
        default: return ASCAN_ERR_INVALID_ARG;
    }
}

// Folds the carries gathered from all ranks of a time-sharded scan into this rank's
// incoming state: prefix = composition of ranks 0..rank-1 (forward), suffix = composition of
// ranks world-1..rank+1 (backward).  gathered[j][r][0..stride): {P, S, (first gate)} of rank j.
template <class V>
__global__ void fold_carries_kernel(const V *gathered, int64_t rows, int world, int rank, int stride, int suffix,
                                    V *state_out, V *halo_out) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    V x = vzero(V());
    if (!suffix) {
        for (int j = 0; j < rank; ++j) {
            const V *c = gathered + (static_cast<int64_t>(j) * rows + r) * stride;
            x = vfma(c[0], x, c[1]);
        }
    } else {
        for (int j = world - 1; j > rank; --j) {
            const V *c = gathered + (static_cast<int64_t>(j) * rows + r) * stride;
            x = vfma(c[0], x, c[1]);
        }
    }
    state_out[r] = x;
    if (halo_out) {
        // gate of the first step of the next rank, or one after the last rank
        halo_out[r] = (rank + 1 < world && stride > 2)
                          ? gathered[(static_cast<int64_t>(rank + 1) * rows + r) * stride + 2]
                          : vone(V());
    }
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int plan_for(int64_t rows, int64_t seqlen, int dtype, int kind, bool aligned, const void *ws, size_t ws_bytes,
                    ascan_plan *pl, bool reverse = false, bool seeded = false) {
    PlanInput in;
    in.reverse = reverse;
    in.allow_grid = !seeded;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = aligned;
    in.workspace = ws && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0;
    in.tune = current_tuning();
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    // prefer the plan that wants the most scratch; step down while the caller's is too small
    rc = make_plan_cached(in, pl);
    if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes && in.workspace) {
        in.allow_lookback = false;
        rc = make_plan_cached(in, pl);
        if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes) {
            in.workspace = false;
            rc = make_plan_cached(in, pl);
        }
    }
    return rc;
}

// Copies the plan's decomposition and the workspace pointers into the kernel parameters.
static void fill_common(StreamParams &p, const ascan_plan &pl, int64_t rows, int64_t seqlen, void *ws, size_t ws_bytes) {
    p.rows = rows;
    p.T = seqlen;
    p.rows_per_item = pl.rows_per_item;
    p.row_groups = pl.row_groups;
    p.seg_elems = pl.seg_elems;
    p.fine_elems = pl.fine_elems;
    p.coarse_segs = pl.coarse_segs;
    p.fine_segs = pl.fine_segs;
    p.segs_per_row = pl.segs_per_row;
    p.items = pl.items;
    p.ctrl = pl.dynamic ? static_cast<uint32_t *>(ws) : nullptr;
    p.records = pl.dynamic ? static_cast<unsigned char *>(ws) + CTRL_BYTES : nullptr;
    p.stages = pl.stages;
    p.team_size = pl.team_size;
    p.test_drop_carry = g_opt_drop_carry.load(std::memory_order_relaxed);
    p.epoch_mask = (1u << g_opt_epoch_bits.load(std::memory_order_relaxed)) - 1u;
    p.scratch_bytes = (pl.dynamic && ws_bytes > static_cast<size_t>(CTRL_BYTES)) ? ws_bytes - CTRL_BYTES : 0;
}

// Plan for the fused variants, which exist only in the chained stream plan with the bulk
// loader and one row or segment per item.
static int plan_for_variant(int64_t rows, int64_t seqlen, int dtype, int kind, bool reverse, void *ws, size_t ws_bytes,
                            ascan_plan *pl) {
    PlanInput in;
    in.three_chunks = true;    // (the sigmoid backward measured 7 % faster with 3 chunks than with 2)
    in.reverse = reverse;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = true;
    in.workspace = ws && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0;
    in.allow_lookback = false;
    in.allow_team = false;
    in.tune = current_tuning();
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    rc = make_plan_cached(in, pl);
    if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes && in.workspace) {
        in.workspace = false;
        rc = make_plan_cached(in, pl);
    }
    if (rc != ASCAN_OK) return rc;
    if (pl->loader != 0 || pl->rows_per_item != 1 || pl->kernel != 0) return ASCAN_ERR_UNSUPPORTED;
    return ASCAN_OK;
}

}  // namespace ascan

using namespace ascan;

extern "C" {

int ascan_version(void) { return 100; }   // 0.1.0

const char *ascan_strerror(int status) {
    switch (status) {
        case ASCAN_OK: return "success";
        case ASCAN_ERR_INVALID_ARG: return "invalid argument";
        case ASCAN_ERR_UNSUPPORTED: return "unsupported combination";
        case ASCAN_ERR_LAUNCH: return "CUDA launch failed";
        case ASCAN_ERR_TIMEOUT: return "a bounded device-side wait expired";
        case ASCAN_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case ASCAN_ERR_DEVICE: return "no usable sm_100 device";
        case ASCAN_ERR_TOO_LARGE:
            return "more rows than the built-in scratch of ascan_forward_no_alloc holds (16384)";
        default: return "unknown status";
    }
}

int ascan_forward(const void *gates, const void *tokens, void *out, int64_t rows, int64_t seqlen, int dtype,
                  int reverse, const void *carry_in, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !tokens || !out) return ASCAN_ERR_INVALID_ARG;
    ascan_plan pl;
    const bool al = aligned16(gates) && aligned16(tokens) && aligned16(out);
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_FORWARD, al, ws, ws_bytes, &pl, reverse != 0, carry_in != nullptr);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens;
    p.out0 = out;
    p.carry_in = carry_in;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_FORWARD, reverse != 0, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_backward(const void *gates, const void *states, const void *grad_out, void *d_gates, void *d_tokens,
                   int64_t rows, int64_t seqlen, int dtype, const void *carry_in, const void *halo_gate_right,
                   const void *halo_state_left, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !states || !grad_out || !d_gates || !d_tokens) return ASCAN_ERR_INVALID_ARG;
    if (carry_in && !halo_gate_right) return ASCAN_ERR_INVALID_ARG;
    ascan_plan pl;
    const bool al = aligned16(gates) && aligned16(states) && aligned16(grad_out) && aligned16(d_gates) &&
                    aligned16(d_tokens);
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_BACKWARD, al, ws, ws_bytes, &pl, false,
                      carry_in || halo_gate_right || halo_state_left);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = grad_out;
    p.in2 = states;
    p.out0 = d_tokens;
    p.out1 = d_gates;
    p.carry_in = carry_in;
    p.halo_gate = halo_gate_right;
    p.halo_state = halo_state_left;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_BACKWARD, true, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_reduce_forward(const void *gates, const void *tokens, void *carry_out, int64_t rows, int64_t seqlen,
                         int dtype, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !tokens || !carry_out) return ASCAN_ERR_INVALID_ARG;
    ascan_plan pl;
    const bool al = aligned16(gates) && aligned16(tokens);
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_REDUCE_FORWARD, al, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens;
    p.carry_out = carry_out;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_REDUCE_FORWARD, false, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_reduce_backward(const void *gates, const void *grad_out, const void *halo_gate_right, void *carry_out,
                          int64_t rows, int64_t seqlen, int dtype, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !grad_out || !carry_out) return ASCAN_ERR_INVALID_ARG;
    ascan_plan pl;
    const bool al = aligned16(gates) && aligned16(grad_out);
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_REDUCE_BACKWARD, al, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = grad_out;
    p.halo_gate = halo_gate_right;
    p.carry_out = carry_out;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_REDUCE_BACKWARD, true, p, pl, static_cast<cudaStream_t>(stream));
}

size_t ascan_workspace_bytes(int64_t rows, int64_t seqlen, int dtype, int kind) {
    PlanInput in;
    in.rows = rows;
    in.seqlen = seqlen < 1 ? 1 : seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = true;
    in.workspace = true;
    in.reverse = false;
    in.tune = current_tuning();
    if (cached_sm_count(&in.sm_count) != ASCAN_OK) {
        cudaGetLastError();
        in.sm_count = 148;          // no device to ask: size for a full B200
    }
    ascan_plan pl;
    if (make_plan_cached(in, &pl) != ASCAN_OK) return static_cast<size_t>(workspace_bytes(rows));
    return static_cast<size_t>(pl.workspace_bytes);
}

int ascan_plan_describe(int64_t rows, int64_t seqlen, int dtype, int kind, int flags, int sm_count,
                        ascan_plan *plan) {
    PlanInput in;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = (flags & 1) != 0;
    in.workspace = (flags & 2) != 0;
    in.reverse = (flags & 4) != 0;
    in.sm_count = sm_count;
    in.allow_lookback = (flags & 8) == 0;
    in.allow_team = (flags & 16) == 0;
    in.allow_grid = (flags & 32) == 0;
    if (sm_count <= 0) {
        int rc = cached_sm_count(&in.sm_count);
        if (rc != ASCAN_OK) return rc;
    }
    in.tune = current_tuning();
    return make_plan(in, plan);
}

int ascan_set_option(int option, int value) {
    switch (option) {
        case ASCAN_OPT_STAGES:
            if (value < 1 || value > 8) return ASCAN_ERR_INVALID_ARG;
            g_opt_stages.store(value);
            break;
        case ASCAN_OPT_WARPS_PER_CTA:
            if (value < 0 || value > 16) return ASCAN_ERR_INVALID_ARG;
            g_opt_wpc.store(value);
            break;
        case ASCAN_OPT_LOOKBACK_TILES:
            if (value < 0 || value > 8) return ASCAN_ERR_INVALID_ARG;
            g_opt_lookback_tiles.store(value);
            break;
        case ASCAN_OPT_DISABLE_PLANS:
            if (value < 0 || value > 63) return ASCAN_ERR_INVALID_ARG;
            g_opt_disable_plans.store(value);
            break;
        case ASCAN_OPT_ITEMS_PER_WARP:
            if (value < 1 || value > 64) return ASCAN_ERR_INVALID_ARG;
            g_opt_items_per_warp.store(value);
            break;
        case ASCAN_OPT_STATIC_BELOW:
            if (value < 0 || value > 1024) return ASCAN_ERR_INVALID_ARG;
            g_opt_static_below.store(value);
            break;
        case ASCAN_OPT_TEST_DROP_CARRY: g_opt_drop_carry.store(value ? 1 : 0); break;
        case ASCAN_OPT_TEST_EPOCH_BITS:
            if (value < 1 || value > 17) return ASCAN_ERR_INVALID_ARG;
            g_opt_epoch_bits.store(value);
            break;
        default: return ASCAN_ERR_INVALID_ARG;
    }
    g_opt_generation.fetch_add(1);
    return ASCAN_OK;
}

int ascan_get_option(int option) {
    switch (option) {
        case ASCAN_OPT_STAGES: return g_opt_stages.load();
        case ASCAN_OPT_WARPS_PER_CTA: return g_opt_wpc.load();
        case ASCAN_OPT_LOOKBACK_TILES: return g_opt_lookback_tiles.load();
        case ASCAN_OPT_DISABLE_PLANS: return g_opt_disable_plans.load();
        case ASCAN_OPT_ITEMS_PER_WARP: return g_opt_items_per_warp.load();
        case ASCAN_OPT_STATIC_BELOW: return g_opt_static_below.load();
        case ASCAN_OPT_TEST_DROP_CARRY: return g_opt_drop_carry.load();
        case ASCAN_OPT_TEST_EPOCH_BITS: return g_opt_epoch_bits.load();
        default: return -1;
    }
}

int ascan_forward_complex_real_tokens(const void *gates, const void *tokens_real, void *out, int64_t rows,
                                       int64_t seqlen, int reverse, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !tokens_real || !out) return ASCAN_ERR_INVALID_ARG;
    // The fused form exists for the bulk loader with one row (or one segment) per item in the
    // chained stream plan; the real rows must start 16-byte aligned as well (seqlen % 4 == 0).
    const bool al = aligned16(gates) && aligned16(tokens_real) && aligned16(out);
    if (!al || seqlen % 4 != 0) return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    int rc = plan_for_variant(rows, seqlen, ASCAN_C64, ASCAN_KIND_FORWARD, reverse != 0, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens_real;
    p.out0 = out;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_c64(VARIANT_REAL_TOKENS, ASCAN_KIND_FORWARD, reverse != 0, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_backward_complex_real_tokens(const void *gates, const void *states, const void *grad_out, void *d_gates,
                                       void *d_tokens_real, int64_t rows, int64_t seqlen, void *ws, size_t ws_bytes,
                                       void *stream) {
    if (rows < 0 || seqlen < 1) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !states || !grad_out || !d_gates || !d_tokens_real) return ASCAN_ERR_INVALID_ARG;
    const bool al = aligned16(gates) && aligned16(states) && aligned16(grad_out) && aligned16(d_gates) &&
                    aligned16(d_tokens_real);
    if (!al || seqlen % 4 != 0) return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    int rc = plan_for_variant(rows, seqlen, ASCAN_C64, ASCAN_KIND_BACKWARD, false, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    if (pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = grad_out;
    p.in2 = states;
    p.out0 = d_tokens_real;
    p.out1 = d_gates;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_c64(VARIANT_REAL_TOKENS, ASCAN_KIND_BACKWARD, true, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_forward_sigmoid_gates(const void *gate_logits, const void *tokens, void *out, int64_t rows, int64_t seqlen,
                                int dtype, void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (dtype == ASCAN_C64) return ASCAN_ERR_UNSUPPORTED;
    if (rows == 0) return ASCAN_OK;
    if (!gate_logits || !tokens || !out) return ASCAN_ERR_INVALID_ARG;
    if (!(aligned16(gate_logits) && aligned16(tokens) && aligned16(out))) return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    int rc = plan_for_variant(rows, seqlen, dtype, ASCAN_KIND_FORWARD, false, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gate_logits;
    p.in1 = tokens;
    p.out0 = out;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_SIGMOID, ASCAN_KIND_FORWARD, false, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_backward_sigmoid_gates(const void *gate_logits, const void *states, const void *grad_out, void *d_logits,
                                 void *d_tokens, int64_t rows, int64_t seqlen, int dtype, void *ws, size_t ws_bytes,
                                 void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (dtype == ASCAN_C64) return ASCAN_ERR_UNSUPPORTED;
    if (rows == 0) return ASCAN_OK;
    if (!gate_logits || !states || !grad_out || !d_logits || !d_tokens) return ASCAN_ERR_INVALID_ARG;
    if (!(aligned16(gate_logits) && aligned16(states) && aligned16(grad_out) && aligned16(d_logits) &&
          aligned16(d_tokens)))
        return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    int rc = plan_for_variant(rows, seqlen, dtype, ASCAN_KIND_BACKWARD, false, ws, ws_bytes, &pl);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gate_logits;
    p.in1 = grad_out;
    p.in2 = states;
    p.out0 = d_tokens;
    p.out1 = d_logits;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_SIGMOID, ASCAN_KIND_BACKWARD, true, p, pl, static_cast<cudaStream_t>(stream));
}

int ascan_fold_carries(const void *gathered, int64_t rows, int world, int rank, int stride, int dtype, int suffix,
                       void *state_out, void *halo_out, void *stream) {
    if (rows < 0 || world < 1 || rank < 0 || rank >= world || stride < 2 || dtype_size(dtype) == 0)
        return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gathered || !state_out) return ASCAN_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((rows + threads - 1) / threads);
    if (dtype == ASCAN_C64) {
        fold_carries_kernel<float2><<<blocks, threads, 0, st>>>(static_cast<const float2 *>(gathered), rows, world, rank,
                                                               stride, suffix, static_cast<float2 *>(state_out),
                                                               static_cast<float2 *>(halo_out));
    } else {
        fold_carries_kernel<float><<<blocks, threads, 0, st>>>(static_cast<const float *>(gathered), rows, world, rank,
                                                              stride, suffix, static_cast<float *>(state_out),
                                                              static_cast<float *>(halo_out));
    }
    return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
}

size_t ascan_exchange_bytes(int64_t rows, int world) {
    if (rows < 0 || world < 1 || world > MAX_WORLD) return 0;
    return static_cast<size_t>(xchg_bytes(rows, world));
}

size_t ascan_workspace_bytes_time_sharded(int64_t rows, int64_t seqlen, int dtype, int kind) {
    PlanInput in;
    in.rows = rows;
    in.seqlen = seqlen < 1 ? 1 : seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = true;
    in.workspace = true;
    in.reverse = false;
    in.force_lookback = true;
    in.tune = current_tuning();
    if (cached_sm_count(&in.sm_count) != ASCAN_OK) {
        cudaGetLastError();
        in.sm_count = 148;
    }
    ascan_plan pl;
    if (make_plan_cached(in, &pl) != ASCAN_OK) return 0;
    return static_cast<size_t>(pl.workspace_bytes);
}

// Plan and shard parameters shared by the two time-sharded entry points.
static int plan_time_sharded(int64_t rows, int64_t seqlen, int dtype, int kind, int rank, int world, uint32_t call,
                             void *const *exchange, void *ws, size_t ws_bytes, ascan_plan *pl, ShardParams *sp) {
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world || call == 0) return ASCAN_ERR_INVALID_ARG;
    if (world > 1 && !exchange) return ASCAN_ERR_INVALID_ARG;
    if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return ASCAN_ERR_WORKSPACE;
    PlanInput in;
    in.reverse = false;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = true;
    in.workspace = true;
    in.force_lookback = true;
    in.tune = current_tuning();
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    rc = make_plan_cached(in, pl);
    if (rc != ASCAN_OK) return rc;
    if (pl->workspace_bytes > ws_bytes) return ASCAN_ERR_WORKSPACE;
    *sp = ShardParams{};
    sp->rank = rank;
    sp->world = world;
    sp->call = call;
    for (int j = 0; j < world && world > 1; ++j) {
        if (!exchange[j] || (reinterpret_cast<uintptr_t>(exchange[j]) & 15u) != 0) return ASCAN_ERR_INVALID_ARG;
        sp->xchg[j] = static_cast<unsigned char *>(exchange[j]);
    }
    return ASCAN_OK;
}

int ascan_forward_time_sharded(const void *gates, const void *tokens, void *out, int64_t rows, int64_t seqlen,
                               int dtype, int rank, int world, uint32_t call, void *const *exchange, void *carry_save,
                               void *ws, size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !tokens || !out) return ASCAN_ERR_INVALID_ARG;
    if (!(aligned16(gates) && aligned16(tokens) && aligned16(out))) return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    ShardParams sp;
    int rc = plan_time_sharded(rows, seqlen, dtype, ASCAN_KIND_FORWARD, rank, world, call, exchange, ws, ws_bytes, &pl, &sp);
    if (rc != ASCAN_OK) return rc;
    sp.carry_save = carry_save;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens;
    p.out0 = out;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_FORWARD, false, p, pl, static_cast<cudaStream_t>(stream), &sp);
}

int ascan_backward_time_sharded(const void *gates, const void *states, const void *grad_out, void *d_gates,
                                void *d_tokens, int64_t rows, int64_t seqlen, int dtype, int rank, int world,
                                uint32_t call, void *const *exchange, const void *halo_state_left, void *ws,
                                size_t ws_bytes, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !states || !grad_out || !d_gates || !d_tokens) return ASCAN_ERR_INVALID_ARG;
    if (!(aligned16(gates) && aligned16(states) && aligned16(grad_out) && aligned16(d_gates) && aligned16(d_tokens)))
        return ASCAN_ERR_UNSUPPORTED;
    ascan_plan pl;
    ShardParams sp;
    int rc = plan_time_sharded(rows, seqlen, dtype, ASCAN_KIND_BACKWARD, rank, world, call, exchange, ws, ws_bytes, &pl, &sp);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = grad_out;
    p.in2 = states;
    p.out0 = d_tokens;
    p.out1 = d_gates;
    p.halo_state = halo_state_left;
    fill_common(p, pl, rows, seqlen, ws, ws_bytes);
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_BACKWARD, true, p, pl, static_cast<cudaStream_t>(stream), &sp);
}

// ---- peer-visible buffers for the exchange of time-sharded scans (the only functions of
// the library that allocate; nothing else calls them)
int ascan_peer_alloc(size_t bytes, void **ptr, void *handle64) {
    if (!ptr || !handle64 || bytes == 0) return ASCAN_ERR_INVALID_ARG;
    void *d = nullptr;
    if (cudaMalloc(&d, bytes) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_DEVICE;
    }
    cudaIpcMemHandle_t h;
    if (cudaMemset(d, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, d) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(d);
        return ASCAN_ERR_DEVICE;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    memcpy(handle64, &h, 64);
    *ptr = d;
    return ASCAN_OK;
}

int ascan_peer_open(const void *handle64, void **ptr) {
    if (!handle64 || !ptr) return ASCAN_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *d = nullptr;
    if (cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_DEVICE;
    }
    *ptr = d;
    return ASCAN_OK;
}

int ascan_peer_close(void *ptr) {
    if (!ptr) return ASCAN_ERR_INVALID_ARG;
    if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_DEVICE;
    }
    return ASCAN_OK;
}

int ascan_peer_free(void *ptr) {
    if (!ptr) return ASCAN_ERR_INVALID_ARG;
    if (cudaFree(ptr) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_DEVICE;
    }
    return ASCAN_OK;
}

int ascan_check(void *ws, void *stream) {
    if (!ws) return ASCAN_ERR_INVALID_ARG;
    uint32_t host[4] = {0, 0, 0, 0};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(host, ws, sizeof(host), cudaMemcpyDeviceToHost, st) != cudaSuccess) return ASCAN_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return ASCAN_ERR_LAUNCH;
    if (host[0] == 0) return ASCAN_OK;
    if (cudaMemsetAsync(ws, 0, sizeof(uint32_t), st) != cudaSuccess) return ASCAN_ERR_LAUNCH;
    return ASCAN_ERR_TIMEOUT;
}

// ---------------------------------------------------------------------------
// Forward scan for callers that cannot supply scratch memory.
//
// The other entry points leave allocation to the caller: to get dynamic load balancing
// and split rows they want a zero-filled workspace.  Some callers cannot provide one:
// a host that reserved all device memory at start-up (a later cudaMalloc fails), a
// serving loop that may not call cudaMalloc because it synchronises the whole device,
// or a binding that can only pass the input and output buffers it already owns.  For
// them the workspace below is part of the library image: every GPU that loads the
// library holds these bytes until the process exits.
constexpr int64_t kNoAllocMaxRows = 16384;
static __device__ __align__(256) unsigned char g_no_alloc_scratch[CTRL_BYTES + CARRY_RECORD_BYTES * kNoAllocMaxRows];

// Device address of g_no_alloc_scratch on the current device.  In host code the array's
// name is only a handle for the runtime, not a pointer a kernel could use, so the address
// is asked for once per device (with that device current) and remembered.
static int no_alloc_scratch_address(unsigned char **out) {
    static std::mutex mu;
    static unsigned char *addr[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (dev < 0 || dev >= 64) return ASCAN_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_no_alloc_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return ASCAN_ERR_DEVICE;
        }
        addr[dev] = static_cast<unsigned char *>(ptr);
    }
    *out = addr[dev];
    return ASCAN_OK;
}

int ascan_forward_no_alloc(const void *gates, const void *tokens, void *out, int64_t rows, int64_t seqlen, int dtype,
                           int reverse, void *stream) {
    if (rows < 0 || seqlen < 1 || dtype_size(dtype) == 0) return ASCAN_ERR_INVALID_ARG;
    if (rows > kNoAllocMaxRows) return ASCAN_ERR_TOO_LARGE;
    if (rows == 0) return ASCAN_OK;
    if (!gates || !tokens || !out) return ASCAN_ERR_INVALID_ARG;
    unsigned char *scratch = nullptr;
    int rc = no_alloc_scratch_address(&scratch);
    if (rc != ASCAN_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left.  The work ticket and the exit
    // counter must start at zero.  The status word in front of them is left alone, so a
    // timeout of an earlier call stays readable by ascan_check_no_alloc; so is the launch
    // epoch behind them, which tells this call's carry records from older ones.
    if (cudaMemsetAsync(scratch + sizeof(uint32_t), 0, 2 * sizeof(uint32_t), st) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_LAUNCH;
    }
    ascan_plan pl;
    const bool al = aligned16(gates) && aligned16(tokens) && aligned16(out);
    rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_FORWARD, al, scratch, sizeof(g_no_alloc_scratch), &pl, reverse != 0);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens;
    p.out0 = out;
    fill_common(p, pl, rows, seqlen, scratch, sizeof(g_no_alloc_scratch));
    return launch_by_dtype(dtype, VARIANT_PLAIN, ASCAN_KIND_FORWARD, reverse != 0, p, pl, st);
}

int ascan_check_no_alloc(void *stream) {
    unsigned char *scratch = nullptr;
    int rc = no_alloc_scratch_address(&scratch);
    if (rc != ASCAN_OK) return rc;
    return ascan_check(scratch, stream);
}

}  // extern "C"

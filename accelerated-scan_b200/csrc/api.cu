// extern "C" entry points of the library (declared in include/ascan_b200.h):
// argument validation, planning, kernel dispatch, launch-error reporting.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>
#include <set>
#include <utility>

#include "../../include/ascan_b200.h"
#include "planner.h"
#include "stream.cuh"
#include "team.cuh"

namespace ascan {

static int cached_sm_count(int *out) {
    static int counts[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (dev >= 0 && dev < 64 && counts[dev] > 0) {
        *out = counts[dev];
        return ASCAN_OK;
    }
    int n = 0, major = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    if (major != 10 || n < 1) return ASCAN_ERR_DEVICE;   // built for sm_100a only
    if (dev >= 0 && dev < 64) counts[dev] = n;
    *out = n;
    return ASCAN_OK;
}

// Opt in to the large dynamic shared-memory carve-out once per (kernel, device).
static int ensure_smem(const void *fn, size_t bytes) {
    static std::mutex mu;
    static std::set<std::pair<const void *, int>> done;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ASCAN_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(mu);
    if (done.count({fn, dev})) return ASCAN_OK;
    (void)bytes;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemPerCta) != cudaSuccess) {
        cudaGetLastError();
        return ASCAN_ERR_LAUNCH;
    }
    done.insert({fn, dev});
    return ASCAN_OK;
}

template <class TR, int NCH, int KIND, bool REVERSE, bool BULK, bool INTERIOR, bool LOOKBACK = false>
static int launch_one(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    auto kfn = stream_kernel<TR, NCH, KIND, REVERSE, BULK, INTERIOR, LOOKBACK>;
    int rc = ensure_smem(reinterpret_cast<const void *>(kfn), pl.smem_bytes);
    if (rc != ASCAN_OK) return rc;
    kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
}

// INTERIOR: items that group several rows have row boundaries inside their tiles.
template <class TR, int NCH, int KIND, bool REVERSE, bool BULK>
static int launch_interior(const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    // look-back plans exist for the bulk loader and the two scan kinds; team plans also for
    // the carry-only kinds of the real dtypes
    if constexpr (BULK && (KIND == K_SCAN || KIND == K_BWD)) {
        if (pl.kernel == 1) return launch_one<TR, NCH, KIND, REVERSE, BULK, false, true>(p, pl, stream);
    }
    if constexpr (BULK && (KIND == K_SCAN || KIND == K_BWD || sizeof(typename TR::V) == 4)) {
        if (pl.kernel == 2) {
            auto kfn = team_kernel<TR, NCH, KIND, REVERSE>;
            int rc = ensure_smem(reinterpret_cast<const void *>(kfn), pl.smem_bytes);
            if (rc != ASCAN_OK) return rc;
            kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, stream>>>(p);
            return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
        }
    }
    if (pl.kernel != 0) return ASCAN_ERR_UNSUPPORTED;
    return pl.rows_per_item > 1 ? launch_one<TR, NCH, KIND, REVERSE, BULK, true>(p, pl, stream)
                                : launch_one<TR, NCH, KIND, REVERSE, BULK, false>(p, pl, stream);
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
            // two chunks per lane: planned for the fused backward of the 16-bit dtypes only
            if constexpr (KIND == K_BWD && TR::EPC == 8) {
                if (pl.kernel == 0) return launch_loader<TR, 2, KIND, REVERSE>(p, pl, stream);
            }
            return ASCAN_ERR_UNSUPPORTED;
        default: return ASCAN_ERR_UNSUPPORTED;
    }
}

template <int KIND, bool REVERSE>
static int launch_dtype(int dtype, const StreamParams &p, const ascan_plan &pl, cudaStream_t stream) {
    switch (dtype) {
        case ASCAN_F32: return launch_nch<TraitsF32, KIND, REVERSE>(p, pl, stream);
        case ASCAN_BF16: return launch_nch<TraitsBF16, KIND, REVERSE>(p, pl, stream);
        case ASCAN_F16: return launch_nch<TraitsF16, KIND, REVERSE>(p, pl, stream);
        case ASCAN_C64: return launch_nch<TraitsC64, KIND, REVERSE>(p, pl, stream);
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

static int l2_hints_env() {
    const char *v = getenv("ASCAN_L2_HINTS");
    int bits = (v && *v) ? (atoi(v) & 15) : 0;
    // test hook: one carry hand-over is dropped so that a bounded device-side wait expires
    const char *d = getenv("ASCAN_TEST_DROP_CARRY");
    if (d && *d == '1') bits |= 256;
    return bits;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int plan_for(int64_t rows, int64_t seqlen, int dtype, int kind, bool aligned, const void *ws, size_t ws_bytes,
                    ascan_plan *pl, bool reverse = false) {
    PlanInput in;
    in.reverse = reverse;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = dtype;
    in.kind = kind;
    in.aligned = aligned;
    in.workspace = ws && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0;
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    // prefer the plan that wants the most scratch; step down while the caller's is too small
    rc = make_plan(in, pl);
    if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes && in.workspace) {
        in.allow_lookback = false;
        rc = make_plan(in, pl);
        if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes) {
            in.workspace = false;
            rc = make_plan(in, pl);
        }
    }
    return rc;
}

// Copies the plan's decomposition and the workspace pointers into the kernel parameters.
static void fill_common(StreamParams &p, const ascan_plan &pl, int64_t rows, int64_t seqlen, void *ws) {
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
    p.l2_hints = l2_hints_env();
    p.team_size = pl.team_size;
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
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    rc = make_plan(in, pl);
    if (rc == ASCAN_OK && pl->workspace_bytes > ws_bytes && in.workspace) {
        in.workspace = false;
        rc = make_plan(in, pl);
    }
    if (rc != ASCAN_OK) return rc;
    if (pl->loader != 0 || pl->rows_per_item != 1 || pl->kernel != 0) return ASCAN_ERR_UNSUPPORTED;
    return ASCAN_OK;
}

template <class KFN>
static int launch_variant(KFN kfn, const StreamParams &p, const ascan_plan &pl, cudaStream_t st) {
    int rc = ensure_smem(reinterpret_cast<const void *>(kfn), pl.smem_bytes);
    if (rc != ASCAN_OK) return rc;
    kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
}

template <class TR>
static int launch_sigmoid(int kind, const StreamParams &p, const ascan_plan &pl, cudaStream_t st) {
    if (kind == ASCAN_KIND_FORWARD) {
        if (pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
        return launch_variant(stream_kernel<TR, 3, K_SCAN, false, true, false, false, false, 1>, p, pl, st);
    }
    if (pl.chunks_per_lane != 3) return ASCAN_ERR_UNSUPPORTED;
    return launch_variant(stream_kernel<TR, 3, K_BWD, true, true, false, false, false, 1>, p, pl, st);
}

static int launch_sigmoid_dtype(int dtype, int kind, const StreamParams &p, const ascan_plan &pl, cudaStream_t st) {
    switch (dtype) {
        case ASCAN_F32: return launch_sigmoid<TraitsF32>(kind, p, pl, st);
        case ASCAN_BF16: return launch_sigmoid<TraitsBF16>(kind, p, pl, st);
        case ASCAN_F16: return launch_sigmoid<TraitsF16>(kind, p, pl, st);
        default: return ASCAN_ERR_UNSUPPORTED;
    }
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
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_FORWARD, al, ws, ws_bytes, &pl, reverse != 0);
    if (rc != ASCAN_OK) return rc;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens;
    p.out0 = out;
    p.carry_in = carry_in;
    fill_common(p, pl, rows, seqlen, ws);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return reverse ? launch_dtype<K_SCAN, true>(dtype, p, pl, st) : launch_dtype<K_SCAN, false>(dtype, p, pl, st);
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
    int rc = plan_for(rows, seqlen, dtype, ASCAN_KIND_BACKWARD, al, ws, ws_bytes, &pl);
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_dtype<K_BWD, true>(dtype, p, pl, static_cast<cudaStream_t>(stream));
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_dtype<K_REDUCE, false>(dtype, p, pl, static_cast<cudaStream_t>(stream));
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_dtype<K_REDUCE_BWD, true>(dtype, p, pl, static_cast<cudaStream_t>(stream));
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
    if (cached_sm_count(&in.sm_count) != ASCAN_OK) {
        cudaGetLastError();
        in.sm_count = 148;          // no device to ask: size for a full B200
    }
    ascan_plan pl;
    if (make_plan(in, &pl) != ASCAN_OK) return static_cast<size_t>(workspace_bytes(rows));
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
    if (sm_count <= 0) {
        int rc = cached_sm_count(&in.sm_count);
        if (rc != ASCAN_OK) return rc;
    }
    return make_plan(in, plan);
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
    PlanInput in;
    in.reverse = reverse != 0;
    in.rows = rows;
    in.seqlen = seqlen;
    in.dtype = ASCAN_C64;
    in.kind = ASCAN_KIND_FORWARD;
    in.aligned = true;
    in.workspace = ws && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0;
    in.allow_lookback = false;
    in.allow_team = false;
    int rc = cached_sm_count(&in.sm_count);
    if (rc != ASCAN_OK) return rc;
    ascan_plan pl;
    rc = make_plan(in, &pl);
    if (rc == ASCAN_OK && pl.workspace_bytes > ws_bytes && in.workspace) {
        in.workspace = false;
        rc = make_plan(in, &pl);
    }
    if (rc != ASCAN_OK) return rc;
    if (pl.loader != 0 || pl.rows_per_item != 1 || pl.kernel != 0) return ASCAN_ERR_UNSUPPORTED;
    StreamParams p = {};
    p.in0 = gates;
    p.in1 = tokens_real;
    p.out0 = out;
    fill_common(p, pl, rows, seqlen, ws);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kfn) -> int {
        int r2 = ensure_smem(reinterpret_cast<const void *>(kfn), pl.smem_bytes);
        if (r2 != ASCAN_OK) return r2;
        kfn<<<pl.grid, pl.warps_per_cta * 32, pl.smem_bytes, st>>>(p);
        return cudaGetLastError() == cudaSuccess ? ASCAN_OK : ASCAN_ERR_LAUNCH;
    };
    return reverse ? launch(stream_kernel<TraitsC64, 3, K_SCAN, true, true, false, false, true>)
                   : launch(stream_kernel<TraitsC64, 3, K_SCAN, false, true, false, false, true>);
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_variant(stream_kernel<TraitsC64, 3, K_BWD, true, true, false, false, true>, p, pl,
                          static_cast<cudaStream_t>(stream));
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_sigmoid_dtype(dtype, ASCAN_KIND_FORWARD, p, pl, static_cast<cudaStream_t>(stream));
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
    fill_common(p, pl, rows, seqlen, ws);
    return launch_sigmoid_dtype(dtype, ASCAN_KIND_BACKWARD, p, pl, static_cast<cudaStream_t>(stream));
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
    // The array keeps whatever the previous call left.  The status word, the work ticket
    // and the exit counter must start at zero; the launch epoch behind them must survive,
    // because it is what tells this call's carry records from older ones.
    if (cudaMemsetAsync(scratch, 0, 3 * sizeof(uint32_t), st) != cudaSuccess) {
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
    fill_common(p, pl, rows, seqlen, scratch);
    return reverse ? launch_dtype<K_SCAN, true>(dtype, p, pl, st) : launch_dtype<K_SCAN, false>(dtype, p, pl, st);
}

}  // extern "C"

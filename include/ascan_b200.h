/*
 * ascan_b200 — C ABI of the B200 (sm_100a) first-order scan library.
 *
 *     x[t] = gate[t] * x[t-1] + token[t]          (forward)
 *     g[t] = grad_out[t] + conj(gate[t+1]) * g[t+1]
 *     d_token[t] = g[t],  d_gate[t] = conj(x[t-1]) * g[t]   (backward)
 *
 * Every array is a dense row-major matrix of `rows` x `seqlen` elements (the
 * reference's contiguous (B, C, T) tensors with rows = B*C; warp.cuh:267-276).
 * All pointers are DEVICE pointers on the current CUDA device; the library
 * allocates nothing and launches asynchronously on the stream it is given (a
 * cudaStream_t passed as void*; NULL = default stream).  What lives between calls
 * is in the caller's workspace, with two exceptions: the process-wide options of
 * ascan_set_option, and the built-in scratch array of ascan_forward_no_alloc
 * (launch epoch and carry records of its previous call).  The library reads no
 * environment variables.  Every function returns an ascan_status; 0 is success.
 *
 * Results are bitwise reproducible from run to run for every plan: the order in
 * which partial results are combined is fixed by the plan, never by timing.
 *
 * This header replaces the reference's pybind/ATen boundary
 * (accelerated_scan/warp.py:8-11,29-30 and accelerated_scan/warp.cuh:394-424) and
 * the Triton launch sites of accelerated_scan/complex.py:174-180,205-213.
 */
#ifndef ASCAN_B200_H
#define ASCAN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    ASCAN_OK = 0,
    ASCAN_ERR_INVALID_ARG = 1,   /* null pointer, rows < 0, seqlen < 1, bad enum          */
    ASCAN_ERR_UNSUPPORTED = 2,   /* combination the library does not implement            */
    ASCAN_ERR_LAUNCH = 3,        /* the CUDA runtime rejected the launch                  */
    ASCAN_ERR_TIMEOUT = 4,       /* a bounded device-side wait gave up (see ascan_check)  */
    ASCAN_ERR_WORKSPACE = 5,     /* workspace missing, misaligned or too small            */
    ASCAN_ERR_DEVICE = 6,        /* no sm_100 device / runtime query failed               */
    ASCAN_ERR_TOO_LARGE = 7      /* more rows than ascan_forward_no_alloc's scratch holds */
} ascan_status;

/* Storage type of gates/tokens/outputs.  Arithmetic is always fp32 (complex64:
 * pairs of fp32).  Replaces the dtype switch of warp.cuh:383-392. */
typedef enum {
    ASCAN_F32 = 0,
    ASCAN_BF16 = 1,
    ASCAN_F16 = 2,
    ASCAN_C64 = 3                /* interleaved (re, im) fp32 pairs, complex.py:171-173   */
} ascan_dtype;

/* Which computation a plan / workspace query is for. */
typedef enum {
    ASCAN_KIND_FORWARD = 0,
    ASCAN_KIND_BACKWARD = 1,
    ASCAN_KIND_REDUCE_FORWARD = 2,
    ASCAN_KIND_REDUCE_BACKWARD = 3
} ascan_kind;

/* Launch plan chosen by the planner; replaces the 12-case sequence-length ladder
 * of warp.cuh:282-380.  Pure host arithmetic, usable without a GPU when
 * sm_count > 0 is passed. */
typedef struct {
    int32_t kernel;            /* 0 = stream: one warp per item, segments of a row chained; 1 = look-back (very few rows, or rows sharded along time: a CTA keeps a segment in shared memory, one part per worker warp, segments are scanned concurrently, incoming states come from segment aggregates; warps_per_cta counts the workers and the CTA's bookkeeper warp); 2 = team (fewer than four rows per warp: several warps share an item) */
    int32_t loader;            /* 0 = bulk-async copies into shared-memory stages, 1 = plain element loads (unaligned data) */
    int32_t chunks_per_lane;   /* 16-byte chunks each lane owns per tile                  */
    int32_t stages;            /* shared-memory stages per warp (look-back: tiles per worker and segment) */
    int32_t warps_per_cta;
    int32_t grid;              /* persistent CTAs                                          */
    int32_t tile_elems;        /* elements per warp tile                                   */
    int32_t dynamic;           /* 1 = items drawn from a ticket counter in the workspace   */
    int32_t team_size;         /* warps that share an item (1 unless kernel == 2)          */
    int32_t row_grid;          /* 1 = short rows on the grid of tiles and lanes: items group whole rows, no per-element row-boundary work */
    int64_t rows_per_item;     /* rows grouped into one item when rows are not split       */
    int64_t row_groups;        /* ceil(rows / rows_per_item)                               */
    int64_t seg_elems;         /* steps per coarse segment when rows are split             */
    int64_t fine_elems;        /* steps per fine segment (the part of a row processed last) */
    int64_t coarse_segs;       /* coarse segments per row                                  */
    int64_t fine_segs;         /* fine segments per row                                    */
    int64_t segs_per_row;      /* coarse_segs + fine_segs; 1 = rows are not split          */
    int64_t items;             /* row_groups * segs_per_row                                */
    uint64_t smem_bytes;       /* dynamic shared memory per CTA                            */
    uint64_t workspace_bytes;  /* scratch the plan uses (0 = none)                         */
} ascan_plan;

/* Library version: major*10000 + minor*100 + patch. */
int ascan_version(void);

/* Static message for a status code. */
const char *ascan_strerror(int status);

/*
 * Forward scan.  Replaces warpscan_forward(gates, tokens, out, reverse)
 * (warp.cuh:394-405) and complex forward_scan (complex.py:20-65).
 *   reverse  != 0 solves x[t] = gate[t]*x[t+1] + token[t] from the last step.
 *   carry_in (nullable): `rows` values of the compute type (float, or float2 for
 *            ASCAN_C64): the state before the first step of every row (after the
 *            last step when reverse).  NULL means zero.
 *   ws/ws_bytes: scratch of ascan_workspace_bytes(...) bytes, 256-byte aligned,
 *            zero-filled ONCE by the caller before its first use and then left
 *            alone (the kernels rearm it); one workspace must not be shared by
 *            launches that can overlap (use one per stream).  NULL = static mode.
 */
int ascan_forward(const void *gates, const void *tokens, void *out,
                  int64_t rows, int64_t seqlen, int dtype, int reverse,
                  const void *carry_in, void *ws, size_t ws_bytes, void *stream);

/*
 * Fused backward.  Replaces warpscan_backward(gates, output, outGrad, gateGradOut,
 * tokenGradOut) (warp.cuh:407-424) and complex backward_scan (complex.py:68-154).
 * The three nullable arrays serve time-sharded callers and hold `rows` values of
 * the compute type:
 *   carry_in         g just after the last step of the row (NULL = 0)
 *   halo_gate_right  gate of the step after the last one    (only read with carry_in)
 *   halo_state_left  state before the first step            (NULL = 0)
 */
int ascan_backward(const void *gates, const void *states, const void *grad_out,
                   void *d_gates, void *d_tokens,
                   int64_t rows, int64_t seqlen, int dtype,
                   const void *carry_in, const void *halo_gate_right,
                   const void *halo_state_left,
                   void *ws, size_t ws_bytes, void *stream);

/*
 * Carry of every row without writing the scan: carry_out[2*r] = product of the
 * row's gates, carry_out[2*r+1] = last state of the row started from zero
 * (compute type).  No counterpart in the reference (it has no multi-GPU path);
 * it is the local step of the time-sharded scan.
 */
int ascan_reduce_forward(const void *gates, const void *tokens, void *carry_out,
                         int64_t rows, int64_t seqlen, int dtype,
                         void *ws, size_t ws_bytes, void *stream);

/*
 * Carry of the backward recurrence: carry_out[2*r] = product over the row of
 * conj(gate[t+1]) (gate[seqlen] := halo_gate_right[r], or 1 when NULL),
 * carry_out[2*r+1] = g[0] of the row started from zero.  No counterpart in the
 * reference.
 */
int ascan_reduce_backward(const void *gates, const void *grad_out,
                          const void *halo_gate_right, void *carry_out,
                          int64_t rows, int64_t seqlen, int dtype,
                          void *ws, size_t ws_bytes, void *stream);

/*
 * Complex forward scan with REAL tokens: gates and out are complex64, tokens_real
 * is fp32 and its imaginary part is taken as zero.  Fuses the promotion
 * torch.complex(inputs, zeros) of the reference's complex Scan.forward
 * (complex.py:162,168-169), which otherwise writes and re-reads a whole complex
 * tensor.  Needs 16-byte aligned pointers and seqlen % 4 == 0, and shapes the
 * stream plan handles with one row or segment per item; otherwise it returns
 * ASCAN_ERR_UNSUPPORTED and the caller promotes the tokens itself.
 */
int ascan_forward_complex_real_tokens(const void *gates, const void *tokens_real, void *out,
                                      int64_t rows, int64_t seqlen, int reverse,
                                      void *ws, size_t ws_bytes, void *stream);

/*
 * Fused complex backward for REAL tokens: as ascan_backward with dtype complex64,
 * but d_tokens_real receives only the real part of the token gradient, as fp32
 * (rows x seqlen floats).  This is what the reference's complex Scan.backward
 * returns for real inputs (`d_inputs.real`, complex.py:217-218) without writing
 * the complex gradient first.  Same conditions and fallback rule as
 * ascan_forward_complex_real_tokens.
 */
int ascan_backward_complex_real_tokens(const void *gates, const void *states, const void *grad_out,
                                       void *d_gates, void *d_tokens_real,
                                       int64_t rows, int64_t seqlen,
                                       void *ws, size_t ws_bytes, void *stream);

/*
 * Scan whose gates are sigmoid(gate_logits), the activation fused into the kernels
 * (real dtypes only).  The reference takes ready-made gates (warp.py:68-83), so a
 * caller with sigmoid gates runs an elementwise pass before the scan and another
 * one in the backward; here the forward reads the logits and the backward returns
 * d_logits[t] = x[t-1] * g[t] * s[t] * (1 - s[t]) directly.  The sigmoid is
 * evaluated in fp32 and is never rounded to the storage dtype.  Needs 16-byte
 * aligned pointers and a shape the stream plan handles with one row or segment per
 * item; otherwise ASCAN_ERR_UNSUPPORTED is returned and the caller applies the
 * activation itself.  No counterpart in the reference.
 */
int ascan_forward_sigmoid_gates(const void *gate_logits, const void *tokens, void *out,
                                int64_t rows, int64_t seqlen, int dtype,
                                void *ws, size_t ws_bytes, void *stream);
int ascan_backward_sigmoid_gates(const void *gate_logits, const void *states, const void *grad_out,
                                 void *d_logits, void *d_tokens,
                                 int64_t rows, int64_t seqlen, int dtype,
                                 void *ws, size_t ws_bytes, void *stream);

/*
 * Time-sharded scans: folds the carries gathered from all ranks into this rank's
 * incoming state.  `gathered` holds world x rows x stride values of the compute
 * type (float, or float2 for ASCAN_C64; other dtypes use float): {P, S, first gate}
 * per rank and row (stride 3) or {P, S} (stride 2).  suffix == 0: state_out[r] =
 * composition of ranks 0..rank-1 applied to zero (forward); suffix != 0: of ranks
 * world-1..rank+1 (backward).  halo_out (nullable): first gate of rank+1, or one.
 * No counterpart in the reference.
 */
int ascan_fold_carries(const void *gathered, int64_t rows, int world, int rank,
                       int stride, int dtype, int suffix,
                       void *state_out, void *halo_out, void *stream);

/*
 * Time-sharded scan: every rank (one GPU each) holds a contiguous time slice of ALL rows
 * (rank order = time order) and calls the same function on its slice.  Each rank streams its
 * slice once; the state entering the slice is folded from the slice aggregates that the other
 * ranks store, with plain 64-bit peer stores, into this rank's exchange buffer, so the ranks run
 * at the same time and no collective is involved.  No counterpart in the reference (it has no
 * multi-device path).
 *   exchange   `world` device pointers: exchange[j] is rank j's exchange buffer as mapped in
 *              THIS process (exchange[rank] is the local one): peer-accessible memory of
 *              ascan_exchange_bytes(rows, world) bytes, 16-byte aligned, zero-filled once
 *              before its first use.  One buffer set per direction: the forward calls of a
 *              group of ranks share one set, the backward calls another.  world == 1 ignores it.
 *   call       number of this call on its buffer set: 1, 2, 3, ... and the same on every rank.
 *              Ranks may drift apart by at most one call; a rank that gets further ahead waits
 *              (bounded) for the slower ones.
 *   carry_save (forward, nullable) receives, per row, the state entering this rank's slice
 *              (compute type); pass it as halo_state_left of the backward.
 *   ws         required: ascan_workspace_bytes_time_sharded(...) bytes, 256-byte aligned,
 *              zero-filled once; not shared with launches that can overlap.
 * carry_in of the whole sequence is not supported (the sequence starts from zero).  Needs
 * 16-byte aligned pointers and seqlen * element size divisible by 16; otherwise
 * ASCAN_ERR_UNSUPPORTED.  Kernels of different ranks wait for one another's aggregates: run
 * each rank on a GPU of its own.
 */
size_t ascan_exchange_bytes(int64_t rows, int world);
size_t ascan_workspace_bytes_time_sharded(int64_t rows, int64_t seqlen, int dtype, int kind);
int ascan_forward_time_sharded(const void *gates, const void *tokens, void *out,
                               int64_t rows, int64_t seqlen, int dtype,
                               int rank, int world, uint32_t call, void *const *exchange,
                               void *carry_save, void *ws, size_t ws_bytes, void *stream);
int ascan_backward_time_sharded(const void *gates, const void *states, const void *grad_out,
                                void *d_gates, void *d_tokens,
                                int64_t rows, int64_t seqlen, int dtype,
                                int rank, int world, uint32_t call, void *const *exchange,
                                const void *halo_state_left,
                                void *ws, size_t ws_bytes, void *stream);

/*
 * Exchange buffers for ranks that are separate processes.  ascan_peer_alloc allocates
 * `bytes` of zero-filled device memory on the current device (cudaMalloc: these four are the
 * only functions of the library that allocate or free) and fills `handle64` (64 bytes) with
 * an inter-process handle; the handle travels to the other ranks by any host channel, and
 * ascan_peer_open maps that rank's buffer into this process with peer access enabled.
 * ascan_peer_close unmaps, ascan_peer_free releases the local buffer.  Ranks inside one
 * process pass their device pointers directly and need none of this.  No counterpart in
 * the reference.
 */
int ascan_peer_alloc(size_t bytes, void **ptr, void *handle64);
int ascan_peer_open(const void *handle64, void **ptr);
int ascan_peer_close(void *ptr);
int ascan_peer_free(void *ptr);

/*
 * Scratch bytes a call of `kind` with these sizes can use: a control block
 * (status word, work ticket) plus one carry record per row, or 32 bytes per segment,
 * block of 32 segments and super-block when the look-back plan applies (clearly fewer
 * rows than SMs: 3/4 of them, 3/2 for the forward kind).  With that much scratch
 * the kernels balance work over the SMs dynamically and split long rows across
 * warps and CTAs; with less they step down to the chained plan (256 + 32*rows
 * bytes), and with none (NULL) to a static deal of whole rows: correct, slower.
 */
size_t ascan_workspace_bytes(int64_t rows, int64_t seqlen, int dtype, int kind);

/*
 * The plan the library would use.  flags: bit 0 = every pointer is 16-byte
 * aligned, bit 1 = a workspace of ascan_workspace_bytes() is supplied, bit 2 =
 * forward kind with reverse != 0, bit 3 = never choose the look-back plan, bit 4 = never
 * choose the team plan, bit 5 = the call has seeds (carry_in or halos: no row-grid kernels);
 * sm_count <= 0 queries the current device.  Host only.
 */
int ascan_plan_describe(int64_t rows, int64_t seqlen, int dtype, int kind,
                        int flags, int sm_count, ascan_plan *plan);

/*
 * Reads the device status word at the start of a workspace after synchronising
 * `stream`.  Returns ASCAN_OK, or ASCAN_ERR_TIMEOUT when a bounded device-side
 * wait expired in an earlier launch that used this workspace (the word is then
 * cleared).  Optional: the hot path never synchronises.
 */
int ascan_check(void *ws, void *stream);

/*
 * Workspace layout, for callers that want failures reported without a
 * synchronisation: bytes 0-3 status word, 4-15 ticket / exit counter / launch
 * epoch (owned by the kernels), bytes 16-23 an optional 64-bit device-accessible
 * address of a second status word, written by the CALLER once after zero-filling
 * the workspace (0 = none).  If that address is mapped pinned host memory, a
 * kernel whose bounded wait expires also stores its status bits there, and the
 * host notices by reading its own memory before its next call.
 */

/*
 * Process-wide options.  Defaults are the measured optimum; the tuning options
 * exist for sweeps, the TEST options for the test-suite (they make a bounded wait
 * expire, or the launch epoch wrap early, without faulting anything).  Returns
 * ASCAN_ERR_INVALID_ARG for an unknown option or a value out of range.  No
 * counterpart in the reference.
 */
typedef enum {
    ASCAN_OPT_STAGES = 0,          /* shared-memory stages per warp, 1..8 (default 2)          */
    ASCAN_OPT_WARPS_PER_CTA = 1,   /* upper bound on warps per CTA, 0 = planner's choice       */
    ASCAN_OPT_LOOKBACK_TILES = 2,  /* tiles per worker and segment of the look-back plan      */
    ASCAN_OPT_DISABLE_PLANS = 3,   /* bit 0 no look-back, bit 1 no team, bit 2 static deal, bit 3 plain loader, bit 4 no row grid, bit 5 no four-chunk tiles */
    ASCAN_OPT_TEST_DROP_CARRY = 4, /* 1: drop one carry hand-over per launch (a wait expires)  */
    ASCAN_OPT_TEST_EPOCH_BITS = 5, /* width of the launch epoch, 1..17 (default 17)            */
    ASCAN_OPT_ITEMS_PER_WARP = 6,  /* items per warp that grouped short rows aim for (default 4) */
    ASCAN_OPT_STATIC_BELOW = 7     /* unsplit rows: up to this many items per warp are dealt without tickets (default 8) */
} ascan_option;
int ascan_set_option(int option, int value);
int ascan_get_option(int option);          /* -1 for an unknown option */

/*
 * Forward scan that needs no workspace from the caller.  It has no counterpart in
 * the reference.  It is for callers that cannot hand over scratch memory: hosts
 * that reserve all device memory at start-up (so a later cudaMalloc fails),
 * serving loops that must not call cudaMalloc because it synchronises the device,
 * and bindings that can only pass the buffers they already own.  The scratch is a
 * fixed array inside the library (about 0.5 MB on every GPU that loads it), which
 * limits the call to rows <= 16384; more rows return ASCAN_ERR_TOO_LARGE.  The
 * function allocates nothing.  Its first call on a device looks up the array's
 * device address (cudaGetSymbolAddress); make that first call outside any stream
 * capture.  All calls on a device share the one array, so two calls that may run
 * at the same time on that device (different streams or threads) race; order them.
 * Same arithmetic as ascan_forward with a workspace of that size; carry_in is not
 * supported.  A device-side timeout is kept in the array's status word until
 * ascan_check_no_alloc reads it.
 */
int ascan_forward_no_alloc(const void *gates, const void *tokens, void *out,
                           int64_t rows, int64_t seqlen, int dtype, int reverse,
                           void *stream);

/*
 * ascan_check for the built-in scratch of ascan_forward_no_alloc on the current
 * device: synchronises `stream`, returns ASCAN_ERR_TIMEOUT (and clears the word)
 * when a bounded wait expired in an earlier ascan_forward_no_alloc call.  No
 * counterpart in the reference.
 */
int ascan_check_no_alloc(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ASCAN_B200_H */

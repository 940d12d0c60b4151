/*
 * CPU oracle for the first-order scan  x[t] = a[t]*x[t-1] + b[t].
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is
 * compared against; it is never part of the product path.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * It restates, in plain C, the algorithm of the reference's CPU-capable
 * implementation accelerated_scan/ref.py (pure torch ops):
 *   - ref.py:77-83   pad T up to the next power of two with gate=1, token=0
 *   - ref.py:100-109 up-sweep: split a level into (even, odd) children and
 *                    combine them into the parent level
 *   - ref.py:111-114 identity (1, 0) at the root
 *   - ref.py:116-121 down-sweep: exclusive prefixes of the children from the
 *                    parent's exclusive prefix
 *   - ref.py:86      inclusive result  out = x_excl * gates + tokens
 * The recursion of ref.py is unrolled into loops over per-level arrays.  Every
 * multiply and add is a separate IEEE operation (compile with
 * -ffp-contract=off), in the same order as the torch ops of ref.py, so the
 * fp32 result is bit-identical to ref.py on CPU.
 *
 * The backward functions restate the reference's hand-written backward
 * (accelerated_scan/warp.py:50-65, accelerated_scan/scalar.py:69-84,
 * accelerated_scan/complex.py:86-92,113-115,144-147; the identity is pinned by
 * tests/test_eq.py:65-90): a reverse scan of grad_out over the gates shifted by
 * one step, then grad_gates[t] = conj(x[t-1]) * g[t].
 *
 * Rows are independent; they are spread over OpenMP threads.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct { float re, im; } c64;

static inline int64_t next_pow2(int64_t n) {
    int64_t p = 1;
    while (p < n) p <<= 1;
    return p;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ real */

/* One row of the ref.py tree (ref.py:49-121).  `lg`, `lx` are scratch arrays of
 * 2*P floats each: level 0 (length P) followed by level 1 (P/2) and so on.
 * `ex` is scratch of 2*P floats for the exclusive prefixes per level. */
static void tree_row_f32(const float *a, const float *b, float *out, int64_t T,
                         int reverse, float *lg, float *lx, float *ex) {
    const int64_t P = next_pow2(T);
    /* ref.py:77-83 padding */
    memcpy(lg, a, (size_t)T * sizeof(float));
    memcpy(lx, b, (size_t)T * sizeof(float));
    for (int64_t i = T; i < P; ++i) { lg[i] = 1.0f; lx[i] = 0.0f; }
    if (P == 1) {
        /* log2(1) = 0 levels never happens in the reference for T>=2; a single
         * step has the exclusive prefix 0. */
        out[0] = 0.0f * lg[0] + lx[0];
        return;
    }
    /* up-sweep (ref.py:100-109).  forward: left = even, right = odd.
     * reverse (ref.py:100-102): left = odd, right = even. */
    int64_t off = 0;
    for (int64_t n = P; n >= 2; n >>= 1) {
        const float *g = lg + off, *x = lx + off;
        float *pg = lg + off + n, *px = lx + off + n;
        for (int64_t i = 0; i < n / 2; ++i) {
            const int64_t l = reverse ? 2 * i + 1 : 2 * i;
            const int64_t r = reverse ? 2 * i : 2 * i + 1;
            pg[i] = g[l] * g[r];
            float m = g[r] * x[l];
            px[i] = m + x[r];
        }
        off += n;
    }
    /* `off` now points at the single-element top level, whose combined value
     * is unused: the root prefix is the identity (ref.py:111-112). */
    /* down-sweep (ref.py:116-121).  Only the token prefix feeds the output. */
    int64_t n = 2;
    int64_t loff = off - 2;            /* offset of the level of length 2 */
    ex[off] = 0.0f;                    /* root_x */
    int64_t poff = off;                /* offset of the parent prefix */
    while (1) {
        const float *g = lg + loff, *x = lx + loff;
        const float *pe = ex + poff;
        float *e = ex + loff;
        for (int64_t i = 0; i < n / 2; ++i) {
            const int64_t l = reverse ? 2 * i + 1 : 2 * i;
            const int64_t r = reverse ? 2 * i : 2 * i + 1;
            e[l] = pe[i];
            float m = pe[i] * g[l];
            e[r] = m + x[l];
        }
        if (n == P) break;
        poff = loff;
        n <<= 1;
        loff -= n;
    }
    /* ref.py:86-87 */
    for (int64_t t = 0; t < T; ++t) {
        float m = ex[t] * lg[t];
        out[t] = m + lx[t];
    }
}

/* Inclusive scan of every row with the tree of ref.py.  reverse!=0 solves the
 * recurrence from the last step to the first (ref.py:56, reverse=True). */
int oracle_tree_scan_f32(const float *gates, const float *tokens, float *out,
                         int64_t rows, int64_t T, int reverse) {
    if (rows < 0 || T < 1) return 1;
    const int64_t P = next_pow2(T);
    int fail = 0;
#pragma omp parallel
    {
        float *buf = (float *)malloc((size_t)(6 * P + 8) * sizeof(float));
        if (!buf) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            if (buf)
                tree_row_f32(gates + r * T, tokens + r * T, out + r * T, T, reverse,
                             buf, buf + 2 * P + 2, buf + 4 * P + 4);
        }
        free(buf);
    }
    return fail;
}

/* Backward of the real scan (warp.py:50-65; scalar.py:69-84):
 *   g[t]  = grad_out[t] + a[t+1] * g[t+1],  a[T] := 1   (reverse tree scan over shifted gates)
 *   d_tokens[t] = g[t]
 *   d_gates[t]  = x[t-1] * g[t],  x[-1] := 0 */
int oracle_backward_f32(const float *gates, const float *states, const float *grad_out,
                        float *d_gates, float *d_tokens, int64_t rows, int64_t T) {
    if (rows < 0 || T < 1) return 1;
    float *shifted = (float *)malloc((size_t)(rows * T + 1) * sizeof(float));
    if (!shifted) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t t = 0; t + 1 < T; ++t) shifted[r * T + t] = gates[r * T + t + 1];
        shifted[r * T + T - 1] = 1.0f;   /* tests/test_eq.py:77 pads with ones */
    }
    int rc = oracle_tree_scan_f32(shifted, grad_out, d_tokens, rows, T, 1);
    free(shifted);
    if (rc) return rc;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        d_gates[r * T] = 0.0f * d_tokens[r * T];
        for (int64_t t = 1; t < T; ++t)
            d_gates[r * T + t] = states[r * T + t - 1] * d_tokens[r * T + t];
    }
    return 0;
}

/* Straight evaluation of the recurrence in double precision (README.md:8 of the
 * reference states the recurrence).  Used to measure how far the fp32 tree and
 * the CUDA kernels sit from the exact answer. */
int oracle_seq_scan_f64(const float *gates, const float *tokens, double *out,
                        int64_t rows, int64_t T, int reverse) {
    if (rows < 0 || T < 1) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double x = 0.0;
        if (!reverse) {
            for (int64_t t = 0; t < T; ++t) {
                x = (double)gates[r * T + t] * x + (double)tokens[r * T + t];
                out[r * T + t] = x;
            }
        } else {
            for (int64_t t = T - 1; t >= 0; --t) {
                x = (double)gates[r * T + t] * x + (double)tokens[r * T + t];
                out[r * T + t] = x;
            }
        }
    }
    return 0;
}

/* --------------------------------------------------------------- complex */

/* Complex product (complex.py:6-8 states the formula).  torch evaluates it in
 * two roundings-orders on CPU, and ref.py meets both: its tree levels multiply
 * strided views (ref.py:23-24, 108-121), which torch 2.11 computes element by
 * element as  re = fma(a.re, b.re, -(a.im*b.im)),  im = fma(a.re, b.im, a.im*b.re);
 * the final step (ref.py:86) multiplies contiguous tensors, which torch computes
 * vectorised with four products, one subtract and one add.  Both are restated
 * so the oracle tracks ref.py to the last bit where torch's kernels allow. */
static inline c64 cmul_strided(c64 p, c64 q) {
    float bd = p.im * q.im, bc = p.im * q.re;
    c64 r = { fmaf(p.re, q.re, -bd), fmaf(p.re, q.im, bc) };
    return r;
}
static inline c64 cmul(c64 p, c64 q) {
    float ac = p.re * q.re, bd = p.im * q.im;
    float ad = p.re * q.im, bc = p.im * q.re;
    c64 r = { ac - bd, ad + bc };
    return r;
}
static inline c64 cadd(c64 p, c64 q) { c64 r = { p.re + q.re, p.im + q.im }; return r; }
static inline c64 cconj(c64 p) { c64 r = { p.re, -p.im }; return r; }

static void tree_row_c64(const c64 *a, const c64 *b, c64 *out, int64_t T,
                         int reverse, c64 *lg, c64 *lx, c64 *ex) {
    const int64_t P = next_pow2(T);
    const c64 one = { 1.0f, 0.0f }, zero = { 0.0f, 0.0f };
    memcpy(lg, a, (size_t)T * sizeof(c64));
    memcpy(lx, b, (size_t)T * sizeof(c64));
    for (int64_t i = T; i < P; ++i) { lg[i] = one; lx[i] = zero; }
    if (P == 1) { out[0] = cadd(cmul(zero, lg[0]), lx[0]); return; }
    int64_t off = 0;
    for (int64_t n = P; n >= 2; n >>= 1) {
        const c64 *g = lg + off, *x = lx + off;
        c64 *pg = lg + off + n, *px = lx + off + n;
        for (int64_t i = 0; i < n / 2; ++i) {
            const int64_t l = reverse ? 2 * i + 1 : 2 * i;
            const int64_t r = reverse ? 2 * i : 2 * i + 1;
            pg[i] = cmul_strided(g[l], g[r]);
            px[i] = cadd(cmul_strided(g[r], x[l]), x[r]);
        }
        off += n;
    }
    int64_t n = 2, loff = off - 2, poff = off;
    ex[off] = zero;
    while (1) {
        const c64 *g = lg + loff, *x = lx + loff;
        const c64 *pe = ex + poff;
        c64 *e = ex + loff;
        for (int64_t i = 0; i < n / 2; ++i) {
            const int64_t l = reverse ? 2 * i + 1 : 2 * i;
            const int64_t r = reverse ? 2 * i : 2 * i + 1;
            e[l] = pe[i];
            e[r] = cadd(cmul_strided(pe[i], g[l]), x[l]);
        }
        if (n == P) break;
        poff = loff;
        n <<= 1;
        loff -= n;
    }
    for (int64_t t = 0; t < T; ++t) out[t] = cadd(cmul(ex[t], lg[t]), lx[t]);
}

/* complex64 arrays are interleaved (re, im) float pairs, as torch.view_as_real
 * exposes them (complex.py:171-173). */
int oracle_tree_scan_c64(const float *gates, const float *tokens, float *out,
                         int64_t rows, int64_t T, int reverse) {
    if (rows < 0 || T < 1) return 1;
    const int64_t P = next_pow2(T);
    int fail = 0;
#pragma omp parallel
    {
        c64 *buf = (c64 *)malloc((size_t)(6 * P + 8) * sizeof(c64));
        if (!buf) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            if (buf)
                tree_row_c64((const c64 *)gates + r * T, (const c64 *)tokens + r * T,
                             (c64 *)out + r * T, T, reverse,
                             buf, buf + 2 * P + 2, buf + 4 * P + 4);
        }
        free(buf);
    }
    return fail;
}

/* Backward of the complex scan (complex.py:86-92,113-115,144-147):
 *   g[t] = d_out[t] + conj(a[t+1]) * g[t+1]
 *   d_inputs[t] = g[t];  d_forget[t] = conj(x[t-1]) * g[t] */
int oracle_backward_c64(const float *gates, const float *states, const float *grad_out,
                        float *d_gates, float *d_tokens, int64_t rows, int64_t T) {
    if (rows < 0 || T < 1) return 1;
    const c64 *a = (const c64 *)gates, *x = (const c64 *)states;
    c64 *dg = (c64 *)d_gates, *dt = (c64 *)d_tokens;
    c64 *shifted = (c64 *)malloc((size_t)(rows * T + 1) * sizeof(c64));
    if (!shifted) return 1;
    const c64 one = { 1.0f, 0.0f }, zero = { 0.0f, 0.0f };
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t t = 0; t + 1 < T; ++t) shifted[r * T + t] = cconj(a[r * T + t + 1]);
        shifted[r * T + T - 1] = one;
    }
    int rc = oracle_tree_scan_c64((const float *)shifted, grad_out, d_tokens, rows, T, 1);
    free(shifted);
    if (rc) return rc;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        dg[r * T] = cmul(zero, dt[r * T]);
        for (int64_t t = 1; t < T; ++t)
            dg[r * T + t] = cmul(cconj(x[r * T + t - 1]), dt[r * T + t]);
    }
    return 0;
}

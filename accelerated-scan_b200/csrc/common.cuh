// Shared device helpers: element traits (storage <-> fp32 compute values), the
// affine-pair arithmetic of the scan, and thin wrappers over the sm_100a PTX used
// by the kernels (mbarrier, bulk asynchronous copies, proxy fences).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ascan {

// ---------------------------------------------------------------- arithmetic
// A scan element is the affine map x -> a*x + b.  Real paths compute in float,
// the complex path in float2 = (re, im).  The combine rule is the one the
// reference states in scalar.py:6-13 / complex.py:11-17.

__device__ __forceinline__ float vzero(float) { return 0.0f; }
__device__ __forceinline__ float vone(float) { return 1.0f; }
__device__ __forceinline__ float vconj(float a) { return a; }
__device__ __forceinline__ float vmul(float a, float b) { return a * b; }
// a*x + b
__device__ __forceinline__ float vfma(float a, float x, float b) { return fmaf(a, x, b); }
__device__ __forceinline__ float vsel(bool p, float a, float b) { return p ? a : b; }

__device__ __forceinline__ float2 vzero(float2) { return make_float2(0.0f, 0.0f); }
__device__ __forceinline__ float2 vone(float2) { return make_float2(1.0f, 0.0f); }
__device__ __forceinline__ float2 vconj(float2 a) { return make_float2(a.x, -a.y); }
__device__ __forceinline__ float2 vmul(float2 a, float2 b) {
    return make_float2(fmaf(a.x, b.x, -(a.y * b.y)), fmaf(a.x, b.y, a.y * b.x));
}
__device__ __forceinline__ float2 vfma(float2 a, float2 x, float2 b) {
    return make_float2(fmaf(a.x, x.x, fmaf(-a.y, x.y, b.x)), fmaf(a.x, x.y, fmaf(a.y, x.x, b.y)));
}
__device__ __forceinline__ float2 vsel(bool p, float2 a, float2 b) {
    return make_float2(p ? a.x : b.x, p ? a.y : b.y);
}

__device__ __forceinline__ float shfl_up(float v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ float shfl_down(float v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
__device__ __forceinline__ float shfl_idx(float v, int l) { return __shfl_sync(0xffffffffu, v, l); }
__device__ __forceinline__ float2 shfl_up(float2 v, int d) {
    return make_float2(__shfl_up_sync(0xffffffffu, v.x, d), __shfl_up_sync(0xffffffffu, v.y, d));
}
__device__ __forceinline__ float2 shfl_down(float2 v, int d) {
    return make_float2(__shfl_down_sync(0xffffffffu, v.x, d), __shfl_down_sync(0xffffffffu, v.y, d));
}
__device__ __forceinline__ float2 shfl_idx(float2 v, int l) {
    return make_float2(__shfl_sync(0xffffffffu, v.x, l), __shfl_sync(0xffffffffu, v.y, l));
}

// Values handed from one warp to another through global memory travel in 64-bit words
// that carry their own tag: {fp32 payload, 32-bit tag}.  A 64-bit access is a single
// transaction, so a reader either sees the old word or the new word, payload and tag
// together; no fence or acquire/release pair is needed on either side.  A complex value
// uses two such words.  `slot` selects one of two values per 32-byte record.
__device__ __forceinline__ void st_relaxed_u64(void *p, uint64_t v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_u64(const void *p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t tagged_word(float payload, uint32_t tag) {
    return (static_cast<uint64_t>(tag) << 32) | __float_as_uint(payload);
}
__device__ __forceinline__ void publish_tagged(unsigned char *rec, int slot, float v, uint32_t tag) {
    st_relaxed_u64(rec + slot * 16, tagged_word(v, tag));
}
__device__ __forceinline__ void publish_tagged(unsigned char *rec, int slot, float2 v, uint32_t tag) {
    st_relaxed_u64(rec + slot * 16, tagged_word(v.x, tag));
    st_relaxed_u64(rec + slot * 16 + 8, tagged_word(v.y, tag));
}
// The words of one value, fetched now and checked later (see decode_tagged).
struct TaggedWords {
    uint64_t w0, w1;
};
__device__ __forceinline__ TaggedWords fetch_tagged(const unsigned char *rec, int slot, bool two_words) {
    TaggedWords t;
    t.w0 = ld_relaxed_u64(rec + slot * 16);
    t.w1 = two_words ? ld_relaxed_u64(rec + slot * 16 + 8) : 0;
    return t;
}
__device__ __forceinline__ bool decode_tagged(const TaggedWords &t, uint32_t tag, float &v) {
    v = __uint_as_float(static_cast<uint32_t>(t.w0));
    return static_cast<uint32_t>(t.w0 >> 32) == tag;
}
__device__ __forceinline__ bool decode_tagged(const TaggedWords &t, uint32_t tag, float2 &v) {
    v = make_float2(__uint_as_float(static_cast<uint32_t>(t.w0)), __uint_as_float(static_cast<uint32_t>(t.w1)));
    return static_cast<uint32_t>(t.w0 >> 32) == tag && static_cast<uint32_t>(t.w1 >> 32) == tag;
}
// Returns true and fills `v` when every word of the value carries `tag`.
__device__ __forceinline__ bool read_tagged(const unsigned char *rec, int slot, uint32_t tag, float &v) {
    const uint64_t w = ld_relaxed_u64(rec + slot * 16);
    v = __uint_as_float(static_cast<uint32_t>(w));
    return static_cast<uint32_t>(w >> 32) == tag;
}
__device__ __forceinline__ bool read_tagged(const unsigned char *rec, int slot, uint32_t tag, float2 &v) {
    const uint64_t w0 = ld_relaxed_u64(rec + slot * 16);
    const uint64_t w1 = ld_relaxed_u64(rec + slot * 16 + 8);
    v = make_float2(__uint_as_float(static_cast<uint32_t>(w0)), __uint_as_float(static_cast<uint32_t>(w1)));
    return static_cast<uint32_t>(w0 >> 32) == tag && static_cast<uint32_t>(w1 >> 32) == tag;
}

// ------------------------------------------------------------ element traits
// EPC = elements per 16-byte chunk.  unpack/pack convert one chunk between its
// storage form and EPC compute values.

struct TraitsF32 {
    using V = float;
    using Raw = uint32_t;
    static constexpr int EPC = 4;
    static constexpr int ESIZE = 4;
    __device__ __forceinline__ static void unpack(const uint4 &q, V *v) {
        v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y);
        v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
    }
    __device__ __forceinline__ static uint4 pack(const V *v) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]),
                          __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    __device__ __forceinline__ static V load_one(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const float *>(base) + i);
    }
    // load_raw + decode = load_one, split so that the conversion (the first use of the
    // loaded register) can sit where the value is needed instead of right after the load
    __device__ __forceinline__ static Raw load_raw(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const uint32_t *>(base) + i);
    }
    __device__ __forceinline__ static V decode(Raw r) { return __uint_as_float(r); }
};

struct TraitsBF16 {
    using V = float;
    using Raw = uint16_t;
    static constexpr int EPC = 8;
    static constexpr int ESIZE = 2;
    __device__ __forceinline__ static void unpack(const uint4 &q, V *v) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static uint4 pack(const V *v) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static V load_one(const void *base, int64_t i) {
        const uint16_t r = __ldg(reinterpret_cast<const uint16_t *>(base) + i);
        return __uint_as_float(static_cast<uint32_t>(r) << 16);
    }
    __device__ __forceinline__ static Raw load_raw(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const uint16_t *>(base) + i);
    }
    __device__ __forceinline__ static V decode(Raw r) { return __uint_as_float(static_cast<uint32_t>(r) << 16); }
};

struct TraitsF16 {
    using V = float;
    using Raw = uint16_t;
    static constexpr int EPC = 8;
    static constexpr int ESIZE = 2;
    __device__ __forceinline__ static void unpack(const uint4 &q, V *v) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ static uint4 pack(const V *v) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static V load_one(const void *base, int64_t i) {
        const unsigned short r = __ldg(reinterpret_cast<const unsigned short *>(base) + i);
        return __half2float(__ushort_as_half(r));
    }
    __device__ __forceinline__ static Raw load_raw(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const unsigned short *>(base) + i);
    }
    __device__ __forceinline__ static V decode(Raw r) { return __half2float(__ushort_as_half(r)); }
};

struct TraitsC64 {
    using V = float2;
    using Raw = uint64_t;
    static constexpr int EPC = 2;
    static constexpr int ESIZE = 8;
    __device__ __forceinline__ static void unpack(const uint4 &q, V *v) {
        v[0] = make_float2(__uint_as_float(q.x), __uint_as_float(q.y));
        v[1] = make_float2(__uint_as_float(q.z), __uint_as_float(q.w));
    }
    __device__ __forceinline__ static uint4 pack(const V *v) {
        return make_uint4(__float_as_uint(v[0].x), __float_as_uint(v[0].y),
                          __float_as_uint(v[1].x), __float_as_uint(v[1].y));
    }
    __device__ __forceinline__ static V load_one(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const float2 *>(base) + i);
    }
    __device__ __forceinline__ static Raw load_raw(const void *base, int64_t i) {
        return __ldg(reinterpret_cast<const unsigned long long *>(base) + i);
    }
    __device__ __forceinline__ static V decode(Raw r) {
        return make_float2(__uint_as_float(static_cast<uint32_t>(r)), __uint_as_float(static_cast<uint32_t>(r >> 32)));
    }
};

// ------------------------------------------------------------------ PTX glue

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes freshly initialised mbarriers visible to the asynchronous proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// One arrival on an mbarrier (release at CTA scope): what the arriving thread, and the threads
// it synchronised with before, wrote to shared memory is visible to whoever sees the phase end.
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Non-blocking test of a phase.
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` polls and reports false.  Every caller
// records the failure in a status word and leaves its loop instead of spinning.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// The same with a suspend-time hint: a thread whose phase is not complete sleeps in hardware
// for up to `hint_ns` per try instead of spinning through issue slots the other warps of the
// SM could use.  For waits that are expected to last a microsecond or so.
__device__ __forceinline__ bool mbar_wait_bounded_suspended(uint64_t *bar, uint32_t parity, uint32_t limit, uint32_t hint_ns) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// Bulk asynchronous copy global -> shared (no multicast), completion on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Bulk asynchronous copy shared -> global, tracked by the bulk async-group.
__device__ __forceinline__ void bulk_s2g(void *dst_gmem, const void *src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}

// L2 eviction-priority policies for streaming data (every byte is touched once).
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar,
                                              uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void bulk_s2g_hint(void *dst_gmem, const void *src_smem, uint32_t bytes, uint64_t pol) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes), "l"(pol)
                 : "memory");
}

// Asks for a range of global memory to be brought into L2 (a hint: no completion to wait for).
// Address 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src_gmem, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most N committed bulk groups still have to READ their shared source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until at most N committed bulk groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders generic-proxy accesses to shared memory before later asynchronous-proxy ones.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Status bits written by kernels whose bounded waits expire.
constexpr uint32_t STATUS_LOAD_TIMEOUT = 1u;
constexpr uint32_t STATUS_LOOKBACK_TIMEOUT = 2u;

}  // namespace ascan

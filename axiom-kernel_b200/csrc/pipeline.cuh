// Asynchronous row pipeline primitives for sm_100a: mbarrier phases, 1-D bulk
// copies (TMA engine, no tensor map, no multicast) between global and shared
// memory, and the shared-memory lookup table of NVFP4 block-scale divisors.
//
// Every wait is bounded: after kSpinLimit failed polls the waiter raises a
// device-global fault flag and leaves its loop, so a kernel can never hang on
// a barrier nobody completes.
#pragma once

#include "common.cuh"

namespace axb {

#ifdef __CUDACC__

constexpr uint32_t kSpinLimit = 1u << 18;

// Set by any kernel of the including translation unit whose bounded wait ran out
// (one word per unit: device variables have internal linkage without -rdc).
static __device__ unsigned int g_pipeline_fault;

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes barrier initialisation visible to the async proxy before any bulk copy names the barrier.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
    return done != 0u;
}

// Bounded wait; false (and the fault flag raised) when the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicOr(&g_pipeline_fault, 1u);
    return false;
}

// global -> shared, completion counted in bytes on `bar`.  Both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void *dst_shared, const void *src_global, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst_shared)), "l"(src_global), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// shared -> global, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_store(void *dst_global, const void *src_shared, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst_global), "r"(smem_addr(src_shared)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once every committed bulk store of this thread has finished READING shared memory.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Orders this thread's earlier generic-proxy shared-memory writes before later async-proxy accesses.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------
// NVFP4 block-scale table: for every E4M3 code c (as produced by the saturating
// converter, before the zero fix-up) the divisor d = e4m3(fix(c)) / G and its
// correctly rounded reciprocal.  128 entries, built once per CTA, so the
// per-block work is one shared-memory load instead of a decode, a division
// and a reciprocal.
// ---------------------------------------------------------------------------
struct scale_lut_entry {
    float d;
    float r;
};

// Called by all threads of the CTA; returns (through __syncthreads_and) whether
// every divisor is inside the range where div_by_shared() is exact.
__device__ __forceinline__ bool build_scale_lut(scale_lut_entry *lut, float G) {
    bool safe = true;
    for (uint32_t c = threadIdx.x; c < 128u; c += blockDim.x) {
        uint32_t code = c;
        if (code == 0u) code = 0x20u;
        if (code == 0x7fu) code = 0x7eu;
        const float d = __fdiv_rn(e4m3_to_f32(code), G);
        lut[c].d = d;
        lut[c].r = __frcp_rn(d);
        safe = safe && d >= 1.0e-25f && d <= 1.0e30f;
    }
    return __syncthreads_and(safe) != 0;
}

// 8 values (half a block) -> 4 code bytes, straight-line code (no branch, so an
// unrolled caller can interleave several chunks).  max_abs is the block maximum;
// *scale_byte receives the E4M3 code to store for the block.  The quotients use
// div_by_shared(); when that is not exact for this block (divisor or quotient
// outside the safe range) *needs_exact is raised and the caller must redo the
// chunk with nvfp4_quantize8_exact() — this happens only for saturated block
// scales or extreme global scales.
__device__ __forceinline__ uint32_t nvfp4_quantize8_fast(const float (&x)[8], float max_abs, float G,
                                                         const scale_lut_entry *lut, uint32_t *scale_byte,
                                                         bool *needs_exact) {
    const uint32_t raw = cvt_e4m3x2(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G), 0.0f) & 0x7fu;
    *scale_byte = raw == 0u ? 0x20u : raw;  // 0x7f cannot occur: the maximum is never NaN
    const scale_lut_entry e = lut[raw];
    *needs_exact = *needs_exact || !(__fmul_rn(max_abs, e.r) <= 1.0e30f);
    const float2 r2 = make_float2(e.r, e.r);
    const float2 nd2 = make_float2(-e.d, -e.d);
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = make_float2(x[2 * i], x[2 * i + 1]);
        const float2 q0 = __fmul2_rn(v, r2);
        const float2 err = __ffma2_rn(nd2, q0, v);
        float2 q = __ffma2_rn(err, r2, q0);
        q.x = __uint_as_float((__float_as_uint(q.x) & 0x7fffffffu) | (__float_as_uint(v.x) & 0x80000000u));
        q.y = __uint_as_float((__float_as_uint(q.y) & 0x7fffffffu) | (__float_as_uint(v.y) & 0x80000000u));
        b[i] = cvt_e2m1x2(q.x, q.y);
    }
    return __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
}

// Same result through IEEE divisions; used on the rare chunks the fast path flags.
static __device__ __noinline__ uint32_t nvfp4_quantize8_exact(float x0, float x1, float x2, float x3, float x4,
                                                              float x5, float x6, float x7, float max_abs, float G) {
    const uint32_t code = encode_block_scale(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G));
    const float d = __fdiv_rn(e4m3_to_f32(code), G);
    const uint32_t b0 = cvt_e2m1x2(__fdiv_rn(x0, d), __fdiv_rn(x1, d)) & 0xffu;
    const uint32_t b1 = cvt_e2m1x2(__fdiv_rn(x2, d), __fdiv_rn(x3, d)) & 0xffu;
    const uint32_t b2 = cvt_e2m1x2(__fdiv_rn(x4, d), __fdiv_rn(x5, d)) & 0xffu;
    const uint32_t b3 = cvt_e2m1x2(__fdiv_rn(x6, d), __fdiv_rn(x7, d)) & 0xffu;
    return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

#endif  // __CUDACC__

#ifdef __CUDACC__
// Host: reads and clears this unit's fault word on the current device (synchronises).
static inline unsigned int read_and_clear_pipeline_fault() {
    unsigned int word = 0u, zero = 0u;
    if (cudaMemcpyFromSymbol(&word, g_pipeline_fault, sizeof(word)) != cudaSuccess) return ~0u;
    if (word) (void)cudaMemcpyToSymbol(g_pipeline_fault, &zero, sizeof(zero));
    return word;
}
#endif

}  // namespace axb

// Asynchronous row pipeline primitives for sm_100a: mbarrier phases, 1-D bulk
// copies (TMA engine, no tensor map, each copy serves one CTA) between global and shared
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

// Adds to the byte count the current phase waits for, without arriving (a later
// mbar_arrive_expect_tx completes the announcement).
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
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

// Bounded wait; false (and the fault flag raised) when the phase never completed within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
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

// Asks the memory system to bring `bytes` of global memory into L2 (no destination, no completion to wait for, no
// architectural effect).  Address and size are multiples of 16.  The register-pipelined kernels issue it for the
// data of their NEXT iteration while they convert the current one, so that DRAM stays busy during the arithmetic
// and the next loads find their lines in L2.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src_global, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_global), "r"(bytes) : "memory");
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
// Returns once all but the most recent committed bulk store of this thread have finished reading.
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// Orders this thread's earlier generic-proxy shared-memory writes before later async-proxy accesses.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------
// NVFP4 block-scale table: for every E4M3 code c (as produced by the saturating
// converter, before the zero fix-up) the divisor d = e4m3(fix(c)) / G and its
// correctly rounded reciprocal.  128 entries, built once per CTA, so the
// per-block work is one shared-memory load instead of a decode, a division
// and a reciprocal.
// ---------------------------------------------------------------------------
struct __align__(8) scale_lut_entry {
    float nr;  // -1/d: correctly rounded reciprocal, negated for the quotient sequence
    float d;
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
        const float r = __frcp_rn(d);
        lut[c].d = d;
        lut[c].nr = -r;
        safe = safe && d >= 1.0e-25f && d <= 1.0e30f;
    }
    return __syncthreads_and(safe) != 0;
}

// max(|a|, |b|) that PROPAGATES NaN (fmaxf drops it).  The straight-line quantizer
// uses it so that a block holding a NaN is recognised (its maximum is NaN) and
// handed to the exact path, which applies the reference's fmaxf semantics.
__device__ __forceinline__ float absmax_nan(float a, float b) {
    float d;
    asm("{\n\t.reg .f32 x, y;\n\tabs.f32 x, %1;\n\tabs.f32 y, %2;\n\tmax.NaN.f32 %0, x, y;\n\t}" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float max_nan(float a, float b) {
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ float absmax8_nan(const float (&x)[8]) {
    return max_nan(max_nan(absmax_nan(x[0], x[1]), absmax_nan(x[2], x[3])),
                   max_nan(absmax_nan(x[4], x[5]), absmax_nan(x[6], x[7])));
}

// 8 values (half a block) -> 4 code bytes, straight-line code (no branch, so an
// unrolled caller can interleave several chunks).  max_abs is the block maximum
// from absmax8_nan() (+ the partner lane); *scale_byte receives the E4M3 code to
// store for the block.  Quotients: with nr = -1/d (correctly rounded),
//   t = RN(x * nr);  e = fma(d, t, x) = x - d*q0 exactly;  nq = fma(e, nr, t) = -RN(x/d)
// — the residual-corrected quotient, negated so that signed zeros survive (a
// positive-form last step would turn -0 into +0); the eight sign bits are flipped
// back on the packed nibbles with one XOR.  When the sequence is not exact for
// this block (divisor or quotient outside the safe range, NaN or infinity in the
// block) *needs_exact is raised and the caller must redo the chunk with
// nvfp4_quantize8_exact(): saturated block scales or extreme global scales only.
__device__ __forceinline__ uint32_t nvfp4_quantize8_fast(const float (&x)[8], float max_abs, float G,
                                                         const scale_lut_entry *lut, uint32_t *scale_byte,
                                                         bool *needs_exact) {
    const uint32_t raw = cvt_e4m3x2(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G), 0.0f) & 0x7fu;
    *scale_byte = raw == 0u ? 0x20u : raw;
    const float2 e = *reinterpret_cast<const float2 *>(lut + raw);
    *needs_exact = *needs_exact || !(__fmul_rn(max_abs, e.x) >= -1.0e30f);  // also true for a NaN maximum
    const float2 nr2 = make_float2(e.x, e.x);
    const float2 d2 = make_float2(e.y, e.y);
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = make_float2(x[2 * i], x[2 * i + 1]);
        const float2 t = __fmul2_rn(v, nr2);
        const float2 err = __ffma2_rn(d2, t, v);
        const float2 nq = __ffma2_rn(err, nr2, t);
        b[i] = cvt_e2m1x2(nq.x, nq.y);
    }
    return __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410) ^ 0x88888888u;
}

// A whole 16-value block held by ONE lane -> 8 code bytes: the block maximum needs no lane exchange and the scale
// byte, table entry and range test are evaluated once per block instead of once per half.  Same quotient sequence
// as nvfp4_quantize8_fast.
__device__ __forceinline__ float absmax16_nan(const float (&x)[16]) {
    const float a = max_nan(max_nan(absmax_nan(x[0], x[1]), absmax_nan(x[2], x[3])), max_nan(absmax_nan(x[4], x[5]), absmax_nan(x[6], x[7])));
    const float b = max_nan(max_nan(absmax_nan(x[8], x[9]), absmax_nan(x[10], x[11])), max_nan(absmax_nan(x[12], x[13]), absmax_nan(x[14], x[15])));
    return max_nan(a, b);
}

__device__ __forceinline__ uint2 nvfp4_quantize16_fast(const float (&x)[16], float G, const scale_lut_entry *lut,
                                                       uint32_t *scale_byte, bool *needs_exact) {
    const float max_abs = absmax16_nan(x);
    const uint32_t raw = cvt_e4m3x2(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G), 0.0f) & 0x7fu;
    *scale_byte = raw == 0u ? 0x20u : raw;
    const float2 e = *reinterpret_cast<const float2 *>(lut + raw);
    *needs_exact = *needs_exact || !(__fmul_rn(max_abs, e.x) >= -1.0e30f);  // also true for a NaN maximum
    const float2 nr2 = make_float2(e.x, e.x);
    const float2 d2 = make_float2(e.y, e.y);
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = make_float2(x[2 * i], x[2 * i + 1]);
        const float2 t = __fmul2_rn(v, nr2);
        const float2 err = __ffma2_rn(d2, t, v);
        const float2 nq = __ffma2_rn(err, nr2, t);
        b[i] = cvt_e2m1x2(nq.x, nq.y);
    }
    return make_uint2(__byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410) ^ 0x88888888u,
                      __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410) ^ 0x88888888u);
}

// Same result through IEEE divisions; max_abs must come from fmaxf (NaN-dropping) reductions.
static __device__ __noinline__ uint32_t nvfp4_quantize8_exact(float x0, float x1, float x2, float x3, float x4,
                                                              float x5, float x6, float x7, float max_abs, float G,
                                                              uint32_t *scale_byte) {
    const uint32_t code = encode_block_scale(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G));
    *scale_byte = code;
    const float d = __fdiv_rn(e4m3_to_f32(code), G);
    const uint32_t b0 = cvt_e2m1x2(__fdiv_rn(x0, d), __fdiv_rn(x1, d)) & 0xffu;
    const uint32_t b1 = cvt_e2m1x2(__fdiv_rn(x2, d), __fdiv_rn(x3, d)) & 0xffu;
    const uint32_t b2 = cvt_e2m1x2(__fdiv_rn(x4, d), __fdiv_rn(x5, d)) & 0xffu;
    const uint32_t b3 = cvt_e2m1x2(__fdiv_rn(x6, d), __fdiv_rn(x7, d)) & 0xffu;
    return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

__device__ __forceinline__ float absmax8_drop_nan(const float (&x)[8]) {
    return fmaxf(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))),
                 fmaxf(fmaxf(fabsf(x[4]), fabsf(x[5])), fmaxf(fabsf(x[6]), fabsf(x[7]))));
}

// bf16x2 + bf16x2, correctly rounded.  Equal to bf16(f32(a) + f32(b)) for every pair of finite
// inputs: when the exponents are close the F32 sum is exact, when they are far apart the
// smaller addend is below a quarter of a BF16 ulp of the larger, so no double rounding exists.
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
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

// Shared device numerics and host launch helpers for libaxiom_b200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "axiom_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "libaxiom_b200 kernels are written for sm_100a"
#endif

namespace axb {

constexpr uint32_t kSmCount = 148u;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this
constexpr uint32_t kGroup = 16u;     // NVFP4 block size

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

// Every kernel launch of the library goes through this counter so the
// benchmark can report how many of the library's kernels ran.
void note_launch(uint32_t n = 1u);

// cudaSetDevice + map failure to the ABI status.
int select_device(int device);

// cudaGetLastError() only: the family convention for stream-explicit entries.
int launch_status();

// Generic convention: return right after the launch when AXIOM_CUDA_LAUNCH_ASYNC
// is truthy or the stream is capturing, otherwise synchronise the stream.
int finish_after_launch(cudaStream_t stream);

inline bool valid_scale(float v) { return std::isfinite(v) && v > 0.0f; }

inline int cuda_to_status(cudaError_t err) {
    if (err == cudaSuccess) return AXIOM_OK;
    return err == cudaErrorMemoryAllocation ? AXIOM_ERR_BUDGET : AXIOM_ERR_CUDA;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; }

// Opaque handle layouts (private to the library).
struct runtime_impl;
struct buffer_impl;

// ---------------------------------------------------------------------------
// device side
// ---------------------------------------------------------------------------

#ifdef __CUDACC__

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of the fused chain is launched with programmatic stream serialisation allowed:
// the next kernel on the stream may be scheduled while this one still runs, executes whatever
// does not depend on earlier work (shared-memory set-up, tables computed from scalar arguments)
// and then blocks in dependency_wait() until all earlier kernels have completed and their
// writes are visible.  At decode shapes, where a layer is a chain of few-microsecond kernels,
// this takes the launch latency of each kernel off the critical path; it also works inside
// CUDA graph capture (the edges become programmatic).  Rules the kernels follow:
//   * dependency_wait() comes before the first access to any caller-visible global memory
//     (reads AND writes) and is executed on every path, so completion of kernel N implies
//     completion of every kernel before it;
//   * allow_dependents() is called at the top: the hardware starts the dependents only once
//     every CTA of this grid has started or finished, so they never take resources this grid
//     still needs.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Raises the dynamic shared-memory limit of one kernel, once per device (the attribute is per device; one
// process may drive several).  The kernel is a template argument so that every kernel has a flag of its own.
template <auto Kernel>
inline void allow_dynamic_smem(size_t bytes) {
    static bool done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        return;
    }
    if (!done[dev]) {
        cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        done[dev] = true;
    }
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
// The two BF16 halves of `packed` as floats through the mixed-precision FMA of sm_100 (x * 1 + (-0) = x for every
// x, signed zeros included): the widening runs on the FMA pipe and reads the halves in place, where the shift / mask
// pair above occupies the ALU pipe.  For kernels whose ALU pipe is the busy one.
// acc.x = fma(lo, lo, acc.x), acc.y = fma(hi, hi, acc.y) for the two BF16 halves of `packed`: the squares go into
// the F32 accumulators with one rounding each, exactly fmaf(x, x, acc) on the widened values, without widening them.
__device__ __forceinline__ float2 bf16x2_square_accumulate(uint32_t packed, float2 acc) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "fma.rn.f32.bf16 %0, l, l, %0;\n\t"
        "fma.rn.f32.bf16 %1, h, h, %1;\n\t}" : "+f"(acc.x), "+f"(acc.y) : "r"(packed));
    return acc;
}
__device__ __forceinline__ float2 bf16x2_widen_fma(uint32_t packed) {
    float2 v;
    asm("{\n\t.reg .b16 l, h, one;\n\tmov.b32 {l, h}, %2;\n\tmov.b16 one, 0x3f80;\n\t"
        "fma.rn.f32.bf16 %0, l, one, 0f80000000;\n\t"
        "fma.rn.f32.bf16 %1, h, one, 0f80000000;\n\t}" : "=f"(v.x), "=f"(v.y) : "r"(packed));
    return v;
}

// Two F32 -> packed BF16 pair, round-to-nearest-even (NaN stays NaN): `lo` lands in bits 0..15.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

// Two F32 -> two E4M3FN codes (RN-even, saturate to +-448, NaN -> 0x7f); `lo` in bits 0..7.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t out;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
    return out;
}

// Two F32 -> two E2M1 nibbles (RN-even, saturate to +-6, NaN -> +6); `lo` in bits 0..3.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t out;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
        : "=h"(out) : "f"(hi), "f"(lo));
    return out;
}

// E4M3FN code -> F32 (finite codes are exact in half precision).
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
    uint32_t halves;
    asm("{\n\t.reg .b16 c;\n\tcvt.u16.u32 c, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, c;\n\t}" : "=r"(halves) : "r"(code & 0xffu));
    float out;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.f32.f16 %0, lo;\n\t}" : "=f"(out) : "r"(halves));
    return out;
}

// Block-scale flavour of the E4M3 encoder: a zero magnitude becomes +0.125
// (0x20) and the NaN code becomes the largest finite code.
__device__ __forceinline__ uint32_t encode_block_scale(float value) {
    const uint32_t code = cvt_e4m3x2(value, 0.0f) & 0xffu;
    const uint32_t magnitude = code & 0x7fu;
    if (magnitude == 0u) return 0x20u;
    if (magnitude == 0x7fu) return (code & 0x80u) | 0x7eu;
    return code;
}

// Correctly rounded x / d for a divisor that is shared by many elements.
// `r` must be __frcp_rn(d).  One residual step from q0 = RN(x*r):
//   e = x - d*q0 (exact in an FMA), q = RN(q0 + e*r) = RN(x/d)
// as long as neither the quotient nor the residual leaves the normal range;
// callers test that once per divisor with divisor_is_safe() and take the
// IEEE division otherwise.  The sign of x is re-applied so -0 and values that
// round to zero keep it, as IEEE division by a positive divisor does.
__device__ __forceinline__ float div_by_shared(float x, float d, float r) {
    const float q0 = __fmul_rn(x, r);
    const float e = __fmaf_rn(-d, q0, x);
    const float q = __fmaf_rn(e, r, q0);
    return __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(x) & 0x80000000u));
}

// True when every |x| <= max_abs divides safely by d with div_by_shared():
// d far enough inside the normal range that the residual of any quotient near
// a rounding boundary of the target format (>= 2^-10) is exactly representable,
// and max_abs/d far from overflow.  r = __frcp_rn(d).
__device__ __forceinline__ bool divisor_is_safe(float d, float r, float max_abs) {
    return d >= 1.0e-25f && d <= 1.0e30f && __fmul_rn(max_abs, r) <= 1.0e30f;
}

__device__ __forceinline__ float div_exact_or_shared(float x, float d, float r, bool safe) {
    return safe ? div_by_shared(x, d, r) : __fdiv_rn(x, d);
}

// Offset of one block scale in the output plane.
__device__ __forceinline__ uint64_t scale_offset(uint32_t row, uint32_t group, uint32_t groups,
                                                 uint32_t inner_tiles, uint32_t layout) {
    if (layout == AXIOM_SCALE_LAYOUT_CANONICAL) return (uint64_t)row * groups + group;
    const uint32_t in_tile = row & 127u;
    return ((uint64_t)(row >> 7) * inner_tiles + (group >> 2)) * 512u + (in_tile & 31u) * 16u +
           (in_tile >> 5) * 4u + (group & 3u);
}

// 128-bit global accesses.  Activations are streamed once: bypass L1 allocation
// on loads and mark stores as streaming so they do not displace reusable lines.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(void *p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream(void *p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream(void *p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// Quantize 8 values (one half of a 16-value block) to 4 packed E2M1 bytes.
// max_abs is the maximum over the WHOLE block; G the global multiplier.
// Returns the packed codes; *scale_code receives the E4M3 block scale.
__device__ __forceinline__ uint32_t nvfp4_quantize8(const float (&x)[8], float max_abs, float G,
                                                    uint32_t *scale_code) {
    // (max * (1/6)) * G, two roundings in this order
    const uint32_t code = encode_block_scale(__fmul_rn(__fmul_rn(max_abs, 1.0f / 6.0f), G));
    const float d = __fdiv_rn(e4m3_to_f32(code), G);
    *scale_code = code;
    const float r = __frcp_rn(d);
    const bool safe = divisor_is_safe(d, r, max_abs);
    uint32_t packed = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = div_exact_or_shared(x[2 * i], d, r, safe);
        const float hi = div_exact_or_shared(x[2 * i + 1], d, r, safe);
        packed |= (cvt_e2m1x2(lo, hi) & 0xffu) << (8 * i);
    }
    return packed;
}

#endif  // __CUDACC__

}  // namespace axb

// SwiGLU fused with the activation quantizer that feeds the down projection,
// and the plain BF16 per-token FP8 quantizer.
//
//   y = (g / (1 + expf(-g))) * u      FP32, true division, precise expf, never rounded
//       silu_mul_batch_kernel (src/axiom_qwen38_fp8_mlp.cu:16-21)
//   FP8:   scale = rowmax|y| / 448 (1 when 0 or not finite), code = e4m3(y / scale)
//       quantize_columns_e4m3_kernel (src/axiom_qwen38_fp8.cu:64-94)
//   NVFP4: per-16 block scale, silu_mul_quantize_batch_to_tc_kernel
//       (src/axiom_qwen38_nvfp4_mlp.cu:229-317)
//
// The FP8 flavour needs the whole row before it can scale it: one CTA owns one
// row at a time, every thread keeps its share of y in registers across the
// row-max reduction, so gate|up is read once and only the codes are written.
//
// silu(g) = g / (1 + expf(-g)) depends on the BF16 gate alone, so it is tabulated
// — 64 binades x 128 mantissas x 2 signs, filled by the very expression the direct
// path evaluates, hence bit-identical — and the hot loop replaces expf + an IEEE
// division per element by one shared-memory load.  Gates outside the table
// (|g| < 2^-57, |g| >= 128, NaN, infinity) take the direct expression.  The table
// does not depend on any input: it is filled once per device into a 64 KB device
// array and every CTA copies it into shared memory (16-byte loads, L2 hits); a
// call that arrives during stream capture before that one-time fill lets each CTA
// fill its own copy instead.
#include <math_constants.h>

#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {

// kFma: widen on the FMA pipe (mixed-precision FMA) instead of the ALU pipe (shift / mask).  Which one is faster
// is a matter of each kernel's instruction mix and schedule; the call sites carry the measured choice.
template <bool kFma = false>
__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    if (kFma) {
        const float2 a = bf16x2_widen_fma(v.x), b = bf16x2_widen_fma(v.y), c = bf16x2_widen_fma(v.z), d = bf16x2_widen_fma(v.w);
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
    } else {
        x[0] = bf16_lo(v.x); x[1] = bf16_hi(v.x);
        x[2] = bf16_lo(v.y); x[3] = bf16_hi(v.y);
        x[4] = bf16_lo(v.z); x[5] = bf16_hi(v.z);
        x[6] = bf16_lo(v.w); x[7] = bf16_hi(v.w);
    }
}

__device__ __forceinline__ float silu(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))); }
// 1.0f / (1.0f + expf(-g)): the output gate of the attention block
// (qwen38_sigmoid_gate_kernel, src/axiom_qwen38_attention.cu:470-479)
__device__ __forceinline__ float sigmoid(float g) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g))); }

// The function of the BF16 gate that a table holds.
enum class gate_fn { silu, sigmoid };
template <gate_fn kFn>
__device__ __forceinline__ float gate_value(float g) { return kFn == gate_fn::silu ? silu(g) : sigmoid(g); }

// f(gate) * other for one pair of BF16 patterns, out of line: the rare path of the table kernels calls it per
// element, so that its expf and division do not take registers from the straight-line code around the call.
template <gate_fn kFn>
static __device__ __noinline__ float gated_product_slow(uint32_t gate_bits, uint32_t other_bits) {
    return __fmul_rn(gate_value<kFn>(__uint_as_float(gate_bits << 16)), __uint_as_float(other_bits << 16));
}

// ---- shared-memory silu table -------------------------------------------------------------
// 64 binades (2^-57 .. 2^7) x 128 mantissas x 2 signs = 16384 floats.  Byte offset of a BF16
// pattern b: (((b & 0x7fff) - first) & 0x1fff) * 4 + (b & 0x8000) — every offset is inside the
// table, patterns outside the tabulated range alias into it and are caught by the range test.
constexpr uint32_t kSiluExpLo = 70u;                                  // 2^-57
constexpr uint32_t kSiluFirst = kSiluExpLo << 7;                      // first tabulated magnitude
constexpr uint32_t kSiluEnd = (kSiluExpLo + 64u) << 7;                // one past the last
constexpr uint32_t kSiluTableBytes = 2u * 8192u * sizeof(float);

constexpr uint32_t kSiluEntries = 16384u;

template <gate_fn kFn>
__device__ __forceinline__ float gate_table_entry(uint32_t i) {
    const uint32_t bits = ((i >> 13) << 15) | (kSiluFirst + (i & 8191u));
    return gate_value<kFn>(__uint_as_float(bits << 16));
}

// The per-device copies of the tables (each filled once by gate_table_fill_kernel).
static __device__ __align__(256) float g_silu_table[kSiluEntries];
static __device__ __align__(256) float g_sigmoid_table[kSiluEntries];

template <gate_fn kFn>
__global__ void gate_table_fill_kernel(float *table) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kSiluEntries) table[i] = gate_table_entry<kFn>(i);
}

// Shared-memory table of a CTA: copied from the device table, or computed here when there is none yet.
template <gate_fn kFn = gate_fn::silu>
__device__ __forceinline__ void build_silu_table(float *table, const float *device_table) {
    if (device_table) {
        const uint4 *src = reinterpret_cast<const uint4 *>(device_table);
        uint4 *dst = reinterpret_cast<uint4 *>(table);
        for (uint32_t i = threadIdx.x; i < kSiluEntries / 4u; i += blockDim.x) dst[i] = __ldg(src + i);
    } else {
        for (uint32_t i = threadIdx.x; i < kSiluEntries; i += blockDim.x) table[i] = gate_table_entry<kFn>(i);
    }
    __syncthreads();
}

// Table lookups for the two BF16 gates packed in w, with everything that can be done on both
// halves at once done on the packed word.  below = magnitude + (0x8000 - first) per half (no half
// can carry into its neighbour: magnitudes are at most 0x7fff).  For a magnitude inside the
// table, below = 0x8000 + index with index < 0x2000; above the table the index reaches bit 13
// or 14, and under it below falls into [0x8000 - first, 0x8000), whose bit 14 is set because
// first < 0x4000 — so "bit 13 or 14 of a half of below" is exactly "this gate is outside the
// table" (|g| < 2^-57, |g| >= 128, NaN, infinity), and `outside` just ORs the words together.
// The low 13 bits of a `below` half are the entry's index inside its sign plane; z puts the sign
// next to them (bit 13), and the last shifts and masks turn each half of z into a byte offset,
// dropping the stray bits the 3-input select lets through.
static_assert(kSiluFirst < 0x4000u && kSiluEnd == kSiluFirst + 0x2000u, "range test relies on the table window");

__device__ __forceinline__ float2 silu_lookup2(const float *table, uint32_t w, uint32_t *outside) {
    const char *base = reinterpret_cast<const char *>(table);
    const uint32_t below = (w & 0x7fff7fffu) + (0x8000u - kSiluFirst) * 0x00010001u;
    *outside |= below;
    uint32_t z;
    asm("lop3.b32 %0, %1, %2, 0x1fff1fff, 0xe4;" : "=r"(z) : "r"(below), "r"(w >> 2));  // (below & c) | ((w>>2) & ~c)
    const uint32_t olo = (z << 2) & 0xfffcu;
    const uint32_t ohi = (z >> 14) & 0xfffcu;
    return make_float2(*reinterpret_cast<const float *>(base + olo), *reinterpret_cast<const float *>(base + ohi));
}

// y[0..7] = f(gate) * other for one 16-byte chunk of each; f = silu (SwiGLU) or sigmoid (output gate)
// kRareOutOfLine: the rare path calls gated_product_slow per element instead of evaluating in line.  Measured per
// kernel: the NVFP4 kernels gain (sigmoid gate 71.4 -> 68.5 us, SwiGLU 247.5 -> 242.0 us), the FP8 kernel loses 2 %.
template <bool kTable, gate_fn kFn = gate_fn::silu, bool kFmaUnpack = false, bool kRareOutOfLine = false>
__device__ __forceinline__ void swiglu8(const float *table, const uint4 &g, const uint4 &u, float (&y)[8]) {
    if (kTable) {
        uint32_t outside = 0u;
        const float2 p0 = __fmul2_rn(silu_lookup2(table, g.x, &outside), bf16x2_widen_fma(u.x));
        const float2 p1 = __fmul2_rn(silu_lookup2(table, g.y, &outside), bf16x2_widen_fma(u.y));
        const float2 p2 = __fmul2_rn(silu_lookup2(table, g.z, &outside), bf16x2_widen_fma(u.z));
        const float2 p3 = __fmul2_rn(silu_lookup2(table, g.w, &outside), bf16x2_widen_fma(u.w));
        y[0] = p0.x; y[1] = p0.y; y[2] = p1.x; y[3] = p1.y; y[4] = p2.x; y[5] = p2.y; y[6] = p3.x; y[7] = p3.y;
        if (outside & 0x60006000u) {
            // rare: a gate beyond the table in this chunk
            if (kRareOutOfLine) {
                const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    y[2 * i] = gated_product_slow<kFn>(gw[i] & 0xffffu, uw[i] & 0xffffu);
                    y[2 * i + 1] = gated_product_slow<kFn>(gw[i] >> 16, uw[i] >> 16);
                }
            } else {
                float gv[8], uv[8];
                unpack8<kFmaUnpack>(g, gv);
                unpack8<kFmaUnpack>(u, uv);
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(gate_value<kFn>(gv[i]), uv[i]);
            }
        }
    } else {
        float gv[8], uv[8];
        unpack8<kFmaUnpack>(g, gv);
        unpack8<kFmaUnpack>(u, uv);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(gate_value<kFn>(gv[i]), uv[i]);
    }
}

// Maximum over the CTA; every thread receives it.  The operands are magnitudes: non-negative floats, +infinity, or
// the canonical NaN that max.NaN.f32 produces (0x7fffffff).  On those the unsigned order of the bit patterns is
// the order of the values with NaN on top, so the maximum of a warp is one redux.sync instead of five shuffles and
// five maxima — NaN-propagating where a NaN can occur (the callers that must drop NaN pass none).
// `warp_max` (32 words) is read by everybody after the one barrier.  A caller that runs row after row gives every row
// the next of four buffers, two per row (the second for a recount): a buffer comes round again two rows later, and
// by then every thread has passed the following row's barrier, which it reaches only after its reads of this one.
__device__ __forceinline__ float cta_max(float m, uint32_t *warp_max) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = (blockDim.x + 31u) >> 5;
    const uint32_t mine = __reduce_max_sync(0xffffffffu, __float_as_uint(m));
    if (lane == 0u) warp_max[warp] = mine;
    __syncthreads();
    const uint32_t all = __reduce_max_sync(0xffffffffu, lane < warps ? warp_max[lane] : 0u);
    return __uint_as_float(all);  // no second barrier: the callers rotate their staging buffers
}

// Two FP8 codes through IEEE divisions, out of line: the rare path of the row kernel (a scale the reciprocal
// sequence is not exact for) calls it, so that the divisions' slow paths take no registers from the common path.
static __device__ __noinline__ uint32_t e4m3_pair_by_division(float a, float b, float scale) {
    return cvt_e4m3x2(__fdiv_rn(a, scale), __fdiv_rn(b, scale));
}

enum class row_op { swiglu, swiglu_table };

// CPT = 16-byte chunks (8 values) per thread; blockDim.x * CPT >= width / 8.
constexpr uint32_t kMaxRowThreads = 576u;
constexpr int kMlpRowThreads = 544;  // 17408 / (4 chunks x 8 values)

// kStatic: the scale is an argument (quantize_columns_static_e4m3_kernel, src/axiom_qwen38_fp8.cu:96-107) — no row
// maximum, no CTA reduction, no scale output; every thread decides for its own values whether the reciprocal
// sequence is exact and takes IEEE divisions otherwise (NaN / infinity / quotients near overflow).
// kThreads != 0: the CTA has exactly kThreads threads and the row exactly kThreads * CPT chunks — no thread is past
// the end of the row and every offset inside a row is a compile-time constant (no predicates, no zero fill, no
// per-chunk address arithmetic).
template <int CPT, row_op kOp, bool kStatic = false, int kThreads = 0>
__global__ void __launch_bounds__(kThreads ? kThreads : kMaxRowThreads, CPT <= 4 ? 2 : 1)
fp8_rows_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, uint32_t in_chunks_per_row,
                uint2 *__restrict__ codes, float *__restrict__ scales, const float *__restrict__ device_table,
                float given_scale) {
    extern __shared__ __align__(16) float silu_table[];
    __shared__ uint32_t warp_max_buffers[4][32];
    uint32_t max_round = 0u;
    constexpr bool kTable = kOp == row_op::swiglu_table;
    const uint32_t tid = threadIdx.x;
    const uint32_t threads = kThreads ? (uint32_t)kThreads : blockDim.x;
    if (kThreads) chunks = (uint32_t)kThreads * CPT;
    allow_dependents();
    if (kTable) build_silu_table(silu_table, device_table);  // the device table never changes once filled
    dependency_wait();
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *gate = in + (uint64_t)row * in_chunks_per_row;
        // the row this CTA takes next, hinted into L2 while this one is converted: a CTA holds a whole row in
        // registers between its loads and its stores (the plain BF16 -> FP8 kernel gained 10 % from the same hint;
        // this one is bound by its instruction count and did not move either way)
        if (tid == 0u && row + gridDim.x < rows) {
            bulk_prefetch_l2(in + (uint64_t)(row + gridDim.x) * in_chunks_per_row, 2u * chunks * 16u);
        }
        float y[CPT][8];
        float m = 0.0f;  // NaN-propagating maximum
        bool nonfinite = false;
        {
            const uint4 *up = gate + chunks;
            uint4 g[CPT], u[CPT];
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + threads * k;
                const bool ok = kThreads != 0 || q < chunks;
                g[k] = ok ? ld_stream(gate + q) : make_uint4(0u, 0u, 0u, 0u);
                u[k] = ok ? ld_stream(up + q) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                swiglu8<kTable>(silu_table, g[k], u[k], y[k]);
                m = max_nan(m, absmax8_nan(y[k]));
            }
        }
        uint32_t *warp_max = warp_max_buffers[max_round & 3u];
        max_round += 2u;
        if (!kStatic) m = cta_max(m, warp_max);
        if (!kStatic && !(m == m)) {
            // a NaN somewhere in the row: the reference's maximum drops it
            float d = 0.0f;
#pragma unroll
            for (int k = 0; k < CPT; ++k) d = fmaxf(d, absmax8_drop_nan(y[k]));
            m = cta_max(d, warp_max + 32);
            nonfinite = true;
        }
        float scale = m == 0.0f ? 1.0f : __fdiv_rn(m, 448.0f);
        if (kStatic) {
            scale = given_scale;
            if (!(m == m)) m = CUDART_INF_F;  // fails the range test below
        } else if (!isfinite(scale) || scale <= 0.0f) {
            scale = 1.0f;
        }
        if (!kStatic && tid == 0u) scales[row] = scale;
        const float r = __frcp_rn(scale);
        // uniform over the CTA for the per-row scale, per thread (its own maximum) for a given scale
        const bool safe = divisor_is_safe(scale, r, m) && (kStatic || !nonfinite);
        uint2 *out = codes + (uint64_t)row * chunks;
        if (safe) {
            // negated residual-corrected quotients (signed zeros survive), signs flipped back on the codes
            const float2 nr2 = make_float2(-r, -r), d2 = make_float2(scale, scale);
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + threads * k;
                uint32_t c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 v = make_float2(y[k][2 * i], y[k][2 * i + 1]);
                    const float2 t = __fmul2_rn(v, nr2);
                    const float2 nq = __ffma2_rn(__ffma2_rn(d2, t, v), nr2, t);
                    c[i] = cvt_e4m3x2(nq.x, nq.y);
                }
                if (kThreads != 0 || q < chunks) {
                    st_stream(out + q, make_uint2(__byte_perm(c[0], c[1], 0x5410) ^ 0x80808080u,
                                                  __byte_perm(c[2], c[3], 0x5410) ^ 0x80808080u));
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + threads * k;
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    w[h] = e4m3_pair_by_division(y[k][4 * h + 0], y[k][4 * h + 1], scale) |
                           (e4m3_pair_by_division(y[k][4 * h + 2], y[k][4 * h + 3], scale) << 16);
                }
                if (kThreads != 0 || q < chunks) st_stream(out + q, make_uint2(w[0], w[1]));
            }
        }
    }
}

// ---- plain BF16 -> FP8 rows ------------------------------------------------------------------
// quantize_columns_e4m3 on BF16 storage: nothing has to be widened before the scale is known.  A thread keeps its
// chunks as the packed words it loaded (4 registers per chunk instead of 8 floats) and takes the row maximum on the
// BF16 magnitudes themselves — the unsigned order of |x| patterns is the order of the values, with infinity and NaN
// (>= 0x7f80) on top — two packed instructions per word.  A row whose maximum pattern is non-finite is redone with
// those values left out (the reference's maximum skips them and raises the status word).  The widening then
// happens once, on the FMA pipe, right before the division.
__device__ __forceinline__ uint32_t magnitude_max4(uint32_t m, const uint4 &w) {
    m = __vmaxu2(m, w.x & 0x7fff7fffu);
    m = __vmaxu2(m, w.y & 0x7fff7fffu);
    m = __vmaxu2(m, w.z & 0x7fff7fffu);
    return __vmaxu2(m, w.w & 0x7fff7fffu);
}
static __device__ __noinline__ uint32_t finite_magnitude_max4(uint32_t m, uint4 w) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = words[i] & 0x7fffu, hi = (words[i] >> 16) & 0x7fffu;
        if (lo < 0x7f80u && lo > m) m = lo;
        if (hi < 0x7f80u && hi > m) m = hi;
    }
    return m;
}
// eight codes of one chunk by IEEE divisions, out of line
static __device__ __noinline__ uint2 e4m3x8_of_bf16_by_division(uint4 w, float scale) {
    float v[8];
    unpack8(w, v);
    return make_uint2(e4m3_pair_by_division(v[0], v[1], scale) | (e4m3_pair_by_division(v[2], v[3], scale) << 16),
                      e4m3_pair_by_division(v[4], v[5], scale) | (e4m3_pair_by_division(v[6], v[7], scale) << 16));
}

template <int CPT, bool kStatic>
__global__ void __launch_bounds__(kMaxRowThreads)
fp8_plain_rows_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, uint32_t in_chunks_per_row,
                      uint2 *__restrict__ codes, float *__restrict__ scales, uint32_t *__restrict__ status_word,
                      float given_scale) {
    __shared__ uint32_t warp_max_buffers[4][32];
    uint32_t max_round = 0u;
    const uint32_t tid = threadIdx.x, threads = blockDim.x;
    allow_dependents();
    dependency_wait();
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *src = in + (uint64_t)row * in_chunks_per_row;
        // the row this CTA takes next, hinted into L2 while this one is converted
        if (tid == 0u && row + gridDim.x < rows) bulk_prefetch_l2(in + (uint64_t)(row + gridDim.x) * in_chunks_per_row, chunks * 16u);
        uint4 w[CPT];
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const uint32_t q = tid + threads * k;
            w[k] = q < chunks ? ld_stream(src + q) : make_uint4(0u, 0u, 0u, 0u);
        }
        uint32_t packed = 0u;
#pragma unroll
        for (int k = 0; k < CPT; ++k) packed = magnitude_max4(packed, w[k]);
        uint32_t top = max(packed & 0xffffu, packed >> 16);  // BF16 pattern of the largest magnitude, non-finite included
        uint32_t *warp_max = warp_max_buffers[max_round & 3u];
        max_round += 2u;
        if (!kStatic) top = __float_as_uint(cta_max(__uint_as_float(top), warp_max));
        bool nonfinite = top >= 0x7f80u;
        if (!kStatic && nonfinite) {
            uint32_t mine = 0u;
#pragma unroll
            for (int k = 0; k < CPT; ++k) mine = finite_magnitude_max4(mine, w[k]);
            top = __float_as_uint(cta_max(__uint_as_float(mine), warp_max + 32));
            if (tid == 0u && status_word) atomicCAS(status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_NONFINITE);
        }
        // kStatic: this thread's own maximum, for the range test only (non-finite: +infinity fails it)
        const float m = __uint_as_float(top << 16);
        float scale = kStatic ? given_scale : (m == 0.0f ? 1.0f : __fdiv_rn(m, 448.0f));
        if (!kStatic && tid == 0u) scales[row] = scale;
        const float r = __frcp_rn(scale);
        // uniform over the CTA for the per-row scale, per thread for a given scale
        const bool safe = divisor_is_safe(scale, r, m) && !nonfinite;
        uint2 *out = codes + (uint64_t)row * chunks;
        if (safe) {
            // negated residual-corrected quotients (signed zeros survive), signs flipped back on the codes
            const float2 nr2 = make_float2(-r, -r), d2 = make_float2(scale, scale);
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + threads * k;
                const uint32_t words[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
                uint32_t c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 v = bf16x2_widen_fma(words[i]);
                    const float2 t = __fmul2_rn(v, nr2);
                    const float2 nq = __ffma2_rn(__ffma2_rn(d2, t, v), nr2, t);
                    c[i] = cvt_e4m3x2(nq.x, nq.y);
                }
                if (q < chunks) {
                    st_stream(out + q, make_uint2(__byte_perm(c[0], c[1], 0x5410) ^ 0x80808080u,
                                                  __byte_perm(c[2], c[3], 0x5410) ^ 0x80808080u));
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + threads * k;
                if (q < chunks) st_stream(out + q, e4m3x8_of_bf16_by_division(w[k], scale));
            }
        }
    }
}

// SwiGLU -> NVFP4: no row-wide dependency; lanes own one chunk of gate and the
// matching chunk of up, lane pairs form a 16-value block.
constexpr uint32_t kNvThreads = 512u;
constexpr uint32_t kNvUnroll = 3u;  // warp tiles in flight per iteration (59 registers; four would pass 64 and halve the resident CTAs)

// A warp tile is 32 consecutive chunks of one row (column group `col` of `col_groups`); a warp
// takes tiles warp, warp + W, ... and advances (row, col) incrementally, so no division runs
// inside the loop.  step_rows = W / col_groups and step_cols = W % col_groups come from the host.
//
// kFn = silu: y = silu(gate) * up, never rounded, rows of `in` are [gate | up].
// kFn = sigmoid: y = bf16(attention * sigmoid(gate)) (qwen38_sigmoid_gate_kernel, src/axiom_qwen38_attention.cu:
// 470-479: the product is rounded to BF16 before anything consumes it), `in` holds the gates and `other` the
// attention output, both [rows x chunks]; y is optionally written out as BF16 as well.
template <bool kTable, gate_fn kFn, bool kHeadGate>
__global__ void __launch_bounds__(kNvThreads)
swiglu_nvfp4_kernel(const uint4 *__restrict__ in, const uint4 *__restrict__ other, uint32_t row_stride,
                    uint32_t other_row_stride, uint32_t in_head_keep, uint32_t in_head_add, uint32_t rows, uint32_t chunks, uint32_t col_groups,
                    uint32_t step_rows, uint32_t step_cols, float G, uint4 *__restrict__ out_bf16,
                    uint32_t *__restrict__ codes,
                    uint8_t *__restrict__ scales, uint32_t layout, uint32_t groups, uint32_t inner_tiles,
                    const float *__restrict__ device_table) {
    extern __shared__ __align__(16) float silu_table[];
    __shared__ scale_lut_entry lut[128];
    allow_dependents();
    if (kTable) build_silu_table<kFn>(silu_table, device_table);  // the device table never changes once filled
    const bool lut_safe = build_scale_lut(lut, G);
    dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kNvThreads + threadIdx.x) >> 5;
    const uint32_t lane_tile_off = (lane >> 3) * 512u + ((lane >> 1) & 3u);  // tiled plane: (group/4, group%4) of lane/2
    uint32_t row = warp / col_groups, col = warp % col_groups;
    while (row < rows) {
        uint32_t rws[kNvUnroll], qs[kNvUnroll];
        bool oks[kNvUnroll];
        uint4 g[kNvUnroll], u[kNvUnroll];
#pragma unroll
        for (uint32_t j = 0; j < kNvUnroll; ++j) {
            rws[j] = row;
            qs[j] = col * 32u + lane;
            oks[j] = row < rows && qs[j] < chunks;
            // kHeadGate: `in` has a row pitch of its own and holds, per head, the head's other values
            // first and then its gate values: chunk q of the row sits at q + (q rounded down to its
            // head) + one head.  Otherwise both planes share the pitch and the chunk index.
            const uint64_t other_at = (uint64_t)row * other_row_stride + qs[j];
            const uint64_t in_at = kHeadGate ? (uint64_t)row * row_stride + qs[j] + (qs[j] & in_head_keep) + in_head_add : other_at;
            // lanes beyond the row hold gate 1.0: a zero would leave the table and send the warp down the rare path
            g[j] = oks[j] ? ld_stream(in + in_at) : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
            u[j] = oks[j] ? ld_stream(other + other_at) : make_uint4(0u, 0u, 0u, 0u);
            row += step_rows;
            col += step_cols;
            if (col >= col_groups) {
                col -= col_groups;
                ++row;
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kNvUnroll; ++j) {
            if (rws[j] >= rows) continue;  // the whole tile lies beyond the last row (uniform over the warp)
            float y[8];
            swiglu8<kTable, kFn, kFn == gate_fn::silu, true>(silu_table, g[j], u[j], y);  // measured: 254.5 -> 249.7 us at 16384 x 17408
            if (kFn == gate_fn::sigmoid) {
                // the gated value exists in BF16 only: round, optionally store, and quantize the rounded values
                const uint4 r = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                           pack_bf16x2(y[6], y[7]));
                if (out_bf16 && oks[j]) st_stream(out_bf16 + (uint64_t)rws[j] * chunks + qs[j], r);
                unpack8(r, y);
            }
            float m = absmax8_nan(y);
            m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, 1));
            uint32_t scale_code;
            bool needs_exact = false;
            uint32_t packed = nvfp4_quantize8_fast(y, m, G, lut, &scale_code, &needs_exact);
            if (!lut_safe || __any_sync(0xffffffffu, needs_exact)) {
                m = absmax8_drop_nan(y);
                m = fmaxf(fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1)), 0.0f);
                packed = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], m, G, &scale_code);
            }
            if (oks[j] && codes) {
                st_stream(codes + (uint64_t)rws[j] * chunks + qs[j], packed);
                if ((lane & 1u) == 0u) {
                    // block (row, group): group = 16 * column group + lane / 2.  Canonical plane: row * groups + group.
                    // Tiled plane: ((row/128) * inner_tiles + group/4) * 512 + (row%32) * 16 + ((row%128)/32) * 4 + group%4,
                    // whose lane-dependent part is a per-thread constant and whose row part is uniform over the warp.
                    const uint32_t r = rws[j], cg = qs[j] >> 5;
                    const uint64_t off = layout == AXIOM_SCALE_LAYOUT_CANONICAL
                            ? (uint64_t)r * groups + (qs[j] >> 1)
                            : ((uint64_t)(r >> 7) * inner_tiles + 4u * cg) * 512u + (r & 31u) * 16u + ((r & 127u) >> 5) * 4u + lane_tile_off;
                    scales[off] = (uint8_t)scale_code;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Streaming flavour of the gated NVFP4 kernels for regular shapes (rows that are whole warp tiles, gate and
// other plane addressed by plain row pitches).  The general kernel above recomputes (row, column) bookkeeping,
// five 64-bit addresses and the scale-plane offset for every tile, which costs as many instructions as the
// arithmetic; here a warp owns a contiguous range of tiles, every address is a pointer that advances by a
// constant per tile (codes, BF16 output and the canonical scale plane are linear in the tile index; the two
// operand planes and the tiled scale plane are fixed up once per row), and kGatedUnroll tiles of one row are
// loaded before any is converted.
// ---------------------------------------------------------------------------
constexpr uint32_t kGatedUnroll = 3u;

// Table lookups and products of one chunk with no branch at all: `outside` collects the range bits of the eight
// gates (see silu_lookup2) for ONE test per loop iteration instead of one per chunk.
__device__ __forceinline__ void gated8_table(const float *table, const uint4 &g, const uint4 &u, float (&y)[8], uint32_t *outside) {
    const float2 p0 = __fmul2_rn(silu_lookup2(table, g.x, outside), bf16x2_widen_fma(u.x));
    const float2 p1 = __fmul2_rn(silu_lookup2(table, g.y, outside), bf16x2_widen_fma(u.y));
    const float2 p2 = __fmul2_rn(silu_lookup2(table, g.z, outside), bf16x2_widen_fma(u.z));
    const float2 p3 = __fmul2_rn(silu_lookup2(table, g.w, outside), bf16x2_widen_fma(u.w));
    y[0] = p0.x; y[1] = p0.y; y[2] = p1.x; y[3] = p1.y; y[4] = p2.x; y[5] = p2.y; y[6] = p3.x; y[7] = p3.y;
}

// One warp tile on the straight-line path: everything is stored, and `outside` / `needs_exact` tell the caller
// afterwards whether the tile has to be redone by gated_tiles_exact().
template <gate_fn kFn, bool kBf16Out, bool kCodes>
__device__ __forceinline__ void gated_tile_fast(const float *silu_table, const scale_lut_entry *lut, float G, const uint4 &g,
                                                const uint4 &u, uint4 *bf16_at, uint32_t *code_at, uint8_t *scale_at,
                                                bool scale_lane, uint32_t *outside, bool *needs_exact) {
    float y[8];
    gated8_table(silu_table, g, u, y, outside);
    if (kFn == gate_fn::sigmoid) {
        // the gated value exists in BF16 only: round, optionally store, and quantize the rounded values
        const uint4 r = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                   pack_bf16x2(y[6], y[7]));
        if (kBf16Out) st_stream(bf16_at, r);
        if (kCodes) unpack8<true>(r, y);
    }
    if (kCodes) {
        float m = absmax8_nan(y);
        m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, 1));
        uint32_t scale_code;
        const uint32_t packed = nvfp4_quantize8_fast(y, m, G, lut, &scale_code, needs_exact);
        st_stream(code_at, packed);
        if (scale_lane) *scale_at = (uint8_t)scale_code;
    }
}

// `n` consecutive tiles of one row again, by the direct expressions (expf, IEEE divisions, the reference's
// NaN-dropping maximum): the rare path — a gate outside the table, a block whose divisor leaves the range the
// reciprocal sequence is exact for, NaN or infinity.  Out of line and self-contained (it reloads its operands),
// so it costs the loop one warp-uniform branch per iteration and no registers.
template <gate_fn kFn>
static __device__ __noinline__ void gated_tiles_exact(const uint4 *pg, const uint4 *po, uint32_t n, float G, uint4 *pb,
                                                      uint32_t *pc, uint8_t *ps, uint32_t scale_step, bool scale_lane) {
    for (uint32_t j = 0; j < n; ++j) {
        const uint4 g = ld_stream(pg + 32u * j), u = ld_stream(po + 32u * j);
        float gv[8], uv[8], y[8];
        unpack8(g, gv);
        unpack8(u, uv);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(gate_value<kFn>(gv[i]), uv[i]);
        if (kFn == gate_fn::sigmoid) {
            const uint4 r = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                                       pack_bf16x2(y[6], y[7]));
            if (pb) st_stream(pb + 32u * j, r);
            unpack8(r, y);
        }
        if (pc) {
            float m = absmax8_drop_nan(y);
            m = fmaxf(fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1)), 0.0f);
            uint32_t scale_code;
            const uint32_t packed = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], m, G, &scale_code);
            st_stream(pc + 32u * j, packed);
            if (scale_lane) ps[(size_t)scale_step * j] = (uint8_t)scale_code;
        }
    }
}

// kBf16Out / kCodes: which outputs the call asked for (at least one).
template <gate_fn kFn, bool kTiled, bool kBf16Out, bool kCodes>
__global__ void __launch_bounds__(kNvThreads, 2)
gated_nvfp4_stream_kernel(const uint4 *__restrict__ gate, const uint4 *__restrict__ other, uint32_t gate_row_stride,
                          uint32_t other_row_stride, uint32_t total_tiles, uint32_t tiles_per_warp, uint32_t col_groups,
                          float G, uint4 *__restrict__ out_bf16, uint32_t *__restrict__ codes,
                          uint8_t *__restrict__ scales, uint32_t inner_tiles, const float *__restrict__ device_table) {
    extern __shared__ __align__(16) float silu_table[];
    __shared__ scale_lut_entry lut[128];
    allow_dependents();
    build_silu_table<kFn>(silu_table, device_table);  // the device table never changes once filled
    const bool lut_safe = build_scale_lut(lut, G);
    dependency_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kNvThreads + threadIdx.x) >> 5;
    const uint64_t first64 = (uint64_t)warp * tiles_per_warp;
    if (first64 >= total_tiles) return;
    const uint32_t first = (uint32_t)first64;
    uint32_t remaining = total_tiles - first < tiles_per_warp ? total_tiles - first : tiles_per_warp;
    uint32_t row = first / col_groups, col = first - row * col_groups;
    const bool scale_lane = (lane & 1u) == 0u;
    const uint32_t lane_tile_off = (lane >> 3) * 512u + ((lane >> 1) & 3u);  // tiled plane: (group / 4, group % 4) of lane / 2

    const uint4 *pg = gate + (uint64_t)row * gate_row_stride + col * 32u + lane;
    const uint4 *po = other + (uint64_t)row * other_row_stride + col * 32u + lane;
    const uint32_t gate_skip = gate_row_stride - col_groups * 32u, other_skip = other_row_stride - col_groups * 32u;
    uint4 *pb = kBf16Out ? out_bf16 + (uint64_t)first * 32u + lane : nullptr;
    uint32_t *pc = kCodes ? codes + (uint64_t)first * 32u + lane : nullptr;
    // scale of the block a lane pair holds: canonical plane = 16 blocks per tile, linear; tiled plane = 2048 bytes
    // per tile inside a row, row part recomputed at every row start
    auto tiled_row_base = [&](uint32_t r) {
        return scales + ((uint64_t)(r >> 7) * inner_tiles) * 512u + (r & 31u) * 16u + ((r & 127u) >> 5) * 4u + lane_tile_off;
    };
    uint8_t *ps = !kCodes ? nullptr : kTiled ? tiled_row_base(row) + (uint64_t)col * 2048u : scales + (uint64_t)first * 16u + (lane >> 1);
    constexpr uint32_t kScaleStep = kTiled ? 2048u : 16u;

    while (remaining != 0u) {
        const uint32_t in_row = col_groups - col;
        uint32_t n;
        uint32_t outside = 0u;
        bool needs_exact = false;
        if (remaining >= kGatedUnroll && in_row >= kGatedUnroll) {
            n = kGatedUnroll;
            uint4 g[kGatedUnroll], u[kGatedUnroll];
#pragma unroll
            for (uint32_t j = 0; j < kGatedUnroll; ++j) {
                g[j] = ld_stream(pg + 32u * j);
                u[j] = ld_stream(po + 32u * j);
            }
            // SwiGLU (gate and up halves of one row): the tiles of the next iteration, hinted into L2 while these are
            // converted (223 -> 217 us at 16384 x 17408; with two separate operand planes, the sigmoid gate, the same
            // hint costs 2 %, so it is not issued there)
            if (kFn == gate_fn::silu && lane < 2u && remaining >= 2u * kGatedUnroll && in_row >= 2u * kGatedUnroll) {
                bulk_prefetch_l2((lane == 0u ? pg : po) - lane + 32u * kGatedUnroll, kGatedUnroll * 512u);
            }
#pragma unroll
            for (uint32_t j = 0; j < kGatedUnroll; ++j) {
                gated_tile_fast<kFn, kBf16Out, kCodes>(silu_table, lut, G, g[j], u[j], pb + 32u * j, pc + 32u * j,
                                                       ps + kScaleStep * j, scale_lane, &outside, &needs_exact);
            }
        } else {
            n = 1u;
            const uint4 g = ld_stream(pg), u = ld_stream(po);
            gated_tile_fast<kFn, kBf16Out, kCodes>(silu_table, lut, G, g, u, pb, pc, ps, scale_lane, &outside, &needs_exact);
        }
        if (__any_sync(0xffffffffu, (outside & 0x60006000u) != 0u || needs_exact) || (kCodes && !lut_safe)) {
            gated_tiles_exact<kFn>(pg, po, n, G, pb, pc, ps, kScaleStep, scale_lane);
        }
        remaining -= n;
        pg += 32u * n; po += 32u * n;
        if (kBf16Out) pb += 32u * n;
        if (kCodes) {
            pc += 32u * n;
            ps += kScaleStep * n;
        }
        col += n;
        if (col == col_groups) {
            col = 0u;
            ++row;
            pg += gate_skip;
            po += other_skip;
            if (kCodes && kTiled) ps = tiled_row_base(row);
        }
    }
}

struct row_shape {
    uint32_t threads;
    uint32_t cpt;
};

// Smallest padding first; between equal paddings the larger CTA (shorter per-row latency), or — many_rows — the
// smaller one with more chunks per thread: more loads in flight per thread and more CTAs per SM, whose load and
// store phases then interleave (plain BF16 -> FP8 at 16384 x 8192: 91 us with 512 x 2, 79 with 256 x 4, 73 with
// 128 x 8).  Padding of up to 1/32 of the row is accepted for that.
row_shape pick_row_shape(uint32_t chunks, bool many_rows = false) {
    static const uint32_t cpts[] = {1u, 2u, 4u, 8u};
    row_shape best{0u, 0u};
    uint64_t best_pad = ~0ull;
    for (uint32_t cpt : cpts) {
        uint32_t threads = (chunks + cpt - 1u) / cpt;
        threads = (threads + 31u) & ~31u;
        if (threads < 64u) threads = 64u;
        if (threads > kMaxRowThreads) continue;
        uint64_t pad = (uint64_t)threads * cpt - chunks;
        if (many_rows && pad * 32u <= chunks) pad = 0u;  // at most 1/32 of the row
        if (pad < best_pad || (pad == best_pad && (many_rows ? threads < best.threads : threads > best.threads))) {
            best_pad = pad;
            best = row_shape{threads, cpt};
        }
    }
    return best;
}

// Device address of the per-device silu table, filling it on the first call for that device:
// one small kernel on `stream` and one synchronisation of that stream, so that calls on any
// other stream may use the table afterwards.  Returns nullptr (each CTA then fills its own
// shared-memory copy) when the table is not ready and cannot be made ready here: `stream` is
// being captured (a synchronisation would invalidate the capture), or the driver refused.
template <gate_fn kFn>
const float *device_gate_table(cudaStream_t stream) {
    static const float *ready[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (ready[dev]) return ready[dev];
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    float *table = nullptr;
    const cudaError_t found = kFn == gate_fn::silu ? cudaGetSymbolAddress((void **)&table, g_silu_table)
                                                   : cudaGetSymbolAddress((void **)&table, g_sigmoid_table);
    if (found != cudaSuccess || !table) {
        cudaGetLastError();
        return nullptr;
    }
    gate_table_fill_kernel<kFn><<<kSiluEntries / 256u, 256, 0, stream>>>(table);
    if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    note_launch();
    ready[dev] = table;
    return table;
}

const float *device_silu_table(cudaStream_t stream) { return device_gate_table<gate_fn::silu>(stream); }

template <row_op kOp, bool kStatic>
void configure_fp8_rows() {
    allow_dynamic_smem<fp8_rows_kernel<1, kOp, kStatic>>(kSiluTableBytes);
    allow_dynamic_smem<fp8_rows_kernel<2, kOp, kStatic>>(kSiluTableBytes);
    allow_dynamic_smem<fp8_rows_kernel<4, kOp, kStatic>>(kSiluTableBytes);
    allow_dynamic_smem<fp8_rows_kernel<8, kOp, kStatic>>(kSiluTableBytes);
    allow_dynamic_smem<fp8_rows_kernel<4, kOp, kStatic, kMlpRowThreads>>(kSiluTableBytes);
}

template <row_op kOp, bool kStatic = false>
int launch_fp8_rows(const void *in, uint32_t rows, uint32_t width, uint32_t in_chunks_per_row, uint8_t *codes,
                    float *scales, cudaStream_t stream, float given_scale = 0.0f) {
    const uint32_t chunks = width / 8u;
    const row_shape s = pick_row_shape(chunks);
    if (s.threads == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    constexpr bool kTable = kOp == row_op::swiglu_table;
    const size_t smem = kTable ? kSiluTableBytes : 0u;
    const float *device_table = kTable ? device_silu_table(stream) : nullptr;
    // table flavour: persistent CTAs (the table is built once per CTA), two per SM
    const uint32_t cap = kTable ? kSmCount * 2u : kSmCount * 16u;
    const uint32_t ctas = rows < cap ? rows : cap;
    const uint4 *src = (const uint4 *)in;
    uint2 *dst = (uint2 *)codes;
    if (kTable) configure_fp8_rows<kOp, kStatic>();
    if (kTable && s.cpt == 4u && s.threads * 4u == chunks && s.threads == kMlpRowThreads) {
        // the reference model's MLP width (17408 = 544 threads x 4 chunks x 8): row geometry as compile-time constants
        launch_chained(fp8_rows_kernel<4, kOp, kStatic, kMlpRowThreads>, dim3(ctas), dim3(s.threads), smem, stream, src, rows, chunks, in_chunks_per_row, dst, scales, device_table, given_scale);
        note_launch();
        return AXIOM_OK;
    }
    switch (s.cpt) {
    case 1: launch_chained(fp8_rows_kernel<1, kOp, kStatic>, dim3(ctas), dim3(s.threads), smem, stream, src, rows, chunks, in_chunks_per_row, dst, scales, device_table, given_scale); break;
    case 2: launch_chained(fp8_rows_kernel<2, kOp, kStatic>, dim3(ctas), dim3(s.threads), smem, stream, src, rows, chunks, in_chunks_per_row, dst, scales, device_table, given_scale); break;
    case 4: launch_chained(fp8_rows_kernel<4, kOp, kStatic>, dim3(ctas), dim3(s.threads), smem, stream, src, rows, chunks, in_chunks_per_row, dst, scales, device_table, given_scale); break;
    default: launch_chained(fp8_rows_kernel<8, kOp, kStatic>, dim3(ctas), dim3(s.threads), smem, stream, src, rows, chunks, in_chunks_per_row, dst, scales, device_table, given_scale); break;
    }
    note_launch();
    return AXIOM_OK;
}

// rows at or above which a 64 KB shared-memory silu table per CTA pays for itself: when every
// CTA fills its own, and when it only copies the device table
constexpr uint32_t kTableMinRows = 2u * kSmCount;
constexpr uint32_t kCopiedTableMinRows = 96u;

}  // namespace

unsigned int swiglu_fault_word() { return read_and_clear_pipeline_fault(); }



int launch_swiglu_fp8_bf16(const void *gate_up, uint32_t rows, uint32_t width, uint8_t *codes, float *scales,
                           cudaStream_t stream) {
    if (rows >= kTableMinRows) {
        return launch_fp8_rows<row_op::swiglu_table>(gate_up, rows, width, width / 4u, codes, scales, stream);
    }
    return launch_fp8_rows<row_op::swiglu>(gate_up, rows, width, width / 4u, codes, scales, stream);
}

// Given-scale flavours: the same row kernels without the row maximum (one pass, nothing to reduce).
template <bool kStatic>
int launch_fp8_plain_rows(const void *in, uint32_t rows, uint32_t cols, uint8_t *codes, float *scales, uint32_t *status_word,
                          cudaStream_t stream, float given_scale) {
    const uint32_t chunks = cols / 8u;
    const row_shape s = pick_row_shape(chunks, rows >= 4u * kSmCount);
    if (s.threads == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint32_t cap = kSmCount * 16u;
    const uint32_t ctas = rows < cap ? rows : cap;
    const uint4 *src = (const uint4 *)in;
    uint2 *dst = (uint2 *)codes;
    switch (s.cpt) {
    case 1: launch_chained(fp8_plain_rows_kernel<1, kStatic>, dim3(ctas), dim3(s.threads), 0, stream, src, rows, chunks, chunks, dst, scales, status_word, given_scale); break;
    case 2: launch_chained(fp8_plain_rows_kernel<2, kStatic>, dim3(ctas), dim3(s.threads), 0, stream, src, rows, chunks, chunks, dst, scales, status_word, given_scale); break;
    case 4: launch_chained(fp8_plain_rows_kernel<4, kStatic>, dim3(ctas), dim3(s.threads), 0, stream, src, rows, chunks, chunks, dst, scales, status_word, given_scale); break;
    default: launch_chained(fp8_plain_rows_kernel<8, kStatic>, dim3(ctas), dim3(s.threads), 0, stream, src, rows, chunks, chunks, dst, scales, status_word, given_scale); break;
    }
    note_launch();
    return AXIOM_OK;
}

int launch_fp8_quantize_static_bf16(const void *input, uint32_t rows, uint32_t cols, float scale, uint8_t *codes,
                                    cudaStream_t stream) {
    return launch_fp8_plain_rows<true>(input, rows, cols, codes, nullptr, nullptr, stream, scale);
}

int launch_swiglu_fp8_static_bf16(const void *gate_up, uint32_t rows, uint32_t width, float scale, uint8_t *codes,
                                  cudaStream_t stream) {
    if (rows >= kTableMinRows) {
        return launch_fp8_rows<row_op::swiglu_table, true>(gate_up, rows, width, width / 4u, codes, nullptr, stream, scale);
    }
    return launch_fp8_rows<row_op::swiglu, true>(gate_up, rows, width, width / 4u, codes, nullptr, stream, scale);
}

int launch_fp8_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, uint8_t *codes, float *scales,
                             uint32_t *status_word, cudaStream_t stream) {
    return launch_fp8_plain_rows<false>(input, rows, cols, codes, scales, status_word, stream, 0.0f);
}

template <gate_fn kFn>
void configure_gated_stream() {
    allow_dynamic_smem<gated_nvfp4_stream_kernel<kFn, true, true, true>>(kSiluTableBytes);
    allow_dynamic_smem<gated_nvfp4_stream_kernel<kFn, false, true, true>>(kSiluTableBytes);
    allow_dynamic_smem<gated_nvfp4_stream_kernel<kFn, true, false, true>>(kSiluTableBytes);
    allow_dynamic_smem<gated_nvfp4_stream_kernel<kFn, false, false, true>>(kSiluTableBytes);
    allow_dynamic_smem<gated_nvfp4_stream_kernel<kFn, false, true, false>>(kSiluTableBytes);
}

// Shared launcher of the two gated NVFP4 ops.  `gate` / `other` are the two operand planes, row_stride their row
// pitch in 16-byte chunks.
template <gate_fn kFn, bool kHeadGate = false>
int launch_gated_nvfp4(const uint4 *gate, const uint4 *other, uint32_t row_stride, uint32_t other_row_stride,
                       uint32_t gate_head_chunks, uint32_t rows, uint32_t width, float G, void *out_bf16, uint8_t *codes,
                       uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    const uint32_t chunks = width / 8u;
    const uint32_t groups = width / kGroup;
    const uint32_t col_groups = (chunks + 31u) / 32u;
    const uint64_t tiles = (uint64_t)rows * col_groups;
    const uint32_t warps_per_block = kNvThreads / 32u;
    const float *device_table = rows >= kCopiedTableMinRows ? device_gate_table<kFn>(stream) : nullptr;
    const bool table = rows >= kTableMinRows || device_table != nullptr;
    // table flavour: persistent CTAs (the table is built once per CTA), two 512-thread CTAs with 64 KB each per SM
    const uint64_t cap = table ? kSmCount * 2u : kSmCount * 8u;
    uint64_t blocks = (tiles + warps_per_block - 1u) / warps_per_block;
    if (blocks > cap) blocks = cap;
    const uint32_t W = (uint32_t)blocks * warps_per_block;
    const uint32_t head_keep = gate_head_chunks ? ~(gate_head_chunks - 1u) : 0u;  // gate_head_chunks is a power of two
    // regular shape with enough rows for persistent CTAs: the streaming kernel (contiguous tile ranges per warp)
    if (!kHeadGate && (chunks % 32u) == 0u && device_table != nullptr && rows >= kTableMinRows && tiles <= 0xffffffffull) {
        const uint32_t ctas = kSmCount * 2u;
        const uint32_t warps = ctas * warps_per_block;
        const uint32_t per_warp = (uint32_t)((tiles + warps - 1u) / warps);
        // one instantiation per (scale layout, outputs asked for)
        configure_gated_stream<kFn>();
        auto launch = [&](auto kernel) {
            launch_chained(kernel, dim3(ctas), dim3(kNvThreads), kSiluTableBytes, stream, gate, other, row_stride, other_row_stride,
                           (uint32_t)tiles, per_warp, col_groups, G, (uint4 *)out_bf16, (uint32_t *)codes, scales,
                           (groups + 3u) / 4u, device_table);
        };
        const bool tiled = layout == AXIOM_SCALE_LAYOUT_TILED;
        if (codes && out_bf16) {
            if (tiled) launch(gated_nvfp4_stream_kernel<kFn, true, true, true>);
            else launch(gated_nvfp4_stream_kernel<kFn, false, true, true>);
        } else if (codes) {
            if (tiled) launch(gated_nvfp4_stream_kernel<kFn, true, false, true>);
            else launch(gated_nvfp4_stream_kernel<kFn, false, false, true>);
        } else {
            launch(gated_nvfp4_stream_kernel<kFn, false, true, false>);
        }
        note_launch();
        return AXIOM_OK;
    }
    if (table) {
        allow_dynamic_smem<swiglu_nvfp4_kernel<true, kFn, kHeadGate>>(kSiluTableBytes);
        launch_chained(swiglu_nvfp4_kernel<true, kFn, kHeadGate>, dim3((uint32_t)blocks), dim3(kNvThreads), kSiluTableBytes, stream,
                       gate, other, row_stride, other_row_stride, head_keep, gate_head_chunks, rows, chunks, col_groups,
                       W / col_groups, W % col_groups, G, (uint4 *)out_bf16,
                       (uint32_t *)codes, scales, layout, groups, (groups + 3u) / 4u, device_table);
    } else {
        launch_chained(swiglu_nvfp4_kernel<false, kFn, kHeadGate>, dim3((uint32_t)blocks), dim3(kNvThreads), 0, stream,
                       gate, other, row_stride, other_row_stride, head_keep, gate_head_chunks, rows, chunks, col_groups,
                       W / col_groups, W % col_groups, G, (uint4 *)out_bf16,
                       (uint32_t *)codes, scales, layout, groups, (groups + 3u) / 4u, nullptr);
    }
    note_launch();
    return AXIOM_OK;
}

int launch_swiglu_nvfp4_bf16(const void *gate_up, uint32_t rows, uint32_t width, float G, uint8_t *codes,
                             uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    const uint4 *gate = (const uint4 *)gate_up;
    return launch_gated_nvfp4<gate_fn::silu>(gate, gate + width / 8u, 2u * (width / 8u), 2u * (width / 8u), 0u, rows, width, G,
                                             nullptr, codes, scales, layout, stream);
}

int launch_sigmoid_gate_nvfp4_bf16(const void *attention, const void *gate, uint32_t rows, uint32_t width, float G,
                                   void *out_bf16, uint8_t *codes, uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    return launch_gated_nvfp4<gate_fn::sigmoid>((const uint4 *)gate, (const uint4 *)attention, width / 8u, width / 8u, 0u, rows,
                                                width, G, out_bf16, codes, scales, layout, stream);
}

// Gate values read where the q projection left them: q_gate is [rows][heads][2 * head_dim], each head's
// gate values behind its query values.
int launch_sigmoid_gate_heads_nvfp4_bf16(const void *attention, const void *q_gate, uint32_t rows, uint32_t heads,
                                         uint32_t head_dim, float G, void *out_bf16, uint8_t *codes, uint8_t *scales,
                                         uint32_t layout, cudaStream_t stream) {
    const uint32_t width = heads * head_dim;
    return launch_gated_nvfp4<gate_fn::sigmoid, true>((const uint4 *)q_gate, (const uint4 *)attention, 2u * (width / 8u), width / 8u,
                                                      head_dim / 8u, rows, width, G, out_bf16, codes, scales, layout, stream);
}

// Everything a first launch would set up lazily, for axiom_b200_prepare(): both gate tables (one small kernel and one
// stream synchronisation each) and the shared-memory limits of every table kernel.  False when a table could not
// be filled (the kernels then keep filling a copy per CTA).
bool prepare_gated_unit() {
    const bool tables = device_gate_table<gate_fn::silu>(nullptr) != nullptr && device_gate_table<gate_fn::sigmoid>(nullptr) != nullptr;
    configure_fp8_rows<row_op::swiglu_table, false>();
    configure_fp8_rows<row_op::swiglu_table, true>();
    configure_gated_stream<gate_fn::silu>();
    configure_gated_stream<gate_fn::sigmoid>();
    allow_dynamic_smem<swiglu_nvfp4_kernel<true, gate_fn::silu, false>>(kSiluTableBytes);
    allow_dynamic_smem<swiglu_nvfp4_kernel<true, gate_fn::sigmoid, false>>(kSiluTableBytes);
    allow_dynamic_smem<swiglu_nvfp4_kernel<true, gate_fn::sigmoid, true>>(kSiluTableBytes);
    return tables;
}

}  // namespace axb

using namespace axb;

extern "C" int axiom_qwen38_fused_swiglu_fp8_bf16_device(
        int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, uint8_t *out_codes,
        float *out_scales, void *stream) {
    if (!gate_up_bf16 || !out_codes || !out_scales || rows == 0u || width == 0u || (width % 8u) != 0u ||
        width > 36864u || !aligned16(gate_up_bf16) || (reinterpret_cast<uintptr_t>(out_codes) & 7u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    rc = launch_swiglu_fp8_bf16(gate_up_bf16, rows, width, out_codes, out_scales, (cudaStream_t)stream);
    return rc != AXIOM_OK ? rc : launch_status();
}

extern "C" int axiom_qwen38_fused_fp8_quantize_bf16_device(
        int device, const void *input_bf16, uint32_t rows, uint32_t cols, uint8_t *out_codes,
        float *out_scales, uint32_t *status_word, void *stream) {
    if (!input_bf16 || !out_codes || !out_scales || rows == 0u || cols == 0u || (cols % 8u) != 0u ||
        cols > 36864u || !aligned16(input_bf16) || (reinterpret_cast<uintptr_t>(out_codes) & 7u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    rc = launch_fp8_quantize_bf16(input_bf16, rows, cols, out_codes, out_scales, status_word, (cudaStream_t)stream);
    return rc != AXIOM_OK ? rc : launch_status();
}

extern "C" int axiom_qwen38_fused_fp8_quantize_static_bf16_device(
        int device, const void *input_bf16, uint32_t rows, uint32_t cols, float scale, uint8_t *out_codes, void *stream) {
    if (!input_bf16 || !out_codes || rows == 0u || cols == 0u || (cols % 8u) != 0u || cols > 36864u || !valid_scale(scale) ||
        !aligned16(input_bf16) || (reinterpret_cast<uintptr_t>(out_codes) & 7u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    rc = launch_fp8_quantize_static_bf16(input_bf16, rows, cols, scale, out_codes, (cudaStream_t)stream);
    return rc != AXIOM_OK ? rc : launch_status();
}

extern "C" int axiom_qwen38_fused_swiglu_fp8_static_bf16_device(
        int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, float scale, uint8_t *out_codes, void *stream) {
    if (!gate_up_bf16 || !out_codes || rows == 0u || width == 0u || (width % 8u) != 0u || width > 36864u ||
        !valid_scale(scale) || !aligned16(gate_up_bf16) || (reinterpret_cast<uintptr_t>(out_codes) & 7u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    rc = launch_swiglu_fp8_static_bf16(gate_up_bf16, rows, width, scale, out_codes, (cudaStream_t)stream);
    return rc != AXIOM_OK ? rc : launch_status();
}

extern "C" int axiom_qwen38_fused_swiglu_nvfp4_bf16_device(
        int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, float global_scale,
        uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!gate_up_bf16 || !out_codes || !out_scales || rows == 0u || width == 0u || (width % kGroup) != 0u ||
        !valid_scale(global_scale) || scale_layout > AXIOM_SCALE_LAYOUT_TILED || !aligned16(gate_up_bf16) ||
        (reinterpret_cast<uintptr_t>(out_codes) & 3u) || (uint64_t)rows * (width / 8u) > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_swiglu_nvfp4_bf16(gate_up_bf16, rows, width, global_scale, out_codes, out_scales, scale_layout,
                             (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_sigmoid_gate_nvfp4_bf16_device(
        int device, const void *attention_bf16, const void *gate_bf16, uint32_t rows, uint32_t width, float global_scale,
        void *out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!attention_bf16 || !gate_bf16 || rows == 0u || width == 0u || (width % kGroup) != 0u ||
        scale_layout > AXIOM_SCALE_LAYOUT_TILED || !aligned16(attention_bf16) || !aligned16(gate_bf16) ||
        (uint64_t)rows * (width / 8u) > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && (!valid_scale(global_scale) || (reinterpret_cast<uintptr_t>(out_codes) & 3u))) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_bf16 && !aligned16(out_bf16)) return AXIOM_ERR_INVALID_ARGUMENT;
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_sigmoid_gate_nvfp4_bf16(attention_bf16, gate_bf16, rows, width, out_codes ? global_scale : 1.0f, out_bf16, out_codes,
                                   out_scales, scale_layout, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_sigmoid_gate_heads_nvfp4_bf16_device(
        int device, const void *attention_bf16, const void *q_gate_bf16, uint32_t rows, uint32_t heads, uint32_t head_dim,
        float global_scale, void *out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!attention_bf16 || !q_gate_bf16 || rows == 0u || heads == 0u || heads > 4096u ||
        (head_dim != 64u && head_dim != 128u && head_dim != 256u) || scale_layout > AXIOM_SCALE_LAYOUT_TILED ||
        !aligned16(attention_bf16) || !aligned16(q_gate_bf16) || (uint64_t)rows * (heads * head_dim / 8u) * 2u > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && (!valid_scale(global_scale) || (reinterpret_cast<uintptr_t>(out_codes) & 3u))) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_bf16 && !aligned16(out_bf16)) return AXIOM_ERR_INVALID_ARGUMENT;
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_sigmoid_gate_heads_nvfp4_bf16(attention_bf16, q_gate_bf16, rows, heads, head_dim, out_codes ? global_scale : 1.0f,
                                         out_bf16, out_codes, out_scales, scale_layout, (cudaStream_t)stream);
    return launch_status();
}

// Attention pre-processing: per-head q/k RMSNorm, NeoX RoPE (YaRN frequencies),
// paged-KV write — one pass over Q and K.
//
// Arithmetic of qwen38_qk_norm_partial_rope_cache8_kernel
// (src/axiom_qwen38_attention.cu:481-554) with the paged addressing of
// axiom_kv_pool_store_paged_f32_kernel (src/axiom_cuda.cu:16954-16969):
//   ss  = sum x^2 in FP64, inv = (float)(1/sqrt(ss/D + eps))
//   n   = (x * inv) * gamma                         FP32
//   ang = (float)pos * inv_freq[p]; c = cosf(ang)*mscale; s = sinf(ang)*mscale
//   out[p]      = bf16(fma(n[p], c, -(n[p+half]*s)))
//   out[p+half] = bf16(fma(n[p], s,   n[p+half]*c))
//   dims >= rope_dim: bf16(n)
//
// A lane owns BOTH members of four NeoX pairs: dims 4l..4l+3 and rope_dim/2 + 4l.. of one
// head (two 8-byte accesses; a warp still covers whole 128-byte lines), so the rotation needs
// no lane exchange, no select and no divergent branch.  Lanes past the rotary dims carry 8
// pass-through dims.  head_dim/8 adjacent lanes form a head, so a head never leaves its warp:
// the FP64 sum is a shuffle butterfly and every lane derives the head's factor itself.  The
// only cross-thread data is the token's rotary table (cos, sin, -sin per pair; sincosf gives
// bit-for-bit the values of separate sinf and cosf calls for every non-negative float —
// checked exhaustively on the device).  Two kernels share this arithmetic: one CTA per token
// for short batches, and a persistent bulk-copy pipeline for long ones.
// The frequency table is an input: it is evaluated once per model on the device
// (yarn_inv_freq_kernel) instead of powf/logf per thread per call.
#include <cuda.h>  // CUtensorMap and its enums only: the encoder is fetched through the runtime, nothing links libcuda

#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {


constexpr uint32_t kMaxHeads = 512u;
constexpr uint32_t kMaxHeadDim = 256u;

struct qk_dev_args {
    const uint4 *q;          // source rows: q_heads heads at a pitch of q_head_stride elements
    uint4 *q_out;            // destination rows, heads packed
    uint32_t q_head_stride;  // head_dim, or 2 * head_dim when each head is followed by its gate values
    uint32_t q_use_map;      // streaming kernel: the strided query halves of a token come through the tensor map
    const uint4 *k;
    const uint4 *v;
    const uint16_t *q_gamma;
    const uint16_t *k_gamma;
    const float *inv_freq;
    const uint32_t *positions;
    const int32_t *block_tables;
    uint4 *k_pool;
    uint4 *v_pool;
    uint4 *k_out;
    uint32_t *status_word;
    uint32_t tokens, q_heads, k_heads, head_dim, rope_dim, flags;
    float eps, mscale;
    uint32_t block_tokens, n_layers, layer, pool_stride, tbl_stride, n_blocks;
    const float *rope_table;        // optional [rope_table_positions][head_dim]: cos(head_dim/2) | sin(head_dim/2) per position
    uint32_t rope_table_positions;
};

__device__ __forceinline__ uint2 ld_stream8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}


// (float)(1.0 / sqrt(v)), v = ss / D + eps, without the FP64 square root and division on the
// common path.  y0 = rsqrt.approx(float(v)) is within 2^-22 of 1/sqrt(v); one Newton step in
// FP64, y = y0 + (y0/2)(1 - v*y0^2), brings that to 1.5 * 2^-44.  The reference value (a
// correctly rounded FP64 sqrt, then a correctly rounded division: within 2^-52 of the true
// quotient) and y therefore both lie in [y(1 - 2^-41), y(1 + 2^-41)]; when the two ends of that
// interval round to the same float, every value inside does, and that float is the answer.
// Otherwise (about one value in 2^17), or when float(v) leaves the range where the
// approximation is specified for normal numbers, the plain expression is evaluated.
// The plain expression, out of line: the FP64 square root and division (and their slow paths) then take no
// registers from the loop that calls inv_rms_from_sum.
static __device__ __noinline__ float inv_rms_plain(double v) { return (float)(1.0 / sqrt(v)); }

__device__ __forceinline__ float inv_rms_from_sum(double ss, double inv_d, double eps) {
    const double v = __fma_rn(ss, inv_d, eps);  // ss / D is exact (D is a power of two)
    const float vf = (float)v;
    float y0;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y0) : "f"(vf));
    const double y0d = (double)y0;
    const double r = __fma_rn(-__dmul_rn(v, y0d), y0d, 1.0);
    const double y = __fma_rn(__dmul_rn(0.5, y0d), r, y0d);
    const float lo = (float)__dmul_rn(y, 1.0 - 0x1p-41), hi = (float)__dmul_rn(y, 1.0 + 0x1p-41);
    if (lo == hi && vf > 1.0e-30f && vf < 1.0e30f) return lo;
    return inv_rms_plain(v);
}

// One row of the rotary table: c = cosf(angle) * mscale, s = sinf(angle) * mscale with
// angle = (float)pos * inv_freq.  sincosf() shares the argument reduction between the two.
__device__ __forceinline__ void rope_table_entry(uint32_t pos, float inv_freq, float mscale, float *c, float *s) {
    const float angle = __fmul_rn((float)pos, inv_freq);
    float sv, cv;
    sincosf(angle, &sv, &cv);
    *c = __fmul_rn(cv, mscale);
    *s = __fmul_rn(sv, mscale);
}

// Rotary factors of one lane: four (cos, sin, -sin) triples as packed pairs.
struct rot_regs {
    float2 c0, c1, s0, s1, n0, n1;
};

__device__ __forceinline__ rot_regs load_rot(const float *cos_t, const float *sin_t, const float *nsin_t, uint32_t off,
                                             bool rotary) {
    float4 c = make_float4(0.f, 0.f, 0.f, 0.f), sn = c, ns = c;
    if (rotary) {
        c = *reinterpret_cast<const float4 *>(cos_t + off);
        sn = *reinterpret_cast<const float4 *>(sin_t + off);
        ns = *reinterpret_cast<const float4 *>(nsin_t + off);
    }
    rot_regs r;
    r.c0 = make_float2(c.x, c.y); r.c1 = make_float2(c.z, c.w);
    r.s0 = make_float2(sn.x, sn.y); r.s1 = make_float2(sn.z, sn.w);
    r.n0 = make_float2(ns.x, ns.y); r.n1 = make_float2(ns.z, ns.w);
    return r;
}

// One work item: eight dims of one head held by one lane (xa = dims off_a.., xb = dims off_b..).
// head_sum: the squares summed in FP64 across the LPH lanes of the head (xor butterfly: every lane ends with
// the total; FP64 sums of BF16 squares are exact unless the row spans more than ~2^18 in
// magnitude, so the order of the additions is immaterial).
__device__ __forceinline__ double lane_sum(uint2 xa, uint2 xb) {
    const float2 fa0 = bf16x2_widen_fma(xa.x), fa1 = bf16x2_widen_fma(xa.y);
    const float2 fb0 = bf16x2_widen_fma(xb.x), fb1 = bf16x2_widen_fma(xb.y);
    const double d0 = (double)fa0.x, d1 = (double)fa0.y, d2 = (double)fa1.x, d3 = (double)fa1.y;
    const double e0 = (double)fb0.x, e1 = (double)fb0.y, e2 = (double)fb1.x, e3 = (double)fb1.y;
    double s = 0.0, s_hi = 0.0;
    s = __fma_rn(d0, d0, s); s_hi = __fma_rn(e0, e0, s_hi);
    s = __fma_rn(d1, d1, s); s_hi = __fma_rn(e1, e1, s_hi);
    s = __fma_rn(d2, d2, s); s_hi = __fma_rn(e2, e2, s_hi);
    s = __fma_rn(d3, d3, s); s_hi = __fma_rn(e3, e3, s_hi);
    return s + s_hi;
}

template <int LPH>
__device__ __forceinline__ double head_sum(uint2 xa, uint2 xb) {
    double s = lane_sum(xa, xb);
#pragma unroll
    for (int off = LPH / 2; off != 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    return s;
}

// The sums of NPT heads, each spread over the same LPH lanes, reduced so that every head's total lands in
// ONE pair of lanes instead of in all of them (recursive halving: in each round a lane keeps half of its
// partial sums and hands the other half to its partner, so the exchange shrinks from NPT values to one).
// Head n's total ends in the lanes n * (LPH / P) .. of the group, P = NPT rounded up to a power of two; the
// other lanes' results are not totals of anything.  For 6 heads on 16 lanes this is 14 64-bit exchanges
// instead of 24.  The additions are exact for the same reason as in head_sum, so their order is immaterial.
template <int NPT>
struct pow2_at_least {
    static constexpr int value = NPT <= 1 ? 1 : NPT <= 2 ? 2 : NPT <= 4 ? 4 : NPT <= 8 ? 8 : NPT <= 16 ? 16 : 32;
};

template <int LPH, int NPT>
__device__ __forceinline__ double scatter_head_sums(const double (&ss)[NPT], uint32_t l) {
    constexpr int P = pow2_at_least<NPT>::value;
    static_assert(P <= LPH, "more heads per thread than lanes per head");
    double a[P];
#pragma unroll
    for (int i = 0; i < P; ++i) a[i] = i < NPT ? ss[i] : 0.0;
#pragma unroll
    for (int C = P; C > 1; C >>= 1) {
        const int half = C / 2;
        const uint32_t bit = (uint32_t)(LPH * C / (2 * P));  // lane distance of this round's partner
        const bool upper = (l & bit) != 0u;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            if (C == P && i + half >= NPT) {
                a[i] += __shfl_xor_sync(0xffffffffu, a[i], bit);  // no head in the upper slot: nothing to choose
            } else {
                const double send = upper ? a[i] : a[i + half];
                const double keep = upper ? a[i + half] : a[i];
                a[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
            }
        }
    }
#pragma unroll
    for (int off = LPH / (2 * P); off != 0; off >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], off);
    return a[0];
}

// qk_apply: normalises with the head's factor, rotates and packs.
__device__ __forceinline__ void qk_apply(uint2 xa, uint2 xb, float inv, const float4 ga, const float4 gb, const rot_regs &r,
                                         bool rotary, uint2 *out_a, uint2 *out_b) {
    const float2 fa0 = bf16x2_widen_fma(xa.x), fa1 = bf16x2_widen_fma(xa.y);
    const float2 fb0 = bf16x2_widen_fma(xb.x), fb1 = bf16x2_widen_fma(xb.y);
    const float2 inv2 = make_float2(inv, inv);
    // n = (x * inv) * gamma
    const float2 a0 = __fmul2_rn(__fmul2_rn(fa0, inv2), make_float2(ga.x, ga.y));
    const float2 a1 = __fmul2_rn(__fmul2_rn(fa1, inv2), make_float2(ga.z, ga.w));
    const float2 b0 = __fmul2_rn(__fmul2_rn(fb0, inv2), make_float2(gb.x, gb.y));
    const float2 b1 = __fmul2_rn(__fmul2_rn(fb1, inv2), make_float2(gb.z, gb.w));
    float2 oa0 = a0, oa1 = a1, ob0 = b0, ob1 = b1;
    if (rotary) {
        // out[p] = fma(first, c, -(second*s)); out[p+half] = fma(second, c, first*s): which product of
        // `first * sine + second * cosine` (src/axiom_qwen38_attention.cu:534-535) the reference's build fuses was
        // settled against its kernel on 2.2 M rotated pairs (the other choice differs in 1.6e-5 of them, mostly
        // where the two terms cancel, and in the sign of results that underflow to zero)
        oa0 = __ffma2_rn(a0, r.c0, __fmul2_rn(b0, r.n0));
        oa1 = __ffma2_rn(a1, r.c1, __fmul2_rn(b1, r.n1));
        ob0 = __ffma2_rn(b0, r.c0, __fmul2_rn(a0, r.s0));
        ob1 = __ffma2_rn(b1, r.c1, __fmul2_rn(a1, r.s1));
    }
    *out_a = make_uint2(pack_bf16x2(oa0.x, oa0.y), pack_bf16x2(oa1.x, oa1.y));
    *out_b = make_uint2(pack_bf16x2(ob0.x, ob0.y), pack_bf16x2(ob1.x, ob1.y));
}

// Both steps for one item, every lane deriving the head's factor itself — the same instructions a single
// lane would cost, and no shared-memory round trip or barrier.
template <int LPH>
__device__ __forceinline__ void qk_item(uint2 xa, uint2 xb, const float4 ga, const float4 gb, const rot_regs &r,
                                        bool rotary, double inv_d, double eps, uint2 *out_a, uint2 *out_b) {
    const float inv = inv_rms_from_sum(head_sum<LPH>(xa, xb), inv_d, eps);
    qk_apply(xa, xb, inv, ga, gb, r, rotary, out_a, out_b);
}

// ---- the BF16 ("draft") rounding convention: qk_rmsnorm_rope_bf16_kernel + round_f32_to_bf16_inplace_kernel
// (src/axiom_qwen38_dspark_compute.cu:250-300,210-213) ------------------------------------------------------------
//   ss   = FP32 tree over the head: squares (exact for BF16 inputs), strides D/2, D/4, .. 1, r[i] += r[i + stride]
//   inv  = rsqrtf(ss / D + eps)
//   n    = bf16((x * inv) * gamma)            <- rounded BEFORE the rotation
//   out[p] = bf16(n[p] * c - n[p+D/2] * s), out[p+D/2] = bf16(n[p] * s + n[p+D/2] * c)
// With a lane holding dims 4l.. and D/2 + 4l.., the first tree level (i, i + D/2) is the lane's own two halves, the
// levels down to stride 4 are lane butterflies (both partners compute the same FP32 sum, addition commutes), and
// strides 2 and 1 combine the lane's four values: every addition has the operands of the reference's tree.
template <int LPH>
__device__ __forceinline__ float head_sum_f32_tree(uint2 xa, uint2 xb) {
    const float2 fa0 = bf16x2_widen_fma(xa.x), fa1 = bf16x2_widen_fma(xa.y);
    const float2 fb0 = bf16x2_widen_fma(xb.x), fb1 = bf16x2_widen_fma(xb.y);
    float q0 = __fadd_rn(__fmul_rn(fa0.x, fa0.x), __fmul_rn(fb0.x, fb0.x));
    float q1 = __fadd_rn(__fmul_rn(fa0.y, fa0.y), __fmul_rn(fb0.y, fb0.y));
    float q2 = __fadd_rn(__fmul_rn(fa1.x, fa1.x), __fmul_rn(fb1.x, fb1.x));
    float q3 = __fadd_rn(__fmul_rn(fa1.y, fa1.y), __fmul_rn(fb1.y, fb1.y));
#pragma unroll
    for (int off = LPH / 2; off != 0; off >>= 1) {
        q0 = __fadd_rn(q0, __shfl_xor_sync(0xffffffffu, q0, off));
        q1 = __fadd_rn(q1, __shfl_xor_sync(0xffffffffu, q1, off));
        q2 = __fadd_rn(q2, __shfl_xor_sync(0xffffffffu, q2, off));
        q3 = __fadd_rn(q3, __shfl_xor_sync(0xffffffffu, q3, off));
    }
    return __fadd_rn(__fadd_rn(q0, q2), __fadd_rn(q1, q3));
}

__device__ __forceinline__ void qk_apply_round_after_norm(uint2 xa, uint2 xb, float inv, const float4 ga, const float4 gb,
                                                          const rot_regs &r, uint2 *out_a, uint2 *out_b) {
    const float2 fa0 = bf16x2_widen_fma(xa.x), fa1 = bf16x2_widen_fma(xa.y);
    const float2 fb0 = bf16x2_widen_fma(xb.x), fb1 = bf16x2_widen_fma(xb.y);
    const float2 inv2 = make_float2(inv, inv);
    const float2 ua0 = __fmul2_rn(__fmul2_rn(fa0, inv2), make_float2(ga.x, ga.y));
    const float2 ua1 = __fmul2_rn(__fmul2_rn(fa1, inv2), make_float2(ga.z, ga.w));
    const float2 ub0 = __fmul2_rn(__fmul2_rn(fb0, inv2), make_float2(gb.x, gb.y));
    const float2 ub1 = __fmul2_rn(__fmul2_rn(fb1, inv2), make_float2(gb.z, gb.w));
    // the normalised values exist in BF16 only
    const float2 a0 = bf16x2_widen_fma(pack_bf16x2(ua0.x, ua0.y)), a1 = bf16x2_widen_fma(pack_bf16x2(ua1.x, ua1.y));
    const float2 b0 = bf16x2_widen_fma(pack_bf16x2(ub0.x, ub0.y)), b1 = bf16x2_widen_fma(pack_bf16x2(ub1.x, ub1.y));
    // here the reference's build fuses the FIRST product of both sums (checked against its kernel on 14 M pairs)
    const float2 oa0 = __ffma2_rn(a0, r.c0, __fmul2_rn(b0, r.n0)), oa1 = __ffma2_rn(a1, r.c1, __fmul2_rn(b1, r.n1));
    const float2 ob0 = __ffma2_rn(a0, r.s0, __fmul2_rn(b0, r.c0)), ob1 = __ffma2_rn(a1, r.s1, __fmul2_rn(b1, r.c1));
    *out_a = make_uint2(pack_bf16x2(oa0.x, oa0.y), pack_bf16x2(oa1.x, oa1.y));
    *out_b = make_uint2(pack_bf16x2(ob0.x, ob0.y), pack_bf16x2(ob1.x, ob1.y));
}

// BF16 -> E4M3 codes at scale 1 for the FP8 flavour of the cache (qwen38_kv_encode_e4m3fn_scale1,
// src/axiom_qwen38_attention.cu:245-248: the saturating converter applied to the BF16-valued float).
__device__ __forceinline__ uint32_t bf16x4_to_e4m3x4(const uint2 v) {
    return __byte_perm(cvt_e4m3x2(bf16_lo(v.x), bf16_hi(v.x)), cvt_e4m3x2(bf16_lo(v.y), bf16_hi(v.y)), 0x5410);
}
__device__ __forceinline__ uint2 bf16x8_to_e4m3x8(const uint4 v) {
    return make_uint2(bf16x4_to_e4m3x4(make_uint2(v.x, v.y)), bf16x4_to_e4m3x4(make_uint2(v.z, v.w)));
}

// ---------------------------------------------------------------------------
// Per-token flavour (few tokens: lowest latency).  One CTA per token, LPH = lanes per head
// (head_dim / 8), NPT = (head, lane) work items per thread.  kFast: every thread's NPT items
// exist and every lane carries rotary pairs, which removes the bounds predicates and the
// pass-through branch.  One CTA barrier: the rotary table (threads below rope_dim/2) and the
// cache address (thread 0) are produced while the Q/K loads are in flight.
// ---------------------------------------------------------------------------
template <int LPH, int NPT, bool kFast, bool kRoundAfterNorm = false>
__global__ void __launch_bounds__(512, 1)
qk_norm_rope_paged_kernel(const qk_dev_args a) {
    __shared__ __align__(16) float cos_sh[kMaxHeadDim / 2];
    __shared__ __align__(16) float sin_sh[kMaxHeadDim / 2];
    __shared__ __align__(16) float nsin_sh[kMaxHeadDim / 2];
    __shared__ __align__(16) float gq_sh[kMaxHeadDim];
    __shared__ __align__(16) float gk_sh[kMaxHeadDim];
    __shared__ unsigned long long kv_base_sh;  // element index into the pools, ~0 = no cache write
    constexpr uint32_t D = LPH * 8u;

    const uint32_t tid = threadIdx.x;
    const uint32_t heads = a.q_heads + a.k_heads;
    const uint32_t half = a.rope_dim >> 1;
    const uint32_t rot_lanes = a.rope_dim >> 3;  // lanes of a head that carry rotary pairs
    allow_dependents();
    dependency_wait();

    for (uint32_t i = tid; i < D; i += blockDim.x) {
        gq_sh[i] = a.q_heads ? __uint_as_float((uint32_t)a.q_gamma[i] << 16) : 0.0f;
        gk_sh[i] = a.k_heads ? __uint_as_float((uint32_t)a.k_gamma[i] << 16) : 0.0f;
    }

    // Work item n of this thread is (head tid/LPH + n*blockDim/LPH, lane tid%LPH): blockDim is a
    // multiple of 32 and LPH divides 32, so the lane geometry is the same for every item.
    const uint32_t l = tid % LPH;
    const uint32_t head0 = tid / LPH, head_step = blockDim.x / LPH;
    const bool rotary = kFast || l < rot_lanes;
    const uint32_t off_a = rotary ? 4u * l : a.rope_dim + 8u * (l - rot_lanes);
    const uint32_t off_b = rotary ? half + 4u * l : off_a + 4u;
    const uint32_t q_elems = a.q_heads * D, k_elems = a.k_heads * D;
    const double inv_d = 1.0 / (double)D, eps = (double)a.eps;
    const bool fp8_cache = (a.flags & AXIOM_QK_FLAG_CACHE_E4M3) != 0u;

    for (uint32_t t = blockIdx.x; t < a.tokens; t += gridDim.x) {
        const uint16_t *q_src = reinterpret_cast<const uint16_t *>(a.q) + (uint64_t)t * a.q_heads * a.q_head_stride;
        uint16_t *q_row = reinterpret_cast<uint16_t *>(a.q_out) + (uint64_t)t * q_elems;
        const uint16_t *k_row = reinterpret_cast<const uint16_t *>(a.k) + (uint64_t)t * k_elems;

        uint2 xa[NPT], xb[NPT];
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const uint32_t h = head0 + head_step * n;
            xa[n] = make_uint2(0u, 0u);
            xb[n] = make_uint2(0u, 0u);
            if (kFast || h < heads) {
                const uint16_t *row = h < a.q_heads ? q_src + h * a.q_head_stride : k_row + (h - a.q_heads) * D;
                xa[n] = ld_stream8(row + off_a);
                xb[n] = ld_stream8(row + off_b);
            }
        }
        const uint32_t pos = a.positions[t];
        // rotary factors of the token: evaluated here, or read from the caller's [position][cos | sin] table
        const bool from_table = kRoundAfterNorm && a.rope_table != nullptr;
        if (from_table && pos >= a.rope_table_positions) {
            // outside the table: the token is left as it is (the reference kernel returns), the status word says so
            if (tid == 0u && a.status_word) atomicCAS(a.status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
            continue;  // uniform over the CTA: every thread read the same position
        }
        for (uint32_t p = tid; p < half; p += blockDim.x) {  // one round unless the CTA is narrower than the table
            float cv, sv;
            if (from_table) {
                const float *row = a.rope_table + (uint64_t)pos * D;
                cv = row[p];
                sv = row[half + p];
            } else {
                rope_table_entry(pos, a.inv_freq[p], a.mscale, &cv, &sv);
            }
            cos_sh[p] = cv;
            sin_sh[p] = sv;
            nsin_sh[p] = -sv;
        }
        if (tid == blockDim.x - 1u) {
            unsigned long long base = ~0ull;
            if (a.k_pool) {
                uint32_t lb = pos / a.block_tokens;
                bool ok = true;
                if (a.flags & AXIOM_QK_FLAG_RING) lb %= a.tbl_stride;
                else if (lb >= a.tbl_stride) ok = false;
                int32_t pb = -1;
                if (ok) {
                    const uint64_t trow = (a.flags & AXIOM_QK_FLAG_PER_TOKEN_TABLE) ? t : 0u;
                    pb = a.block_tables[trow * a.tbl_stride + lb];
                    ok = pb >= 0 && (uint32_t)pb < a.n_blocks;
                }
                if (ok) {
                    base = (((uint64_t)pb * a.n_layers + a.layer) * a.block_tokens + pos % a.block_tokens) * a.pool_stride;
                } else if (a.status_word) {
                    atomicCAS(a.status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
                }
            }
            kv_base_sh = base;
        }
        __syncthreads();

        const unsigned long long kv_base = kv_base_sh;
        const rot_regs r = load_rot(cos_sh, sin_sh, nsin_sh, off_a, rotary);
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const uint32_t h = head0 + head_step * n;
            const bool is_k = h >= a.q_heads;
            const float *gamma = is_k ? gk_sh : gq_sh;
            const float4 ga = *reinterpret_cast<const float4 *>(gamma + off_a);
            const float4 gb = *reinterpret_cast<const float4 *>(gamma + off_b);
            uint2 pa, pb;
            if (kRoundAfterNorm) {
                const float ss = head_sum_f32_tree<LPH>(xa[n], xb[n]);
                const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)D), a.eps));
                qk_apply_round_after_norm(xa[n], xb[n], inv, ga, gb, r, &pa, &pb);
            } else {
                qk_item<LPH>(xa[n], xb[n], ga, gb, r, rotary, inv_d, eps, &pa, &pb);
            }
            if (kFast || h < heads) {
                if (!is_k) {
                    uint16_t *dst = q_row + h * D;
                    st_stream(dst + off_a, pa);
                    st_stream(dst + off_b, pb);
                } else {
                    const uint32_t off = (h - a.q_heads) * D;
                    if (kv_base != ~0ull) {
                        if (fp8_cache) {
                            uint8_t *dst = reinterpret_cast<uint8_t *>(a.k_pool) + kv_base + off;
                            st_stream(reinterpret_cast<uint32_t *>(dst + off_a), bf16x4_to_e4m3x4(pa));
                            st_stream(reinterpret_cast<uint32_t *>(dst + off_b), bf16x4_to_e4m3x4(pb));
                        } else {
                            uint16_t *dst = reinterpret_cast<uint16_t *>(a.k_pool) + kv_base + off;
                            st_stream(dst + off_a, pa);
                            st_stream(dst + off_b, pb);
                        }
                    }
                    if (a.k_out) {
                        uint16_t *dst = reinterpret_cast<uint16_t *>(a.k_out) + (uint64_t)t * k_elems + off;
                        st_stream(dst + off_a, pa);
                        st_stream(dst + off_b, pb);
                    }
                }
            }
        }
        // V rides along: a copy into a BF16 cache, a conversion into an E4M3 cache
        if (a.v && a.v_pool && kv_base != ~0ull) {
            const uint4 *v_row = a.v + (uint64_t)t * a.k_heads * LPH;
            if (fp8_cache) {
                uint2 *dst = reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(a.v_pool) + kv_base);
                for (uint32_t j = tid; j < a.k_heads * LPH; j += blockDim.x) st_stream(dst + j, bf16x8_to_e4m3x8(ld_stream(v_row + j)));
            } else {
                uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(a.v_pool) + kv_base);
                for (uint32_t j = tid; j < a.k_heads * LPH; j += blockDim.x) st_stream(dst + j, ld_stream(v_row + j));
            }
        }
        __syncthreads();  // the shared tables are rewritten for the next token
    }
}

// ---------------------------------------------------------------------------
// Streaming flavour for many tokens: a persistent CTA per SM made of independent teams.
// A team is a set of worker warps plus one manager warp and owns `slots` shared-memory token
// slots laid out [Q heads | K heads].  The manager's first lane keeps bulk loads of the next
// tokens in flight and sends finished slots out with bulk stores (Q row back in place, K row
// to its cache page and/or k_out); its lanes also compute the rotary table of the next token
// (double-buffered) and fetch positions and block-table entries two and one tokens ahead, so
// the dependent pos -> table -> address chain and every single-threaded instruction sequence
// run beside the arithmetic instead of in front of it.  The workers normalise and rotate the
// slot IN PLACE and meet the manager at one team barrier per token; V, a 2 KB copy per token,
// is moved by the first workers with 16-byte accesses.  With three or more slots, slot (i-1)
// is refilled at the end of token i, once its stores have finished reading shared memory (one
// store group may stay pending), so loads run `slots - 1` tokens ahead.
// ---------------------------------------------------------------------------
// One box of a 3-D tensor map -> shared memory, completion counted in bytes on `bar`.  The
// innermost coordinate times the element size has to be a multiple of 16 bytes (here it is 0),
// the destination 128-byte aligned.
__device__ __forceinline__ void tensor_load_3d(void *dst_shared, const CUtensorMap *map, int32_t x, int32_t y, int32_t z,
                                               uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_addr(dst_shared)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_addr(bar))
                 : "memory");
}

constexpr uint32_t kQkMaxSlots = 4u;
constexpr uint32_t kQkVRegs = 2u;  // 16-byte V chunks a thread carries across the token's barrier
constexpr uint32_t kQkStreamThreads = 896u;  // 28 warps: leaves 72 registers per thread

struct qk_stream_geom {
    uint32_t team_threads, teams, slots, slot_bytes;
};

// floats of one team's table area: two buffers of three D/2 tables, two 64-bit cache addresses
__host__ __device__ inline uint32_t qk_team_words(uint32_t D) { return (D / 2u) * 6u + 4u; }

__device__ __forceinline__ void team_sync(uint32_t team, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(team + 1u), "r"(threads) : "memory");
}

template <int LPH, int NPT, bool kFullRot>
__global__ void __launch_bounds__(kQkStreamThreads, 1)
qk_norm_rope_stream_kernel(const qk_dev_args a, const qk_stream_geom g, const __grid_constant__ CUtensorMap q_map) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t D = LPH * 8u;
    const uint32_t half = a.rope_dim >> 1;
    const uint32_t rot_lanes = a.rope_dim >> 3;
    const uint32_t q_bytes = a.q_heads * D * 2u, k_bytes = a.k_heads * D * 2u;
    const bool has_v = a.v != nullptr && a.v_pool != nullptr;
    const uint32_t v_chunks = a.k_heads * LPH;  // 16-byte chunks of a V row

    // [teams][slots][slot_bytes] | gq[D] gk[D] | per team: 2 x (cos, sin, -sin)[D/2], 2 cache addresses | barriers
    float *gq_sh = reinterpret_cast<float *>(smem + (size_t)g.teams * g.slots * g.slot_bytes);
    float *gk_sh = gq_sh + D;
    float *team_area = gk_sh + D;
    const uint32_t tid = threadIdx.x, team = tid / g.team_threads, t = tid % g.team_threads;
    // The last warp of a team is its manager: it owns no work items.  Its first lane drives the
    // bulk copies and the cache addressing, all its lanes compute the rotary tables.  Everything
    // that is serial by nature therefore runs beside the arithmetic warps, which only ever wait
    // for data and for each other.
    const uint32_t workers = g.team_threads - 32u;
    const bool manager = t >= workers;
    const bool lead = t == workers;
    float *tables = team_area + (size_t)team * qk_team_words(D);
    unsigned long long *v_base_sh = reinterpret_cast<unsigned long long *>(tables + (D / 2u) * 6u);  // [2], ~0 = none
    uint64_t *bars = reinterpret_cast<uint64_t *>(team_area + (size_t)g.teams * qk_team_words(D)) + team * kQkMaxSlots;
    uint8_t *my_slots = smem + (size_t)team * g.slots * g.slot_bytes;
    allow_dependents();
    dependency_wait();

    const bool fp8_cache = (a.flags & AXIOM_QK_FLAG_CACHE_E4M3) != 0u;
    // tokens of this CTA: blockIdx.x + n * gridDim.x; this team takes n = team + teams * i
    const uint32_t cta_tokens = a.tokens > blockIdx.x ? (a.tokens - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
    const uint32_t my_tokens = team < cta_tokens ? (cta_tokens - team + g.teams - 1u) / g.teams : 0u;
    auto token_of = [&](uint32_t i) { return blockIdx.x + (team + g.teams * i) * gridDim.x; };
    // With three or more slots the refill lags one token behind (the stores of the previous token
    // are the older bulk group: only they have to be done reading) and slots - 1 tokens are
    // requested up front; fewer slots are refilled as soon as their own stores have drained.
    const uint32_t ahead = g.slots > 2u ? g.slots - 1u : g.slots;
    // Requests token i into its slot; called by the whole manager warp.  A packed Q row is one copy.
    // When every head is followed by its gate values, the query halves of the token are one box of a
    // 3-D tensor map over (head_dim, heads at a pitch of two heads, tokens), which lands packed in
    // the slot; without a map the lanes fetch the heads one by one.  The slot holds the same packed
    // row in every case.
    const bool q_packed = a.q_head_stride == D;
    auto issue = [&](uint32_t i, uint32_t j, uint32_t lane) {  // j = i % slots
        const uint64_t tok = token_of(i);
        uint8_t *slot = my_slots + (size_t)j * g.slot_bytes;
        if (lane == 0u) {
            mbar_arrive_expect_tx(bars + j, q_bytes + k_bytes);
            if (q_bytes && q_packed) bulk_load(slot, reinterpret_cast<const uint8_t *>(a.q) + tok * q_bytes, q_bytes, bars + j);
            else if (q_bytes && a.q_use_map) tensor_load_3d(slot, &q_map, 0, 0, (int32_t)tok, bars + j);
            if (k_bytes) bulk_load(slot + q_bytes, reinterpret_cast<const uint8_t *>(a.k) + tok * k_bytes, k_bytes, bars + j);
        }
        if (!q_packed && !a.q_use_map) {
            __syncwarp();
            const uint8_t *row = reinterpret_cast<const uint8_t *>(a.q) + tok * a.q_heads * a.q_head_stride * 2u;
            for (uint32_t h = lane; h < a.q_heads; h += 32u) {
                bulk_load(slot + h * D * 2u, row + (size_t)h * a.q_head_stride * 2u, D * 2u, bars + j);
            }
        }
    };

    // the first tokens are requested before anything else is set up: nobody else touches the
    // barriers or the slots until the CTA barrier below
    if (manager) {
        if (lead) {
            for (uint32_t j = 0; j < g.slots; ++j) mbar_init(bars + j, 1u);
            mbar_init_fence();
        }
        __syncwarp();
        for (uint32_t i = 0; i < ahead && i < my_tokens; ++i) issue(i, i, t - workers);  // ahead <= slots
    }
    for (uint32_t i = tid; i < D; i += blockDim.x) {
        gq_sh[i] = a.q_heads ? __uint_as_float((uint32_t)a.q_gamma[i] << 16) : 0.0f;
        gk_sh[i] = a.k_heads ? __uint_as_float((uint32_t)a.k_gamma[i] << 16) : 0.0f;
    }
    __syncthreads();

    if (manager) {
        // ------------------------------------------------------------------ manager warp
        const uint32_t ml = t - workers;  // lane
        // table entry that maps a position's logical cache block (~0: outside the table)
        auto table_index = [&](uint32_t pos, uint32_t tok) -> uint64_t {
            uint32_t lb = pos / a.block_tokens;
            if (a.flags & AXIOM_QK_FLAG_RING) lb %= a.tbl_stride;
            else if (lb >= a.tbl_stride) return ~0ull;
            const uint64_t trow = (a.flags & AXIOM_QK_FLAG_PER_TOKEN_TABLE) ? tok : 0u;
            return trow * a.tbl_stride + lb;
        };
        auto write_table = [&](uint32_t buffer, uint32_t pos) {
            float *cos_t = tables + buffer * (D / 2u) * 3u, *sin_t = cos_t + D / 2u, *nsin_t = sin_t + D / 2u;
            for (uint32_t p = ml; p < half; p += 32u) {
                float cv, sv;
                rope_table_entry(pos, a.inv_freq[p], a.mscale, &cv, &sv);
                cos_t[p] = cv;
                sin_t[p] = sv;
                nsin_t[p] = -sv;
            }
        };
        // positions run two tokens ahead and block-table entries one (dependent loads off the critical path)
        const bool paged = a.k_pool != nullptr && lead;
        uint32_t pos_cur = my_tokens > 0u ? a.positions[token_of(0u)] : 0u;
        uint32_t pos_n1 = my_tokens > 1u ? a.positions[token_of(1u)] : 0u;
        int32_t pb_cur = -1;  // physical block of the current token, -1 = none
        if (paged && my_tokens > 0u) {
            const uint64_t idx = table_index(pos_cur, token_of(0u));
            if (idx != ~0ull) pb_cur = a.block_tables[idx];
        }
        if (my_tokens > 0u) write_table(0u, pos_cur);
        team_sync(team, g.team_threads);

        bool faulted = false;
        // slot of token i and the parity of its barrier (i % slots, (i / slots) & 1), and the slot of token i + ahead,
        // all advanced by one per token instead of divided out
        uint32_t j = 0u, phase = 0u, j_next = ahead % g.slots;
        for (uint32_t i = 0; i < my_tokens; ++i) {
            const uint32_t tok = token_of(i);
            const uint32_t pos_n2 = i + 2u < my_tokens ? a.positions[token_of(i + 2u)] : 0u;
            int32_t pb_n1 = -1;
            if (paged && i + 1u < my_tokens) {
                const uint64_t idx = table_index(pos_n1, token_of(i + 1u));
                if (idx != ~0ull) pb_n1 = a.block_tables[idx];
            }
            if (i + 1u < my_tokens) write_table((i + 1u) & 1u, pos_n1);
            const bool in_pool = pb_cur >= 0 && (uint32_t)pb_cur < a.n_blocks;
            const uint64_t row_index = (((uint64_t)(in_pool ? pb_cur : 0) * a.n_layers + a.layer) * a.block_tokens +
                                        pos_cur % a.block_tokens) * a.pool_stride;  // element index in the pools
            if (lead && (has_v || fp8_cache)) v_base_sh[i & 1u] = in_pool ? row_index : ~0ull;
            uint8_t *slot = my_slots + (size_t)j * g.slot_bytes;
            // A wait that ran out raises the fault word; the team carries on (on whatever the slot
            // holds) so that its barriers stay matched, and stops waiting and storing.
            if (!faulted && !mbar_wait(bars + j, phase)) faulted = true;
            faulted = __any_sync(0xffffffffu, faulted);  // one verdict for the warp: its lanes issue copies together
            team_sync(team, g.team_threads);  // the workers have rewritten the slot
            if (fp8_cache && g.slots <= 2u) team_sync(team, g.team_threads);  // ... and converted its K row (see the workers)

            const uint32_t nxt = i + ahead;
            if (lead && !faulted) {
                const uint8_t *src = slot;
                if (q_bytes) bulk_store(reinterpret_cast<uint8_t *>(a.q_out) + (uint64_t)tok * q_bytes, src, q_bytes);
                if (k_bytes && a.k_out) bulk_store(reinterpret_cast<uint8_t *>(a.k_out) + (uint64_t)tok * k_bytes, src + q_bytes, k_bytes);
                if (a.k_pool) {
                    if (in_pool) {
                        if (k_bytes && !fp8_cache) bulk_store(reinterpret_cast<uint8_t *>(a.k_pool) + row_index * 2u, src + q_bytes, k_bytes);
                    } else if (a.status_word) {
                        atomicCAS(a.status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
                    }
                }
                bulk_commit();
                if (nxt < my_tokens) {
                    if (g.slots > 2u) bulk_wait_read_but_one();
                    else bulk_wait_read_all();
                }
            }
            if (!faulted && nxt < my_tokens) {
                __syncwarp();  // the first lane's stores have finished reading the slot that is refilled
                issue(nxt, j_next, ml);
            }
            pos_cur = pos_n1;
            pos_n1 = pos_n2;
            pb_cur = pb_n1;
            if (++j == g.slots) {
                j = 0u;
                phase ^= 1u;
            }
            if (++j_next == g.slots) j_next = 0u;
        }
        if (lead) bulk_wait_read_all();
        return;
    }

    // ---------------------------------------------------------------------- worker warps
    const bool v_in_regs = v_chunks <= kQkVRegs * workers;
    const uint32_t l = t % LPH;
    const uint32_t head0 = t / LPH, head_step = workers / LPH;
    const bool rotary = kFullRot || l < rot_lanes;
    const uint32_t off_a = rotary ? 4u * l : a.rope_dim + 8u * (l - rot_lanes);
    const uint32_t off_b = rotary ? half + 4u * l : off_a + 4u;
    const double inv_d = 1.0 / (double)D, eps = (double)a.eps;
    // byte offset of this thread's first item inside a slot, and the step to its next item
    const uint32_t item0 = (head0 * D + off_a) * 2u, item_step = head_step * D * 2u, b_delta = (off_b - off_a) * 2u;
    team_sync(team, g.team_threads);  // the first rotary table is there

    bool faulted = false;
    uint32_t j = 0u, phase = 0u;  // i % slots and (i / slots) & 1
    for (uint32_t i = 0; i < my_tokens; ++i) {
        const uint32_t tok = token_of(i);
        // V is a plain copy into the token's cache row: too small to deserve slot space.  The
        // team's first threads read it now and write it after the barrier, when the manager has
        // published the row's address.
        uint4 v_reg[kQkVRegs];
        if (has_v && v_in_regs) {
#pragma unroll
            for (uint32_t c = 0; c < kQkVRegs; ++c) {
                const uint32_t q = t + c * workers;
                if (q < v_chunks) v_reg[c] = ld_stream(a.v + (uint64_t)tok * v_chunks + q);
            }
        }
        uint8_t *slot = my_slots + (size_t)j * g.slot_bytes;
        if (!faulted && !mbar_wait(bars + j, phase)) faulted = true;

        const float *cos_t = tables + (i & 1u) * (D / 2u) * 3u;
        const rot_regs r = load_rot(cos_t, cos_t + D / 2u, cos_t + D, off_a, rotary);
        // Sweep 1: the sum of squares of every item.  The inverse rms of a head is the same in all LPH lanes
        // that hold it, and a thread holds NPT heads: the lane sums are reduced so that head n's total lands in
        // one lane pair of the group, that lane evaluates the head's factor and the group reads it back by
        // shuffle, so the FP64 Newton step and its conversions run once per thread and token instead of once
        // per item.  Sweep 2 re-reads the slot (two 8-byte shared loads per
        // item, cheaper than keeping NPT items in registers across the exchange).
        float inv[NPT];
        {
            double ss[NPT];
            const uint8_t *item = slot + item0;
#pragma unroll
            for (int n = 0; n < NPT; ++n) {
                const uint2 xa = *reinterpret_cast<const uint2 *>(item), xb = *reinterpret_cast<const uint2 *>(item + b_delta);
                if constexpr (NPT <= LPH) ss[n] = lane_sum(xa, xb);
                else ss[n] = head_sum<LPH>(xa, xb);
                item += item_step;
            }
            if constexpr (NPT <= LPH) {
                const float inv_mine = inv_rms_from_sum(scatter_head_sums<LPH, NPT>(ss, l), inv_d, eps);
#pragma unroll
                for (int n = 0; n < NPT; ++n) inv[n] = __shfl_sync(0xffffffffu, inv_mine, n * (LPH / pow2_at_least<NPT>::value), LPH);
            } else {
#pragma unroll
                for (int n = 0; n < NPT; ++n) inv[n] = inv_rms_from_sum(ss[n], inv_d, eps);
            }
        }
        uint8_t *item = slot + item0;
        uint32_t h = head0;
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const float *gamma = h >= a.q_heads ? gk_sh : gq_sh;
            uint2 *pa_ptr = reinterpret_cast<uint2 *>(item);
            uint2 *pb_ptr = reinterpret_cast<uint2 *>(item + b_delta);
            const float4 ga = *reinterpret_cast<const float4 *>(gamma + off_a);
            const float4 gb = *reinterpret_cast<const float4 *>(gamma + off_b);
            uint2 pa, pb;
            qk_apply(*pa_ptr, *pb_ptr, inv[n], ga, gb, r, rotary, &pa, &pb);
            *pa_ptr = pa;
            *pb_ptr = pb;
            item += item_step;
            h += head_step;
        }
        fence_async_shared();
        team_sync(team, g.team_threads);

        if ((has_v || fp8_cache) && !faulted) {
            const unsigned long long v_base = v_base_sh[i & 1u];  // element index of the row in the pools
            if (v_base != ~0ull && has_v) {
                if (fp8_cache) {
                    uint2 *dst = reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(a.v_pool) + v_base);
                    if (v_in_regs) {
#pragma unroll
                        for (uint32_t c = 0; c < kQkVRegs; ++c) {
                            const uint32_t q = t + c * workers;
                            if (q < v_chunks) st_stream(dst + q, bf16x8_to_e4m3x8(v_reg[c]));
                        }
                    } else {
                        for (uint32_t q = t; q < v_chunks; q += workers) {
                            st_stream(dst + q, bf16x8_to_e4m3x8(ld_stream(a.v + (uint64_t)tok * v_chunks + q)));
                        }
                    }
                } else {
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(a.v_pool) + v_base);
                    if (v_in_regs) {
#pragma unroll
                        for (uint32_t c = 0; c < kQkVRegs; ++c) {
                            const uint32_t q = t + c * workers;
                            if (q < v_chunks) st_stream(dst + q, v_reg[c]);
                        }
                    } else {
                        for (uint32_t q = t; q < v_chunks; q += workers) {
                            st_stream(dst + q, ld_stream(a.v + (uint64_t)tok * v_chunks + q));
                        }
                    }
                }
            }
            if (fp8_cache && v_base != ~0ull && a.k_pool) {
                // the rotated K row sits in the slot as BF16 (it leaves as such for k_out): its E4M3
                // image for the cache is produced here, 8 values per thread
                const uint4 *k_sh = reinterpret_cast<const uint4 *>(slot + q_bytes);
                uint2 *dst = reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(a.k_pool) + v_base);
                for (uint32_t q = t; q < v_chunks; q += workers) st_stream(dst + q, bf16x8_to_e4m3x8(k_sh[q]));
            }
        }
        // with one or two slots the manager refills THIS slot next: everyone has to be done reading it
        if (fp8_cache && g.slots <= 2u) team_sync(team, g.team_threads);
        if (++j == g.slots) {
            j = 0u;
            phase ^= 1u;
        }
    }
}

// Frequency table.  The correction range (floor/ceil of the two YaRN
// correction dims) arrives from the host; powf and the blend run here so they
// use the same device math library as the kernels that used to evaluate them
// per thread (src/axiom_qwen38_attention.cu:98-116).
__global__ void yarn_inv_freq_kernel(float *out, uint32_t rope_dim, float theta, float factor, float low,
                                     float high, int yarn) {
    const uint32_t pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= rope_dim / 2u) return;
    const float dim = (float)rope_dim;
    if (!yarn) {
        out[pair] = powf(theta, __fdiv_rn(__fmul_rn(-2.0f, (float)pair), dim));
        return;
    }
    const float exponent = __fdiv_rn(__fmul_rn(2.0f, (float)pair), dim);
    const float inv = __fdiv_rn(1.0f, powf(theta, exponent));
    float ramp = high > low ? __fdiv_rn(__fsub_rn((float)pair, low), __fsub_rn(high, low))
                            : ((float)pair >= high ? 1.0f : 0.0f);
    ramp = fminf(1.0f, fmaxf(0.0f, ramp));
    out[pair] = __fmaf_rn(inv, __fsub_rn(1.0f, ramp), __fmul_rn(__fdiv_rn(inv, factor), ramp));
}

template <int LPH>
void launch_qk(const qk_dev_args &a, cudaStream_t stream) {
    const uint32_t items = (a.q_heads + a.k_heads) * LPH;
    const uint32_t grid = a.tokens;
    // items per thread: the count that wastes the fewest lanes, ties to the larger CTA
    uint32_t best_npt = 4u, best_threads = 0u, best_waste = ~0u;
    for (uint32_t npt = 2u; npt <= 8u; npt *= 2u) {
        for (uint32_t v = npt; v <= npt + (npt == 2u ? 1u : 0u); ++v) {  // 2, 3, 4, 8
            const uint32_t threads = ((items + v - 1u) / v + 31u) & ~31u;
            if (threads > 512u || threads < 32u) continue;
            const uint32_t waste = threads * v - items;
            if (waste < best_waste) { best_waste = waste; best_npt = v; best_threads = threads; }
        }
    }
    if (best_threads == 0u) { best_npt = 8u; best_threads = 512u; }
    const bool fast = best_waste == 0u && a.rope_dim == a.head_dim;
    const bool round_after_norm = (a.flags & AXIOM_QK_FLAG_ROUND_AFTER_NORM) != 0u;
#define AXB_QK_LAUNCH(NPT)                                                                              \
    do {                                                                                                 \
        if (round_after_norm) launch_chained(qk_norm_rope_paged_kernel<LPH, NPT, false, true>, dim3(grid), dim3(best_threads), 0, stream, a); \
        else if (fast) launch_chained(qk_norm_rope_paged_kernel<LPH, NPT, true>, dim3(grid), dim3(best_threads), 0, stream, a);  \
        else launch_chained(qk_norm_rope_paged_kernel<LPH, NPT, false>, dim3(grid), dim3(best_threads), 0, stream, a);           \
    } while (0)
    switch (best_npt) {
    case 2: AXB_QK_LAUNCH(2); break;
    case 3: AXB_QK_LAUNCH(3); break;
    case 4: AXB_QK_LAUNCH(4); break;
    default: AXB_QK_LAUNCH(8); break;
    }
#undef AXB_QK_LAUNCH
}

// Tensor map over the query halves of a q|gate-interleaved projection output: BF16, dimensions
// (head_dim, heads, tokens), a head pitch of two heads, box = (head_dim, heads, 1) = one token's
// packed Q row.  The driver's encoder is fetched through the runtime once; false (the kernel then
// falls back to one bulk copy per head) when it is missing or refuses the shape.
// The driver's cuTensorMapEncodeTiled, fetched through the runtime once per process (nullptr when it is missing).
void *tensor_map_encoder() {
    static void *const encoder = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            fn = nullptr;
        }
        return fn;
    }();
    return encoder;
}

bool encode_strided_q_map(const qk_dev_args &a, CUtensorMap *map) {
    using encode_fn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static const encode_fn encode = reinterpret_cast<encode_fn>(tensor_map_encoder());
    if (!encode || a.q_heads > 256u || a.head_dim > 256u || a.tokens > 0x7fffffffu) return false;
    const cuuint64_t dims[3] = {a.head_dim, a.q_heads, a.tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)a.q_head_stride * 2u, (cuuint64_t)a.q_heads * a.q_head_stride * 2u};  // bytes
    const cuuint32_t box[3] = {a.head_dim, a.q_heads, 1u};
    const cuuint32_t steps[3] = {1u, 1u, 1u};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3u, const_cast<uint4 *>(a.q), dims, strides, box, steps,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr size_t kQkSmemBudget = 227u * 1024u;

size_t qk_stream_smem(const qk_dev_args &a, const qk_stream_geom &g) {
    return (size_t)g.teams * g.slots * g.slot_bytes + 2u * a.head_dim * sizeof(float) +
           (size_t)g.teams * qk_team_words(a.head_dim) * sizeof(float) +
           (size_t)g.teams * kQkMaxSlots * sizeof(uint64_t);
}

// Picks the team shape of the streaming kernel; false when the problem does not fit it
// (work items do not divide evenly into whole warps, or fewer than three slots fit).
template <int LPH>
bool launch_qk_stream(const qk_dev_args &a, cudaStream_t stream) {
    const uint32_t items = (a.q_heads + a.k_heads) * LPH;
    qk_stream_geom best{};
    uint32_t best_npt = 0u, best_score = 0u;
    static const uint32_t kNpt[] = {2u, 3u, 4u, 6u, 8u, 9u};
    for (uint32_t npt : kNpt) {
        if (items % npt) continue;
        qk_stream_geom g{};
        const uint32_t workers = items / npt;
        if (workers % 32u || workers > 512u || workers < 64u) continue;
        g.team_threads = workers + 32u;  // plus the manager warp
        g.slot_bytes = (a.q_heads + a.k_heads) * a.head_dim * 2u;
        g.slots = 3u;
        g.teams = kQkStreamThreads / g.team_threads;
        while (g.teams != 0u && qk_stream_smem(a, g) > kQkSmemBudget) --g.teams;
        if (g.teams == 0u) continue;
        while (g.slots < kQkMaxSlots) {
            qk_stream_geom wider = g;
            ++wider.slots;
            if (qk_stream_smem(a, wider) > kQkSmemBudget) break;
            g = wider;
        }
        // most resident threads first, then the shape with more independent teams
        const uint32_t score = g.teams * g.team_threads * 16u + g.teams;
        if (score > best_score) { best_score = score; best = g; best_npt = npt; }
    }
    if (best_npt == 0u || best.teams == 0u) return false;
    // Two CTAs of half the teams per SM instead of one: the same threads, slots and registers, but a CTA of the next
    // launch on the stream becomes resident (and runs its set-up as far as the dependency wait) as soon as ONE of the
    // two finishes, instead of after the whole SM has drained (8192 tokens of 64 + 8 heads: 56.6 -> 56.4 us, with the
    // interleaved source 55.7 -> 55.0 us).
    uint32_t ctas_per_sm = 1u;
    if (best.teams >= 2u && best.teams % 2u == 0u) {
        qk_stream_geom half_geom = best;
        half_geom.teams = best.teams / 2u;
        if (2u * (qk_stream_smem(a, half_geom) + 1024u) <= 228u * 1024u) {
            best = half_geom;
            ctas_per_sm = 2u;
        }
    }
    const size_t smem = qk_stream_smem(a, best);
    const uint32_t ctas = std::min<uint32_t>(kSmCount * ctas_per_sm, (a.tokens + best.teams - 1u) / best.teams);
    const bool full = a.rope_dim == a.head_dim;
    qk_dev_args a2 = a;
    CUtensorMap q_map;
    memset(&q_map, 0, sizeof q_map);
    a2.q_use_map = a.q_heads != 0u && a.q_head_stride != a.head_dim && encode_strided_q_map(a, &q_map) ? 1u : 0u;
#define AXB_QK_STREAM(NPT)                                                                               \
    do {                                                                                                 \
        if (full) {                                                                                      \
            auto kern = qk_norm_rope_stream_kernel<LPH, NPT, true>;                                      \
            allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, NPT, true>>(kQkSmemBudget);               \
            launch_chained(kern, dim3(ctas), dim3(best.teams * best.team_threads), smem, stream, a2, best, q_map);               \
        } else {                                                                                         \
            auto kern = qk_norm_rope_stream_kernel<LPH, NPT, false>;                                     \
            allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, NPT, false>>(kQkSmemBudget);              \
            launch_chained(kern, dim3(ctas), dim3(best.teams * best.team_threads), smem, stream, a2, best, q_map);               \
        }                                                                                                \
    } while (0)
    switch (best_npt) {
    case 2: AXB_QK_STREAM(2); break;
    case 3: AXB_QK_STREAM(3); break;
    case 4: AXB_QK_STREAM(4); break;
    case 6: AXB_QK_STREAM(6); break;
    case 8: AXB_QK_STREAM(8); break;
    case 9: AXB_QK_STREAM(9); break;
    default: return false;
    }
#undef AXB_QK_STREAM
    return true;
}

template <int LPH>
void launch_qk_any(const qk_dev_args &a, cudaStream_t stream) {
    // The per-token kernel has the shortest latency; the streaming kernel the highest throughput.
    // (the BF16 rounding convention exists in the per-token kernel only)
    if (a.tokens >= 2u * kSmCount && !(a.flags & AXIOM_QK_FLAG_ROUND_AFTER_NORM) && launch_qk_stream<LPH>(a, stream)) return;
    launch_qk<LPH>(a, stream);
}

bool is_pow2(uint32_t v) { return v && !(v & (v - 1u)); }

}  // namespace

unsigned int qk_fault_word() { return read_and_clear_pipeline_fault(); }

namespace {
template <int LPH>
void prepare_qk_stream_kernels() {
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 2, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 2, false>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 3, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 3, false>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 4, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 4, false>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 6, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 6, false>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 8, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 8, false>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 9, true>>(kQkSmemBudget);
    allow_dynamic_smem<qk_norm_rope_stream_kernel<LPH, 9, false>>(kQkSmemBudget);
}
}  // namespace

// Everything a first launch would set up lazily, for axiom_b200_prepare().
void prepare_qk_unit() {
    prepare_qk_stream_kernels<8>();
    prepare_qk_stream_kernels<16>();
    prepare_qk_stream_kernels<32>();
    (void)tensor_map_encoder();
}

int launch_qk_norm_rope_paged_bf16(const axiom_qk_rope_args *p, cudaStream_t stream) {
    qk_dev_args a{};
    const bool has_q_out = p->struct_size >= offsetof(axiom_qk_rope_args, rope_table) && p->q_out_bf16 != nullptr;
    if (p->struct_size >= sizeof(axiom_qk_rope_args)) {
        a.rope_table = p->rope_table;
        a.rope_table_positions = p->rope_table_positions;
    }
    a.q = (const uint4 *)p->q_bf16;
    a.q_out = has_q_out ? (uint4 *)p->q_out_bf16 : (uint4 *)p->q_bf16;
    a.q_head_stride = (p->flags & AXIOM_QK_FLAG_Q_GATE_INTERLEAVED) ? 2u * p->head_dim : p->head_dim;
    a.k = (const uint4 *)p->k_bf16;
    a.v = (const uint4 *)p->v_bf16;
    a.q_gamma = (const uint16_t *)p->q_gamma_bf16;
    a.k_gamma = (const uint16_t *)p->k_gamma_bf16;
    a.inv_freq = p->inv_freq;
    a.positions = p->positions;
    a.block_tables = p->block_tables;
    a.k_pool = (uint4 *)p->k_pool_bf16;
    a.v_pool = (uint4 *)p->v_pool_bf16;
    a.k_out = (uint4 *)p->k_out_bf16;
    a.status_word = p->status_word;
    a.tokens = p->tokens; a.q_heads = p->q_heads; a.k_heads = p->k_heads; a.head_dim = p->head_dim;
    a.rope_dim = p->rope_dim; a.flags = p->flags; a.eps = p->eps; a.mscale = p->mscale;
    a.block_tokens = p->block_tokens; a.n_layers = p->n_layers; a.layer = p->layer;
    a.pool_stride = p->pool_stride; a.tbl_stride = p->tbl_stride; a.n_blocks = p->n_blocks;
    switch (p->head_dim) {
    case 64: launch_qk_any<8>(a, stream); break;
    case 128: launch_qk_any<16>(a, stream); break;
    default: launch_qk_any<32>(a, stream); break;
    }
    note_launch();
    return AXIOM_OK;
}

int launch_yarn_inv_freq(const axiom_rope_config *c, float *out, cudaStream_t stream) {
    const int yarn = c->factor > 1.0f;
    float low = 0.0f, high = 0.0f;
    if (yarn) {
        // Same FP32 expression as the reference evaluates with compile-time constants.
        const float dim = (float)c->rope_dim;
        const float fast = dim * logf(c->original_context / (c->beta_fast * 6.283185307179586f)) / (2.0f * logf(c->theta));
        const float slow = dim * logf(c->original_context / (c->beta_slow * 6.283185307179586f)) / (2.0f * logf(c->theta));
        low = floorf(fast < slow ? fast : slow);
        high = ceilf(fast > slow ? fast : slow);
    }
    const uint32_t pairs = c->rope_dim / 2u;
    yarn_inv_freq_kernel<<<(pairs + 127u) / 128u, 128, 0, stream>>>(out, c->rope_dim, c->theta, c->factor, low, high, yarn);
    note_launch();
    return AXIOM_OK;
}

}  // namespace axb

using namespace axb;

extern "C" float axiom_qwen38_fused_yarn_mscale(float factor) {
    if (!(factor > 1.0f)) return 1.0f;
    return (float)(0.1 * std::log((double)factor) + 1.0);
}

extern "C" int axiom_qwen38_fused_yarn_inv_freq_device(int device, const axiom_rope_config *config,
                                                       float *out_inv_freq, void *stream) {
    if (!config || !out_inv_freq || config->abi_version != AXIOM_ABI_VERSION || config->rope_dim == 0u ||
        (config->rope_dim & 1u) || config->rope_dim > kMaxHeadDim || !(config->theta > 1.0f) ||
        !std::isfinite(config->theta)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (config->factor > 1.0f &&
        (!(config->original_context > 0.0f) || !(config->beta_fast > 0.0f) || !(config->beta_slow > 0.0f))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_yarn_inv_freq(config, out_inv_freq, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_qk_norm_rope_paged_bf16_device(int device, const axiom_qk_rope_args *p,
                                                                 void *stream) {
    // the struct has grown twice by appending: every earlier size is accepted, the missing members read as NULL / 0
    if (!p || p->abi_version != AXIOM_ABI_VERSION ||
        (p->struct_size != sizeof(axiom_qk_rope_args) && p->struct_size != offsetof(axiom_qk_rope_args, rope_table) &&
         p->struct_size != offsetof(axiom_qk_rope_args, q_out_bf16))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    void *const q_out = p->struct_size >= offsetof(axiom_qk_rope_args, rope_table) ? p->q_out_bf16 : nullptr;
    const float *const rope_table = p->struct_size == sizeof(axiom_qk_rope_args) ? p->rope_table : nullptr;
    if (p->flags & AXIOM_QK_FLAG_ROUND_AFTER_NORM) {
        // the BF16 convention is defined for full-head rotation; its cos/sin come from the table when one is given
        if (p->rope_dim != p->head_dim || p->rope_dim == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
        if (rope_table && (p->rope_table_positions == 0u || (reinterpret_cast<uintptr_t>(rope_table) & 3u))) return AXIOM_ERR_INVALID_ARGUMENT;
    } else if (rope_table) {
        return AXIOM_ERR_INVALID_ARGUMENT;  // the table belongs to the BF16 convention
    }
    if (q_out && (!p->q_heads || !aligned16(q_out))) return AXIOM_ERR_INVALID_ARGUMENT;
    if ((p->flags & AXIOM_QK_FLAG_Q_GATE_INTERLEAVED) && (!p->q_heads || !q_out)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (p->tokens == 0u || (p->q_heads + p->k_heads) == 0u || (p->q_heads + p->k_heads) > kMaxHeads ||
        (uint64_t)(p->q_heads + p->k_heads) * (p->head_dim / 8u) > 4096u ||
        (p->head_dim != 64u && p->head_dim != 128u && p->head_dim != 256u) || p->rope_dim > p->head_dim ||
        (p->rope_dim != 0u && (!is_pow2(p->rope_dim) || p->rope_dim < 16u)) || !(p->eps > 0.0f) ||
        !std::isfinite(p->eps) || !std::isfinite(p->mscale) || !p->positions) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (p->rope_dim != 0u && !p->inv_freq && !rope_table) return AXIOM_ERR_INVALID_ARGUMENT;
    if (p->q_heads && (!p->q_bf16 || !p->q_gamma_bf16 || !aligned16(p->q_bf16))) return AXIOM_ERR_INVALID_ARGUMENT;
    if (p->k_heads && (!p->k_bf16 || !p->k_gamma_bf16 || !aligned16(p->k_bf16))) return AXIOM_ERR_INVALID_ARGUMENT;
    if (p->k_heads && !p->k_pool_bf16 && !p->k_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (p->k_pool_bf16) {
        if (!p->block_tables || p->block_tokens == 0u || p->n_layers == 0u || p->layer >= p->n_layers ||
            p->tbl_stride == 0u || p->n_blocks == 0u || p->pool_stride < p->k_heads * p->head_dim ||
            (p->pool_stride % 8u) != 0u || !aligned16(p->k_pool_bf16)) {
            return AXIOM_ERR_INVALID_ARGUMENT;
        }
        if ((p->v_bf16 == nullptr) != (p->v_pool_bf16 == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
        if (p->v_bf16 && (!aligned16(p->v_bf16) || !aligned16(p->v_pool_bf16))) return AXIOM_ERR_INVALID_ARGUMENT;
    } else if (p->v_bf16 || p->v_pool_bf16) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (p->k_out_bf16 && !aligned16(p->k_out_bf16)) return AXIOM_ERR_INVALID_ARGUMENT;
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_qk_norm_rope_paged_bf16(p, (cudaStream_t)stream);
    return launch_status();
}

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
// One CTA per token.  A lane owns BOTH members of four NeoX pairs: dims 4l..4l+3 and
// rope_dim/2 + 4l.. of one head (two 8-byte accesses; a warp still reads whole 128-byte
// lines), so the rotation needs no lane exchange, no select and no divergent branch.
// Lanes past the rotary dims carry 8 pass-through dims.  head_dim/8 adjacent lanes form a
// head.  Three phases separated by CTA barriers keep the scalar work out of the replicated
// lane code:
//   1. load, FP64 sum of squares per head (shuffle tree) -> shared
//   2. one thread per head: inv; one thread per (pair, cos|sin): table row (cos, sin, -sin)
//   3. normalise, rotate, round, store (packed F32x2 arithmetic)
// The frequency table is an input: it is evaluated once per model on the device
// (yarn_inv_freq_kernel) instead of powf/logf per thread per call.
#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {


constexpr uint32_t kMaxHeads = 512u;
constexpr uint32_t kMaxHeadDim = 256u;

struct qk_dev_args {
    uint4 *q;
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
};

__device__ __forceinline__ uint2 ld_stream8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// LPH = lanes per head (head_dim / 8); NPT = (head, lane) work items per thread.
// kFast: every thread's NPT items exist and every lane carries rotary pairs (full-head
// rotation), which removes the bounds predicates and the pass-through branch.
template <int LPH, int NPT, bool kFast>
__global__ void __launch_bounds__(512, NPT <= 4 ? 2 : 1)
qk_norm_rope_paged_kernel(const qk_dev_args a) {
    __shared__ double ss_sh[kMaxHeads];
    __shared__ float inv_sh[kMaxHeads];
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

    for (uint32_t i = tid; i < D; i += blockDim.x) {
        gq_sh[i] = a.q_heads ? __uint_as_float((uint32_t)a.q_gamma[i] << 16) : 0.0f;
        gk_sh[i] = a.k_heads ? __uint_as_float((uint32_t)a.k_gamma[i] << 16) : 0.0f;
    }

    // Work item n of this thread is (head tid/LPH + n*blockDim/LPH, lane tid%LPH): blockDim is a
    // multiple of 32 and LPH divides 32, so the lane geometry is the same for every item and
    // everything below is fixed across tokens.
    const uint32_t l = tid % LPH;
    const uint32_t head0 = tid / LPH, head_step = blockDim.x / LPH;
    const bool rotary = kFast || l < rot_lanes;
    const uint32_t off_a = rotary ? 4u * l : a.rope_dim + 8u * (l - rot_lanes);
    const uint32_t off_b = rotary ? half + 4u * l : off_a + 4u;
    const uint32_t q_elems = a.q_heads * D, k_elems = a.k_heads * D;
    // element offset of item n inside the token's Q row (heads < q_heads) or K row
    uint32_t item_off[NPT];
#pragma unroll
    for (int n = 0; n < NPT; ++n) {
        const uint32_t h = head0 + head_step * n;
        item_off[n] = (h < a.q_heads ? h : h - a.q_heads) * D;
    }
    __syncthreads();

    for (uint32_t t = blockIdx.x; t < a.tokens; t += gridDim.x) {
        uint16_t *q_row = reinterpret_cast<uint16_t *>(a.q) + (uint64_t)t * q_elems;
        const uint16_t *k_row = reinterpret_cast<const uint16_t *>(a.k) + (uint64_t)t * k_elems;

        // ---- phase 1: loads and per-head FP64 sum of squares
        uint2 xa[NPT], xb[NPT];
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const uint32_t h = head0 + head_step * n;
            xa[n] = make_uint2(0u, 0u);
            xb[n] = make_uint2(0u, 0u);
            if (kFast || h < heads) {
                const uint16_t *row = (h < a.q_heads ? q_row : k_row) + item_off[n];
                xa[n] = ld_stream8(row + off_a);
                xb[n] = ld_stream8(row + off_b);
            }
        }
        const uint32_t pos = a.positions[t];
        if (tid == 0u) {
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
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const float f[8] = {bf16_lo(xa[n].x), bf16_hi(xa[n].x), bf16_lo(xa[n].y), bf16_hi(xa[n].y),
                                bf16_lo(xb[n].x), bf16_hi(xb[n].x), bf16_lo(xb[n].y), bf16_hi(xb[n].y)};
            double s = 0.0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const double d = (double)f[i];
                s = __fma_rn(d, d, s);
            }
#pragma unroll
            for (int off = LPH / 2; off != 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            const uint32_t h = head0 + head_step * n;
            if (l == 0u && (kFast || h < heads)) ss_sh[h] = s;
        }
        __syncthreads();

        // ---- phase 2: one thread per head / per table entry
        for (uint32_t e = tid; e < heads + a.rope_dim; e += blockDim.x) {
            if (e < heads) {
                inv_sh[e] = (float)(1.0 / sqrt(ss_sh[e] / (double)D + (double)a.eps));
            } else {
                const uint32_t idx = e - heads;
                const uint32_t p = idx < half ? idx : idx - half;
                const float angle = __fmul_rn((float)pos, a.inv_freq[p]);
                if (idx < half) {
                    cos_sh[p] = __fmul_rn(cosf(angle), a.mscale);
                } else {
                    const float sv = __fmul_rn(sinf(angle), a.mscale);
                    sin_sh[p] = sv;
                    nsin_sh[p] = -sv;
                }
            }
        }
        __syncthreads();

        // ---- phase 3: normalise, rotate, round, store
        const unsigned long long kv_base = kv_base_sh;
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f), sn = c, ns = c;
        if (rotary) {
            c = *reinterpret_cast<const float4 *>(cos_sh + off_a);
            sn = *reinterpret_cast<const float4 *>(sin_sh + off_a);
            ns = *reinterpret_cast<const float4 *>(nsin_sh + off_a);
        }
        const float2 c0 = make_float2(c.x, c.y), c1 = make_float2(c.z, c.w);
        const float2 s0 = make_float2(sn.x, sn.y), s1 = make_float2(sn.z, sn.w);
        const float2 n0 = make_float2(ns.x, ns.y), n1 = make_float2(ns.z, ns.w);
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const uint32_t h = head0 + head_step * n;
            const bool is_k = h >= a.q_heads;
            const float *gamma = is_k ? gk_sh : gq_sh;
            const float inv = inv_sh[(kFast || h < heads) ? h : 0u];
            const float2 inv2 = make_float2(inv, inv);
            const float4 ga = *reinterpret_cast<const float4 *>(gamma + off_a);
            const float4 gb = *reinterpret_cast<const float4 *>(gamma + off_b);
            // n = (x * inv) * gamma
            const float2 a0 = __fmul2_rn(__fmul2_rn(make_float2(bf16_lo(xa[n].x), bf16_hi(xa[n].x)), inv2), make_float2(ga.x, ga.y));
            const float2 a1 = __fmul2_rn(__fmul2_rn(make_float2(bf16_lo(xa[n].y), bf16_hi(xa[n].y)), inv2), make_float2(ga.z, ga.w));
            const float2 b0 = __fmul2_rn(__fmul2_rn(make_float2(bf16_lo(xb[n].x), bf16_hi(xb[n].x)), inv2), make_float2(gb.x, gb.y));
            const float2 b1 = __fmul2_rn(__fmul2_rn(make_float2(bf16_lo(xb[n].y), bf16_hi(xb[n].y)), inv2), make_float2(gb.z, gb.w));
            float2 oa0 = a0, oa1 = a1, ob0 = b0, ob1 = b1;
            if (rotary) {
                // out[p] = fma(first, c, -(second*s)); out[p+half] = fma(first, s, second*c)
                oa0 = __ffma2_rn(a0, c0, __fmul2_rn(b0, n0));
                oa1 = __ffma2_rn(a1, c1, __fmul2_rn(b1, n1));
                ob0 = __ffma2_rn(a0, s0, __fmul2_rn(b0, c0));
                ob1 = __ffma2_rn(a1, s1, __fmul2_rn(b1, c1));
            }
            const uint2 pa = make_uint2(pack_bf16x2(oa0.x, oa0.y), pack_bf16x2(oa1.x, oa1.y));
            const uint2 pb = make_uint2(pack_bf16x2(ob0.x, ob0.y), pack_bf16x2(ob1.x, ob1.y));
            if (kFast || h < heads) {
                if (!is_k) {
                    uint16_t *dst = q_row + item_off[n];
                    st_stream(dst + off_a, pa);
                    st_stream(dst + off_b, pb);
                } else {
                    if (kv_base != ~0ull) {
                        uint16_t *dst = reinterpret_cast<uint16_t *>(a.k_pool) + kv_base + item_off[n];
                        st_stream(dst + off_a, pa);
                        st_stream(dst + off_b, pb);
                    }
                    if (a.k_out) {
                        uint16_t *dst = reinterpret_cast<uint16_t *>(a.k_out) + (uint64_t)t * k_elems + item_off[n];
                        st_stream(dst + off_a, pa);
                        st_stream(dst + off_b, pb);
                    }
                }
            }
        }
        // V rides along unchanged (BF16 in, BF16 cache)
        if (a.v && a.v_pool && kv_base != ~0ull) {
            const uint4 *v_row = a.v + (uint64_t)t * a.k_heads * LPH;
            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(a.v_pool) + kv_base);
            for (uint32_t j = tid; j < a.k_heads * LPH; j += blockDim.x) st_stream(dst + j, ld_stream(v_row + j));
        }
        __syncthreads();  // shared tables are rewritten by the next token
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
#define AXB_QK_LAUNCH(NPT)                                                                              \
    do {                                                                                                 \
        if (fast) qk_norm_rope_paged_kernel<LPH, NPT, true><<<grid, best_threads, 0, stream>>>(a);       \
        else qk_norm_rope_paged_kernel<LPH, NPT, false><<<grid, best_threads, 0, stream>>>(a);           \
    } while (0)
    switch (best_npt) {
    case 2: AXB_QK_LAUNCH(2); break;
    case 3: AXB_QK_LAUNCH(3); break;
    case 4: AXB_QK_LAUNCH(4); break;
    default: AXB_QK_LAUNCH(8); break;
    }
#undef AXB_QK_LAUNCH
}

bool is_pow2(uint32_t v) { return v && !(v & (v - 1u)); }

}  // namespace

unsigned int qk_fault_word() { return read_and_clear_pipeline_fault(); }

int launch_qk_norm_rope_paged_bf16(const axiom_qk_rope_args *p, cudaStream_t stream) {
    qk_dev_args a{};
    a.q = (uint4 *)p->q_bf16;
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
    case 64: launch_qk<8>(a, stream); break;
    case 128: launch_qk<16>(a, stream); break;
    default: launch_qk<32>(a, stream); break;
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
    if (!p || p->abi_version != AXIOM_ABI_VERSION || p->struct_size != sizeof(axiom_qk_rope_args)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (p->tokens == 0u || (p->q_heads + p->k_heads) == 0u || (p->q_heads + p->k_heads) > kMaxHeads ||
        (uint64_t)(p->q_heads + p->k_heads) * (p->head_dim / 8u) > 4096u ||
        (p->head_dim != 64u && p->head_dim != 128u && p->head_dim != 256u) || p->rope_dim > p->head_dim ||
        (p->rope_dim != 0u && (!is_pow2(p->rope_dim) || p->rope_dim < 16u)) || !(p->eps > 0.0f) ||
        !std::isfinite(p->eps) || !std::isfinite(p->mscale) || !p->positions) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (p->rope_dim != 0u && !p->inv_freq) return AXIOM_ERR_INVALID_ARGUMENT;
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

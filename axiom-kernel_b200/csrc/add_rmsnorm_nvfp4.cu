// Residual add + RMSNorm (+ NVFP4 quantize) in one pass over HBM.
//
// Arithmetic of qwen38_add_bf16_rmsnorm8_kernel / qwen38_rmsnorm_bf16_8_kernel
// (src/axiom_qwen38_model.cu:190-292) followed by the activation quantizer
// (src/axiom_qwen38_nvfp4_mlp.cu:144-223), including the reference's FP32
// summation order: 256 partial sums over features (c + 256*k) accumulated with
// fmaf in k order, then the tree 128/64/32/16/8/4/2/1.
//
// Throughput kernel: ONE WARP PER ROW.  Lane u loads the 16-byte chunks
// u + 32*k, so each warp-wide load is 512 contiguous bytes, and the 8 values
// of a lane's chunk are exactly partial sums 8u..8u+7 of the reference order:
// the fmaf chains run along k in registers and the tree is a shuffle
// butterfly (16,8,4 lanes = strides 128,64,32; 2,1 lanes = strides 16,8;
// strides 4,2,1 inside the lane).  The merged row stays in registers as packed
// BF16 (it is BF16-valued by construction) for the second sweep.
//
// Latency kernel: one 256-thread CTA per row for small token counts.
#include "runtime.hpp"

namespace axb {

namespace {

__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    x[0] = bf16_lo(v.x); x[1] = bf16_hi(v.x);
    x[2] = bf16_lo(v.y); x[3] = bf16_hi(v.y);
    x[4] = bf16_lo(v.z); x[5] = bf16_hi(v.z);
    x[6] = bf16_lo(v.w); x[7] = bf16_hi(v.w);
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    return make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                      pack_bf16x2(x[6], x[7]));
}

__device__ __forceinline__ uint4 ld_cached(const void *p) { return *reinterpret_cast<const uint4 *>(p); }

struct norm_args {
    const uint4 *hidden;    // may be null
    uint4 *residual;        // read; rewritten when hidden != null
    const uint4 *gamma;
    uint4 *norm_out;        // may be null
    uint32_t *codes;        // may be null
    uint8_t *scales;
    float eps;
    float G;
    uint32_t rows;
    uint32_t cols;
    uint32_t chunks_per_row;
    uint32_t layout;
    uint32_t groups;
    uint32_t inner_tiles;
};

constexpr uint32_t kWarpsPerCta = 4u;

template <int NCH, bool kAdd>
__global__ void __launch_bounds__(kWarpsPerCta * 32u)
add_rmsnorm_warp_rows_kernel(const norm_args a) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const uint32_t warps = gridDim.x * kWarpsPerCta;
    const float count = (float)a.cols;

    for (uint32_t row = warp; row < a.rows; row += warps) {
        const uint64_t base = (uint64_t)row * a.chunks_per_row;
        uint4 m[NCH];  // merged row, packed BF16
        if (kAdd) {
            uint4 h[NCH];
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const uint32_t q = lane + 32u * k;
                const bool ok = q < a.chunks_per_row;
                h[k] = ok ? ld_stream(a.hidden + base + q) : make_uint4(0u, 0u, 0u, 0u);
                m[k] = ok ? ld_stream(a.residual + base + q) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                float x[8], y[8];
                unpack8(h[k], x);
                unpack8(m[k], y);
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = __fadd_rn(y[i], x[i]);
                m[k] = pack8(y);  // bf16(bf16(res) + bf16(add)): inputs are BF16 already
                const uint32_t q = lane + 32u * k;
                if (q < a.chunks_per_row) st_stream(a.residual + base + q, m[k]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const uint32_t q = lane + 32u * k;
                m[k] = q < a.chunks_per_row ? ld_stream(a.residual + base + q) : make_uint4(0u, 0u, 0u, 0u);
            }
        }

        float p[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            float y[8];
            unpack8(m[k], y);
#pragma unroll
            for (int i = 0; i < 8; ++i) p[i] = __fmaf_rn(y[i], y[i], p[i]);
        }
#pragma unroll
        for (uint32_t off = 16u; off != 0u; off >>= 1u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) p[i] = __fadd_rn(p[i], __shfl_xor_sync(0xffffffffu, p[i], off));
        }
        const float s4[4] = {__fadd_rn(p[0], p[4]), __fadd_rn(p[1], p[5]), __fadd_rn(p[2], p[6]), __fadd_rn(p[3], p[7])};
        const float total = __fadd_rn(__fadd_rn(s4[0], s4[2]), __fadd_rn(s4[1], s4[3]));
        const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(total, count), a.eps));

#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const uint32_t q = lane + 32u * k;
            const bool ok = q < a.chunks_per_row;
            float y[8], w[8];
            unpack8(m[k], y);
            unpack8(ok ? ld_cached(a.gamma + q) : make_uint4(0u, 0u, 0u, 0u), w);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(__fmul_rn(y[i], inverse), w[i]);
            const uint4 n = pack8(y);
            if (a.norm_out && ok) st_stream(a.norm_out + base + q, n);
            if (a.codes) {
                unpack8(n, y);  // the quantizer sees the BF16-rounded values
                float mx = fmaxf(fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3]))),
                                 fmaxf(fmaxf(fabsf(y[4]), fabsf(y[5])), fmaxf(fabsf(y[6]), fabsf(y[7]))));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, 0.0f);
                uint32_t scale_code;
                const uint32_t packed = nvfp4_quantize8(y, mx, a.G, &scale_code);
                if (ok) {
                    st_stream(a.codes + base + q, packed);
                    if ((lane & 1u) == 0u) {
                        a.scales[scale_offset(row, q >> 1, a.groups, a.inner_tiles, a.layout)] = (uint8_t)scale_code;
                    }
                }
            }
        }
    }
}

// One CTA per row, thread t owns features t + 256*k (the reference's own
// thread/feature assignment), merged row kept in shared memory as BF16.
constexpr uint32_t kCtaThreads = 256u;

__global__ void __launch_bounds__(kCtaThreads)
add_rmsnorm_cta_rows_kernel(const norm_args a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint16_t *merged = reinterpret_cast<uint16_t *>(smem_raw);  // [cols]
    __shared__ float sums[kCtaThreads];
    const uint32_t tid = threadIdx.x;
    const uint16_t *hidden = reinterpret_cast<const uint16_t *>(a.hidden);
    uint16_t *residual = reinterpret_cast<uint16_t *>(a.residual);
    const uint16_t *gamma = reinterpret_cast<const uint16_t *>(a.gamma);
    uint16_t *norm_out = reinterpret_cast<uint16_t *>(a.norm_out);
    uint8_t *codes = reinterpret_cast<uint8_t *>(a.codes);

    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const uint64_t base = (uint64_t)row * a.cols;
        float sum = 0.0f;
        for (uint32_t f = tid; f < a.cols; f += kCtaThreads) {
            float r = __uint_as_float((uint32_t)residual[base + f] << 16);
            uint16_t bits = residual[base + f];
            if (hidden) {
                r = __fadd_rn(r, __uint_as_float((uint32_t)hidden[base + f] << 16));
                bits = (uint16_t)(pack_bf16x2(r, 0.0f) & 0xffffu);
                r = __uint_as_float((uint32_t)bits << 16);
                residual[base + f] = bits;
            }
            merged[f] = bits;
            sum = __fmaf_rn(r, r, sum);
        }
        sums[tid] = sum;
        __syncthreads();
        for (uint32_t stride = kCtaThreads / 2u; stride >= 32u; stride >>= 1u) {
            if (tid < stride) sums[tid] = __fadd_rn(sums[tid], sums[tid + stride]);
            __syncthreads();
        }
        if (tid < 32u) {
            float total = sums[tid];
#pragma unroll
            for (uint32_t stride = 16u; stride != 0u; stride >>= 1u) {
                total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, stride));
            }
            if (tid == 0u) sums[0] = total;
        }
        __syncthreads();
        const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(sums[0], (float)a.cols), a.eps));
        // cols % 16 == 0, so all 16 lanes of a block are in range together
        for (uint32_t f0 = 0; f0 < a.cols; f0 += kCtaThreads) {
            const uint32_t f = f0 + tid;
            const bool ok = f < a.cols;
            float n = 0.0f;
            if (ok) {
                const float r = __uint_as_float((uint32_t)merged[f] << 16);
                const float w = __uint_as_float((uint32_t)gamma[f] << 16);
                const uint16_t bits = (uint16_t)(pack_bf16x2(__fmul_rn(__fmul_rn(r, inverse), w), 0.0f) & 0xffffu);
                if (norm_out) norm_out[base + f] = bits;
                n = __uint_as_float((uint32_t)bits << 16);
            }
            if (codes) {
                float mx = fabsf(n);
#pragma unroll
                for (uint32_t off = 8u; off != 0u; off >>= 1u) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                mx = fmaxf(mx, 0.0f);
                const uint32_t scale_code = encode_block_scale(__fmul_rn(__fmul_rn(mx, 1.0f / 6.0f), a.G));
                const float d = __fdiv_rn(e4m3_to_f32(scale_code), a.G);
                const float qv = __fdiv_rn(n, d);
                const float next = __shfl_down_sync(0xffffffffu, qv, 1);
                if (ok && (tid & 1u) == 0u) {
                    codes[(base + f) >> 1] = (uint8_t)(cvt_e2m1x2(qv, next) & 0xffu);
                    if ((tid & 15u) == 0u) {
                        a.scales[scale_offset(row, f >> 4, a.groups, a.inner_tiles, a.layout)] = (uint8_t)scale_code;
                    }
                }
            }
        }
        __syncthreads();
    }
}

template <int NCH>
void launch_warp_rows(const norm_args &a, cudaStream_t stream) {
    uint32_t ctas = (a.rows + kWarpsPerCta - 1u) / kWarpsPerCta;
    const uint32_t cap = kSmCount * 4u;
    if (ctas > cap) ctas = cap;
    if (a.hidden) add_rmsnorm_warp_rows_kernel<NCH, true><<<ctas, kWarpsPerCta * 32u, 0, stream>>>(a);
    else add_rmsnorm_warp_rows_kernel<NCH, false><<<ctas, kWarpsPerCta * 32u, 0, stream>>>(a);
}

}  // namespace

int launch_add_rmsnorm_nvfp4_bf16(const void *hidden, void *residual, const void *gamma, float eps, uint32_t rows,
                                  uint32_t cols, float G, void *norm_out, uint8_t *codes, uint8_t *scales,
                                  uint32_t layout, cudaStream_t stream) {
    norm_args a{};
    a.hidden = (const uint4 *)hidden;
    a.residual = (uint4 *)residual;
    a.gamma = (const uint4 *)gamma;
    a.norm_out = (uint4 *)norm_out;
    a.codes = (uint32_t *)codes;
    a.scales = scales;
    a.eps = eps;
    a.G = G;
    a.rows = rows;
    a.cols = cols;
    a.chunks_per_row = cols / 8u;
    a.layout = layout;
    a.groups = cols / kGroup;
    a.inner_tiles = (a.groups + 3u) / 4u;

    const uint32_t nch = (a.chunks_per_row + 31u) / 32u;
    // Few rows: latency matters, spread each row over a whole CTA.  Very wide
    // rows do not fit the register-resident warp kernel either.
    const bool use_cta = rows < 2u * kSmCount || nch > 32u;
    if (use_cta) {
        uint32_t ctas = rows < kSmCount * 8u ? rows : kSmCount * 8u;
        add_rmsnorm_cta_rows_kernel<<<ctas, kCtaThreads, (size_t)cols * sizeof(uint16_t), stream>>>(a);
    } else if (nch <= 4u) launch_warp_rows<4>(a, stream);
    else if (nch <= 8u) launch_warp_rows<8>(a, stream);
    else if (nch <= 12u) launch_warp_rows<12>(a, stream);
    else if (nch <= 16u) launch_warp_rows<16>(a, stream);
    else if (nch <= 20u) launch_warp_rows<20>(a, stream);
    else if (nch <= 24u) launch_warp_rows<24>(a, stream);
    else if (nch <= 28u) launch_warp_rows<28>(a, stream);
    else launch_warp_rows<32>(a, stream);
    note_launch();
    return AXIOM_OK;
}

}  // namespace axb

using namespace axb;

extern "C" int axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device(
        int device, const void *hidden_bf16, void *residual_bf16, const void *gamma_bf16, float eps,
        uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes,
        uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!residual_bf16 || !gamma_bf16 || rows == 0u || cols == 0u || (cols % kGroup) != 0u || cols > 16384u ||
        scale_layout > AXIOM_SCALE_LAYOUT_TILED || !(eps > 0.0f) || !std::isfinite(eps)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !norm_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!aligned16(residual_bf16) || !aligned16(gamma_bf16) || (hidden_bf16 && !aligned16(hidden_bf16)) ||
        (norm_out_bf16 && !aligned16(norm_out_bf16)) || (reinterpret_cast<uintptr_t>(out_codes) & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_rmsnorm_nvfp4_bf16(hidden_bf16, residual_bf16, gamma_bf16, eps, rows, cols, global_scale,
                                  norm_out_bf16, out_codes, out_scales, scale_layout, (cudaStream_t)stream);
    return launch_status();
}

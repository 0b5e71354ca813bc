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
// row, every thread keeps its share of y in registers across the row-max
// reduction, so gate|up is read once and only the codes are written.
#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {

__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    x[0] = bf16_lo(v.x); x[1] = bf16_hi(v.x);
    x[2] = bf16_lo(v.y); x[3] = bf16_hi(v.y);
    x[4] = bf16_lo(v.z); x[5] = bf16_hi(v.z);
    x[6] = bf16_lo(v.w); x[7] = bf16_hi(v.w);
}

__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

__device__ __forceinline__ float absmax8(const float (&x)[8]) {
    const float a = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    const float b = fmaxf(fmaxf(fabsf(x[4]), fabsf(x[5])), fmaxf(fabsf(x[6]), fabsf(x[7])));
    return fmaxf(a, b);
}

// Maximum over the CTA; every thread receives it.  fmaxf drops NaN operands,
// the final clamp makes an all-NaN row give 0 as a running fmaxf from 0 does.
__device__ __forceinline__ float cta_max(float m, float *warp_max) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = (blockDim.x + 31u) >> 5;
#pragma unroll
    for (uint32_t off = 16u; off != 0u; off >>= 1u) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0u) warp_max[warp] = m;
    __syncthreads();
    float all = lane < warps ? warp_max[lane] : 0.0f;
#pragma unroll
    for (uint32_t off = 16u; off != 0u; off >>= 1u) all = fmaxf(all, __shfl_xor_sync(0xffffffffu, all, off));
    __syncthreads();  // warp_max is reused by the next row
    return fmaxf(all, 0.0f);
}

enum class row_op { swiglu, plain_finite_only };

// CPT = 16-byte chunks (8 values) per thread; blockDim.x * CPT >= width / 8.
constexpr uint32_t kMaxRowThreads = 576u;

template <int CPT, row_op kOp>
__global__ void __launch_bounds__(kMaxRowThreads, CPT <= 4 ? 2 : 1)
fp8_rows_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, uint32_t in_chunks_per_row,
                uint2 *__restrict__ codes, float *__restrict__ scales, uint32_t *__restrict__ status_word) {
    __shared__ float warp_max[32];
    const uint32_t tid = threadIdx.x;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *gate = in + (uint64_t)row * in_chunks_per_row;
        float y[CPT][8];
        float m = 0.0f;
        bool nonfinite = false;
        if (kOp == row_op::swiglu) {
            const uint4 *up = gate + chunks;
            uint4 g[CPT], u[CPT];
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + blockDim.x * k;
                const bool ok = q < chunks;
                g[k] = ok ? ld_stream(gate + q) : make_uint4(0u, 0u, 0u, 0u);
                u[k] = ok ? ld_stream(up + q) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                float gv[8], uv[8];
                unpack8(g[k], gv);
                unpack8(u[k], uv);
#pragma unroll
                for (int i = 0; i < 8; ++i) y[k][i] = silu_mul(gv[i], uv[i]);
                m = fmaxf(m, absmax8(y[k]));
            }
        } else {
            uint4 g[CPT];
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + blockDim.x * k;
                g[k] = q < chunks ? ld_stream(gate + q) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                unpack8(g[k], y[k]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // non-finite inputs do not take part in the maximum and raise the status word
                    const bool fin = (__float_as_uint(y[k][i]) & 0x7f800000u) != 0x7f800000u;
                    nonfinite |= !fin;
                    m = fmaxf(m, fin ? fabsf(y[k][i]) : 0.0f);
                }
            }
        }
        m = cta_max(m, warp_max);
        float scale = m == 0.0f ? 1.0f : __fdiv_rn(m, 448.0f);
        if (kOp == row_op::swiglu) {
            if (!isfinite(scale) || scale <= 0.0f) scale = 1.0f;
        } else if (nonfinite && status_word) {
            atomicCAS(status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_NONFINITE);
        }
        if (tid == 0u) scales[row] = scale;
        const float r = __frcp_rn(scale);
        const bool safe = divisor_is_safe(scale, r, m) && !nonfinite;
        uint2 *out = codes + (uint64_t)row * chunks;
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const uint32_t q = tid + blockDim.x * k;
            uint32_t w[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float a0 = div_exact_or_shared(y[k][4 * h + 0], scale, r, safe);
                const float a1 = div_exact_or_shared(y[k][4 * h + 1], scale, r, safe);
                const float a2 = div_exact_or_shared(y[k][4 * h + 2], scale, r, safe);
                const float a3 = div_exact_or_shared(y[k][4 * h + 3], scale, r, safe);
                w[h] = cvt_e4m3x2(a0, a1) | (cvt_e4m3x2(a2, a3) << 16);
            }
            if (q < chunks) st_stream(out + q, make_uint2(w[0], w[1]));
        }
    }
}

// SwiGLU -> NVFP4: no row-wide dependency; lanes own one chunk of gate and the
// matching chunk of up, lane pairs form a 16-value block.
constexpr uint32_t kNvThreads = 256u;
constexpr uint32_t kNvUnroll = 2u;

__global__ void __launch_bounds__(kNvThreads)
swiglu_nvfp4_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, float G,
                    uint32_t *__restrict__ codes, uint8_t *__restrict__ scales, uint32_t layout,
                    uint32_t groups, uint32_t inner_tiles) {
    __shared__ scale_lut_entry lut[128];
    const bool lut_safe = build_scale_lut(lut, G);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kNvThreads + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * kNvThreads) >> 5;
    const uint32_t total = rows * chunks;
    constexpr uint32_t kTile = 32u * kNvUnroll;
    for (uint64_t tile = warp; tile * kTile < total; tile += warps) {
        uint4 g[kNvUnroll], u[kNvUnroll];
        uint32_t row[kNvUnroll], q[kNvUnroll];
#pragma unroll
        for (uint32_t j = 0; j < kNvUnroll; ++j) {
            const uint64_t c = tile * kTile + j * 32u + lane;
            const bool ok = c < total;
            row[j] = ok ? (uint32_t)(c / chunks) : 0u;
            q[j] = ok ? (uint32_t)c - row[j] * chunks : 0u;
            const uint4 *gate = in + (uint64_t)row[j] * 2u * chunks + q[j];
            g[j] = ok ? ld_stream(gate) : make_uint4(0u, 0u, 0u, 0u);
            u[j] = ok ? ld_stream(gate + chunks) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (uint32_t j = 0; j < kNvUnroll; ++j) {
            const uint64_t c = tile * kTile + j * 32u + lane;
            float gv[8], uv[8], y[8];
            unpack8(g[j], gv);
            unpack8(u[j], uv);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = silu_mul(gv[i], uv[i]);
            float m = absmax8_nan(y);
            m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, 1));
            uint32_t scale_code;
            bool needs_exact = false;
            uint32_t packed = nvfp4_quantize8_fast(y, m, G, lut, &scale_code, &needs_exact);
            if (!lut_safe || __any_sync(0xffffffffu, needs_exact)) {
                m = absmax8(y);
                m = fmaxf(fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1)), 0.0f);
                packed = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], m, G, &scale_code);
            }
            if (c < total) {
                st_stream(codes + c, packed);
                if ((lane & 1u) == 0u) {
                    scales[scale_offset(row[j], q[j] >> 1, groups, inner_tiles, layout)] = (uint8_t)scale_code;
                }
            }
        }
    }
}

struct row_shape {
    uint32_t threads;
    uint32_t cpt;
};

// Smallest padding first, then the larger CTA (shorter per-row latency).
row_shape pick_row_shape(uint32_t chunks) {
    static const uint32_t cpts[] = {1u, 2u, 4u, 8u};
    row_shape best{0u, 0u};
    uint64_t best_pad = ~0ull;
    for (uint32_t cpt : cpts) {
        uint32_t threads = (chunks + cpt - 1u) / cpt;
        threads = (threads + 31u) & ~31u;
        if (threads < 64u) threads = 64u;
        if (threads > kMaxRowThreads) continue;
        const uint64_t pad = (uint64_t)threads * cpt - chunks;
        if (pad < best_pad || (pad == best_pad && threads > best.threads)) {
            best_pad = pad;
            best = row_shape{threads, cpt};
        }
    }
    return best;
}

template <row_op kOp>
int launch_fp8_rows(const void *in, uint32_t rows, uint32_t width, uint32_t in_chunks_per_row, uint8_t *codes,
                    float *scales, uint32_t *status_word, cudaStream_t stream) {
    const uint32_t chunks = width / 8u;
    const row_shape s = pick_row_shape(chunks);
    if (s.threads == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint32_t ctas = rows < kSmCount * 16u ? rows : kSmCount * 16u;
    const uint4 *src = (const uint4 *)in;
    uint2 *dst = (uint2 *)codes;
    switch (s.cpt) {
    case 1: fp8_rows_kernel<1, kOp><<<ctas, s.threads, 0, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    case 2: fp8_rows_kernel<2, kOp><<<ctas, s.threads, 0, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    case 4: fp8_rows_kernel<4, kOp><<<ctas, s.threads, 0, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    default: fp8_rows_kernel<8, kOp><<<ctas, s.threads, 0, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    }
    note_launch();
    return AXIOM_OK;
}

}  // namespace

unsigned int swiglu_fault_word() { return read_and_clear_pipeline_fault(); }

int launch_swiglu_fp8_bf16(const void *gate_up, uint32_t rows, uint32_t width, uint8_t *codes, float *scales,
                           cudaStream_t stream) {
    return launch_fp8_rows<row_op::swiglu>(gate_up, rows, width, width / 4u, codes, scales, nullptr, stream);
}

int launch_fp8_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, uint8_t *codes, float *scales,
                             uint32_t *status_word, cudaStream_t stream) {
    return launch_fp8_rows<row_op::plain_finite_only>(input, rows, cols, cols / 8u, codes, scales, status_word, stream);
}

int launch_swiglu_nvfp4_bf16(const void *gate_up, uint32_t rows, uint32_t width, float G, uint8_t *codes,
                             uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    const uint32_t chunks = width / 8u;
    const uint32_t groups = width / kGroup;
    const uint32_t total = rows * chunks;
    const uint32_t tiles = (total + 32u * kNvUnroll - 1u) / (32u * kNvUnroll);
    uint32_t blocks = (tiles + kNvThreads / 32u - 1u) / (kNvThreads / 32u);
    if (blocks > kSmCount * 16u) blocks = kSmCount * 16u;
    swiglu_nvfp4_kernel<<<blocks, kNvThreads, 0, stream>>>((const uint4 *)gate_up, rows, chunks, G, (uint32_t *)codes,
                                                            scales, layout, groups, (groups + 3u) / 4u);
    note_launch();
    return AXIOM_OK;
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

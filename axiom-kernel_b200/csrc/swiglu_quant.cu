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
// silu(g) = g / (1 + expf(-g)) depends on the BF16 gate alone, so the throughput
// kernels tabulate it once per CTA in shared memory — 47 binades x 128 mantissas
// x 2 signs, filled by the very expression the direct path evaluates, hence
// bit-identical — and replace expf + an IEEE division per element by one
// shared-memory load.  Gates outside the table (|g| < 2^-40, |g| >= 128, NaN,
// infinity) take the direct expression.
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

__device__ __forceinline__ float silu(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))); }
__device__ __forceinline__ float silu_mul(float g, float u) { return __fmul_rn(silu(g), u); }

// ---- shared-memory silu table -------------------------------------------------------------
constexpr uint32_t kSiluExpLo = 87u;    // 2^-40
constexpr uint32_t kSiluExpHi = 133u;   // up to (not including) 2^7
constexpr uint32_t kSiluFirst = kSiluExpLo << 7;                       // first tabulated BF16 magnitude
constexpr uint32_t kSiluCount = (kSiluExpHi - kSiluExpLo + 1u) << 7;   // magnitudes per sign
constexpr uint32_t kSiluTableBytes = 2u * kSiluCount * sizeof(float);

__device__ __forceinline__ void build_silu_table(float *table) {
    for (uint32_t i = threadIdx.x; i < 2u * kSiluCount; i += blockDim.x) {
        const uint32_t sign = i >= kSiluCount ? 1u : 0u;
        const uint32_t bits = (sign << 15) | (kSiluFirst + (i - sign * kSiluCount));
        table[i] = silu(__uint_as_float(bits << 16));
    }
    __syncthreads();
}

// bits16: one BF16 pattern in the low half.  Out-of-table patterns read entry 0 and raise *outside.
__device__ __forceinline__ float silu_lookup(const float *table, uint32_t bits16, bool *outside) {
    const uint32_t rel = (bits16 & 0x7fffu) - kSiluFirst;
    const bool in = rel < kSiluCount;
    *outside = *outside || !in;
    return table[(in ? rel : 0u) + (bits16 >> 15) * kSiluCount];
}

// y[0..7] = silu(gate) * up for one 16-byte chunk of each
template <bool kTable>
__device__ __forceinline__ void swiglu8(const float *table, const uint4 &g, const uint4 &u, float (&y)[8]) {
    float uv[8];
    unpack8(u, uv);
    if (kTable) {
        const uint32_t w[4] = {g.x, g.y, g.z, g.w};
        bool outside = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 s = make_float2(silu_lookup(table, w[i] & 0xffffu, &outside), silu_lookup(table, w[i] >> 16, &outside));
            const float2 p = __fmul2_rn(s, make_float2(uv[2 * i], uv[2 * i + 1]));
            y[2 * i] = p.x;
            y[2 * i + 1] = p.y;
        }
        if (outside) {  // rare: a gate beyond the table in this chunk
            float gv[8];
            unpack8(g, gv);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = silu_mul(gv[i], uv[i]);
        }
    } else {
        float gv[8];
        unpack8(g, gv);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = silu_mul(gv[i], uv[i]);
    }
}

// Maximum over the CTA; every thread receives it.  kNan: NaN-propagating (a NaN anywhere in the
// row gives NaN), otherwise fmaxf semantics with the clamp that makes an all-NaN row give 0.
template <bool kNan>
__device__ __forceinline__ float cta_max(float m, float *warp_max) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, warps = (blockDim.x + 31u) >> 5;
#pragma unroll
    for (uint32_t off = 16u; off != 0u; off >>= 1u) {
        const float o = __shfl_xor_sync(0xffffffffu, m, off);
        m = kNan ? max_nan(m, o) : fmaxf(m, o);
    }
    if (lane == 0u) warp_max[warp] = m;
    __syncthreads();
    float all = lane < warps ? warp_max[lane] : 0.0f;
#pragma unroll
    for (uint32_t off = 16u; off != 0u; off >>= 1u) {
        const float o = __shfl_xor_sync(0xffffffffu, all, off);
        all = kNan ? max_nan(all, o) : fmaxf(all, o);
    }
    __syncthreads();  // warp_max is reused
    return kNan ? all : fmaxf(all, 0.0f);
}

enum class row_op { swiglu, swiglu_table, plain_finite_only };

// CPT = 16-byte chunks (8 values) per thread; blockDim.x * CPT >= width / 8.
constexpr uint32_t kMaxRowThreads = 576u;

template <int CPT, row_op kOp>
__global__ void __launch_bounds__(kMaxRowThreads, CPT <= 4 ? 2 : 1)
fp8_rows_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, uint32_t in_chunks_per_row,
                uint2 *__restrict__ codes, float *__restrict__ scales, uint32_t *__restrict__ status_word) {
    extern __shared__ __align__(16) float silu_table[];
    __shared__ float warp_max[32];
    constexpr bool kSwiglu = kOp != row_op::plain_finite_only;
    constexpr bool kTable = kOp == row_op::swiglu_table;
    const uint32_t tid = threadIdx.x;
    if (kTable) build_silu_table(silu_table);
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *gate = in + (uint64_t)row * in_chunks_per_row;
        float y[CPT][8];
        float m = 0.0f;       // NaN-propagating maximum (swiglu) / finite-only maximum (plain)
        bool nonfinite = false;
        if (kSwiglu) {
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
                swiglu8<kTable>(silu_table, g[k], u[k], y[k]);
                m = max_nan(m, absmax8_nan(y[k]));
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
        m = kSwiglu ? cta_max<true>(m, warp_max) : cta_max<false>(m, warp_max);
        if (kSwiglu && !(m == m)) {
            // a NaN somewhere in the row: the reference's maximum drops it
            float d = 0.0f;
#pragma unroll
            for (int k = 0; k < CPT; ++k) d = fmaxf(d, absmax8_drop_nan(y[k]));
            m = cta_max<false>(d, warp_max);
            nonfinite = true;
        }
        float scale = m == 0.0f ? 1.0f : __fdiv_rn(m, 448.0f);
        if (kSwiglu) {
            if (!isfinite(scale) || scale <= 0.0f) scale = 1.0f;
        } else if (nonfinite && status_word) {
            atomicCAS(status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_NONFINITE);
        }
        if (tid == 0u) scales[row] = scale;
        const float r = __frcp_rn(scale);
        const bool safe = divisor_is_safe(scale, r, m) && !nonfinite;  // uniform over the CTA
        uint2 *out = codes + (uint64_t)row * chunks;
        if (safe) {
            // negated residual-corrected quotients (signed zeros survive), signs flipped back on the codes
            const float2 nr2 = make_float2(-r, -r), d2 = make_float2(scale, scale);
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const uint32_t q = tid + blockDim.x * k;
                uint32_t c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 v = make_float2(y[k][2 * i], y[k][2 * i + 1]);
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
                const uint32_t q = tid + blockDim.x * k;
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    w[h] = cvt_e4m3x2(__fdiv_rn(y[k][4 * h + 0], scale), __fdiv_rn(y[k][4 * h + 1], scale)) |
                           (cvt_e4m3x2(__fdiv_rn(y[k][4 * h + 2], scale), __fdiv_rn(y[k][4 * h + 3], scale)) << 16);
                }
                if (q < chunks) st_stream(out + q, make_uint2(w[0], w[1]));
            }
        }
    }
}

// SwiGLU -> NVFP4: no row-wide dependency; lanes own one chunk of gate and the
// matching chunk of up, lane pairs form a 16-value block.
constexpr uint32_t kNvThreads = 256u;
constexpr uint32_t kNvUnroll = 2u;

template <bool kTable>
__global__ void __launch_bounds__(kNvThreads)
swiglu_nvfp4_kernel(const uint4 *__restrict__ in, uint32_t rows, uint32_t chunks, float G,
                    uint32_t *__restrict__ codes, uint8_t *__restrict__ scales, uint32_t layout,
                    uint32_t groups, uint32_t inner_tiles) {
    extern __shared__ __align__(16) float silu_table[];
    __shared__ scale_lut_entry lut[128];
    if (kTable) build_silu_table(silu_table);
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
            float y[8];
            swiglu8<kTable>(silu_table, g[j], u[j], y);
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
    constexpr bool kTable = kOp == row_op::swiglu_table;
    const size_t smem = kTable ? kSiluTableBytes : 0u;
    // table flavour: persistent CTAs (the table is built once per CTA), two per SM
    const uint32_t cap = kTable ? kSmCount * 2u : kSmCount * 16u;
    const uint32_t ctas = rows < cap ? rows : cap;
    const uint4 *src = (const uint4 *)in;
    uint2 *dst = (uint2 *)codes;
    switch (s.cpt) {
    case 1: fp8_rows_kernel<1, kOp><<<ctas, s.threads, smem, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    case 2: fp8_rows_kernel<2, kOp><<<ctas, s.threads, smem, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    case 4: fp8_rows_kernel<4, kOp><<<ctas, s.threads, smem, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    default: fp8_rows_kernel<8, kOp><<<ctas, s.threads, smem, stream>>>(src, rows, chunks, in_chunks_per_row, dst, scales, status_word); break;
    }
    note_launch();
    return AXIOM_OK;
}

// rows at or above which building the 47 KB silu table per CTA pays for itself
constexpr uint32_t kTableMinRows = 2u * kSmCount;

}  // namespace

unsigned int swiglu_fault_word() { return read_and_clear_pipeline_fault(); }

int launch_swiglu_fp8_bf16(const void *gate_up, uint32_t rows, uint32_t width, uint8_t *codes, float *scales,
                           cudaStream_t stream) {
    if (rows >= kTableMinRows) {
        return launch_fp8_rows<row_op::swiglu_table>(gate_up, rows, width, width / 4u, codes, scales, nullptr, stream);
    }
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
    if (rows >= kTableMinRows) {
        static bool configured[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            cudaFuncSetAttribute(swiglu_nvfp4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSiluTableBytes);
            configured[dev] = true;
        }
        if (blocks > kSmCount * 4u) blocks = kSmCount * 4u;  // persistent: the table is built once per CTA
        swiglu_nvfp4_kernel<true><<<blocks, kNvThreads, kSiluTableBytes, stream>>>(
                (const uint4 *)gate_up, rows, chunks, G, (uint32_t *)codes, scales, layout, groups, (groups + 3u) / 4u);
    } else {
        swiglu_nvfp4_kernel<false><<<blocks, kNvThreads, 0, stream>>>(
                (const uint4 *)gate_up, rows, chunks, G, (uint32_t *)codes, scales, layout, groups, (groups + 3u) / 4u);
    }
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

// BF16 -> NVFP4 activation quantizer (packed E2M1 codes, one E4M3 scale per 16
// values, FP32 global multiplier).  Arithmetic of the reference quantizers
// (src/axiom_qwen38_nvfp4.cu:57-88, src/axiom_qwen38_nvfp4_mlp.cu:144-223),
// restructured for HBM streaming: every lane owns one 16-byte chunk (8 values,
// half a block), the block maximum is one lane-pair shuffle, and a warp reads
// 4 x 512 contiguous bytes before it converts anything.
#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {

constexpr uint32_t kThreads = 256u;
constexpr uint32_t kUnroll = 4u;  // 16-byte loads in flight per lane

__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    const float2 a = bf16x2_widen_fma(v.x), b = bf16x2_widen_fma(v.y), c = bf16x2_widen_fma(v.z), d = bf16x2_widen_fma(v.w);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}


// One chunk through the exact path, out of line (the whole warp takes it together): code word in the low half of
// the result, scale byte in the high half.
static __device__ __noinline__ uint64_t quantize_chunk_exact(uint4 v, float G) {
    float x[8];
    unpack8(v, x);
    float m = absmax8_drop_nan(x);  // an all-NaN block has maximum 0, as a running fmaxf from 0 gives
    m = fmaxf(fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1)), 0.0f);
    uint32_t scale_byte;
    const uint32_t packed = nvfp4_quantize8_exact(x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], m, G, &scale_byte);
    return (uint64_t)packed | ((uint64_t)scale_byte << 32);
}

// Quantizes the kUnroll chunks a lane holds for one warp tile (lane pairs form the 16-value blocks).
__device__ __forceinline__ void quantize_tile(const uint4 (&v)[kUnroll], float G, const scale_lut_entry *lut,
                                              bool lut_safe, uint32_t (&packed)[kUnroll],
                                              uint32_t (&scale_byte)[kUnroll]) {
    bool needs_exact = false;
#pragma unroll
    for (uint32_t j = 0; j < kUnroll; ++j) {
        float x[8];
        unpack8(v[j], x);
        float m = absmax8_nan(x);
        m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, 1));
        packed[j] = nvfp4_quantize8_fast(x, m, G, lut, &scale_byte[j], &needs_exact);
    }
    if (!lut_safe || __any_sync(0xffffffffu, needs_exact)) {
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            const uint64_t both = quantize_chunk_exact(v[j], G);
            packed[j] = (uint32_t)both;
            scale_byte[j] = (uint32_t)(both >> 32);
        }
    }
}

// Every warp streams one contiguous range of chunks (ranges differ by at most one 128-byte
// step, so all warps of the persistent grid finish together).  A warp tile is kUnroll x 32
// chunks; full tiles run without a single bounds predicate and with addresses that are a
// per-lane pointer plus a compile-time offset, the ragged last tile of a range takes the
// predicated copy of the same code.  The next tile's loads are issued before the current
// tile is converted.  kTiled: block scales go to the 128 x 4 tiled plane, whose (row, group)
// coordinates a lane tracks incrementally (one division per warp, none per chunk).
template <bool kTiled>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_bf16_kernel(const uint4 *__restrict__ in, uint32_t total_chunks, uint32_t chunks_per_warp,
                           uint32_t chunks_per_row, float G, uint32_t *__restrict__ codes,
                           uint8_t *__restrict__ scales, uint32_t groups, uint32_t inner_tiles) {
    __shared__ scale_lut_entry lut[128];
    constexpr uint32_t kTile = 32u * kUnroll;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    allow_dependents();
    const bool lut_safe = build_scale_lut(lut, G);  // depends on the scalar argument only
    dependency_wait();
    const uint64_t first64 = (uint64_t)warp * chunks_per_warp;
    if (first64 >= total_chunks) return;
    const uint32_t first = (uint32_t)first64;
    const uint32_t count = total_chunks - first < chunks_per_warp ? total_chunks - first : chunks_per_warp;

    const uint4 *src = in + first + lane;
    uint32_t *dst = codes + first + lane;
    uint8_t *sc = scales + ((first + lane) >> 1);          // canonical plane: block index = chunk / 2
    uint32_t row = 0u, col = 0u;                            // tiled plane: this lane's chunk as (row, chunk in row)
    if (kTiled) {
        row = (first + lane) / chunks_per_row;
        col = (first + lane) - row * chunks_per_row;
    }
    uint64_t tile_off = 0u;  // tiled plane: offset of this lane's block (row, col / 2)
    auto store_scale = [&](uint32_t j, uint32_t byte) {
        if (!kTiled) {
            sc[j * 16u] = (uint8_t)byte;
        } else {
            const uint32_t c = col + 32u * j;
            if (c < chunks_per_row) {
                // same row: 32 chunks further is 16 blocks further = 4 tiles of 512 bytes further
                scales[tile_off + j * 2048u] = (uint8_t)byte;
            } else {
                uint32_t r = row, cc = c;
                while (cc >= chunks_per_row) { cc -= chunks_per_row; ++r; }
                scales[scale_offset(r, cc >> 1, groups, inner_tiles, AXIOM_SCALE_LAYOUT_TILED)] = (uint8_t)byte;
            }
        }
    };
    auto locate = [&]() { tile_off = scale_offset(row, col >> 1, groups, inner_tiles, AXIOM_SCALE_LAYOUT_TILED); };
    if (kTiled) locate();
    auto advance = [&]() {
        src += kTile; dst += kTile; sc += kTile / 2u;
        if (kTiled) {
            col += kTile;
            if (col < chunks_per_row) {
                tile_off += (kTile / 32u) * 2048u;
            } else {
                while (col >= chunks_per_row) { col -= chunks_per_row; ++row; }
                locate();
            }
        }
    };

    const uint32_t full_tiles = count / kTile;
    uint4 v[kUnroll];
    if (full_tiles) {
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) v[j] = ld_stream(src + 32u * j);
    }
    for (uint32_t t = 0; t < full_tiles; ++t) {
        uint4 nxt[kUnroll];
        if (t + 1u < full_tiles) {
#pragma unroll
            for (uint32_t j = 0; j < kUnroll; ++j) nxt[j] = ld_stream(src + kTile + 32u * j);
        }
        uint32_t packed[kUnroll], scale_byte[kUnroll];
        quantize_tile(v, G, lut, lut_safe, packed, scale_byte);
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            st_stream(dst + 32u * j, packed[j]);
            if ((lane & 1u) == 0u) store_scale(j, scale_byte[j]);
            v[j] = nxt[j];
        }
        advance();
    }
    const uint32_t rest = count - full_tiles * kTile;  // < kTile chunks, a whole number of blocks
    if (rest) {
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            v[j] = 32u * j + lane < rest ? ld_stream(src + 32u * j) : make_uint4(0u, 0u, 0u, 0u);
        }
        uint32_t packed[kUnroll], scale_byte[kUnroll];
        quantize_tile(v, G, lut, lut_safe, packed, scale_byte);
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            if (32u * j + lane < rest) {
                st_stream(dst + 32u * j, packed[j]);
                if ((lane & 1u) == 0u) store_scale(j, scale_byte[j]);
            }
        }
    }
}

// One F32 row, canonical scales: the exported oracle entry keeps F32 input.
__global__ void __launch_bounds__(128)
nvfp4_quantize_f32_row_kernel(const float *__restrict__ in, float G, uint8_t *__restrict__ codes,
                              uint8_t *__restrict__ scales, uint32_t halves) {
    const uint32_t h = blockIdx.x * 128u + threadIdx.x;  // half-block index (8 values)
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = h < halves ? in[(uint64_t)h * 8u + i] : 0.0f;
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(x[i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    uint32_t scale_code;
    const uint32_t packed = nvfp4_quantize8(x, m, G, &scale_code);
    if (h < halves) {
        // byte stores: the reference entry accepts output pointers of any alignment
#pragma unroll
        for (int i = 0; i < 4; ++i) codes[(uint64_t)h * 4u + i] = (uint8_t)(packed >> (8 * i));
        if ((h & 1u) == 0u) scales[h >> 1] = (uint8_t)scale_code;
    }
}

}  // namespace

int check_nvfp4_quantize(const void *input, uint32_t rows, uint32_t cols, float G, const void *codes,
                         const void *scales, uint32_t layout) {
    if (!input || !codes || !scales || rows == 0u || cols == 0u || (cols % kGroup) != 0u || !valid_scale(G) ||
        layout > AXIOM_SCALE_LAYOUT_TILED) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((uint64_t)rows * (cols / 8u) > 0xffffffffull) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!aligned16(input) || (reinterpret_cast<uintptr_t>(codes) & 3u)) return AXIOM_ERR_INVALID_ARGUMENT;
    return AXIOM_OK;
}

int launch_nvfp4_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, float G, uint8_t *codes,
                               uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    const uint32_t chunks_per_row = cols / 8u;
    const uint32_t total = rows * chunks_per_row;
    const uint32_t groups = cols / kGroup;
    const uint32_t warps_per_block = kThreads / 32u;
    // persistent grid: the 3 CTAs of 256 threads per SM that are resident at 80 registers (one wave), or
    // fewer when there is little to do
    uint32_t blocks = kSmCount * 3u;
    const uint32_t min_chunks_per_warp = 32u * kUnroll;
    const uint32_t needed = (total + min_chunks_per_warp * warps_per_block - 1u) / (min_chunks_per_warp * warps_per_block);
    if (blocks > needed) blocks = needed;
    const uint32_t warps = blocks * warps_per_block;
    uint32_t per_warp = (total + warps - 1u) / warps;
    per_warp = (per_warp + 7u) & ~7u;  // ranges start on 128-byte boundaries and never split a block
    if (layout == AXIOM_SCALE_LAYOUT_TILED) {
        launch_chained(nvfp4_quantize_bf16_kernel<true>, dim3(blocks), dim3(kThreads), 0, stream, (const uint4 *)input,
                       total, per_warp, chunks_per_row, G, (uint32_t *)codes, scales, groups, (groups + 3u) / 4u);
    } else {
        launch_chained(nvfp4_quantize_bf16_kernel<false>, dim3(blocks), dim3(kThreads), 0, stream, (const uint4 *)input,
                       total, per_warp, chunks_per_row, G, (uint32_t *)codes, scales, groups, (groups + 3u) / 4u);
    }
    note_launch();
    return AXIOM_OK;
}

int launch_nvfp4_quantize_f32_row(const float *input, float G, uint8_t *codes, uint8_t *scales, uint32_t cols,
                                  cudaStream_t stream) {
    const uint32_t halves = cols / 8u;
    nvfp4_quantize_f32_row_kernel<<<(halves + 127u) / 128u, 128, 0, stream>>>(input, G, codes, scales, halves);
    note_launch();
    return AXIOM_OK;
}

}  // namespace axb

using namespace axb;

extern "C" int axiom_qwen38_fused_nvfp4_quantize_bf16_device(
        int device, const void *input_bf16, uint32_t rows, uint32_t cols, float global_scale,
        uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    int rc = check_nvfp4_quantize(input_bf16, rows, cols, global_scale, out_codes, out_scales, scale_layout);
    if (rc != AXIOM_OK) return rc;
    if ((rc = select_device(device)) != AXIOM_OK) return rc;
    launch_nvfp4_quantize_bf16(input_bf16, rows, cols, global_scale, out_codes, out_scales, scale_layout,
                               (cudaStream_t)stream);
    return launch_status();
}

// Same contract as the reference symbol: argument checks first, one F32 row,
// canonical scale order, and the stream is synchronised before returning
// (src/axiom_qwen38_nvfp4.cu:121-152).
extern "C" int axiom_qwen38_nvfp4_quantize_reference_f32(
        int device, const float *input, float input_global_scale, uint8_t *out_packed,
        uint8_t *out_scale, uint32_t cols, void *stream) {
    if (!input || !out_packed || !out_scale || cols == 0u || (cols % kGroup) != 0u ||
        !valid_scale(input_global_scale)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (cudaSetDevice(device) != cudaSuccess) return AXIOM_ERR_CUDA;
    launch_nvfp4_quantize_f32_row(input, input_global_scale, out_packed, out_scale, cols, (cudaStream_t)stream);
    if (cudaGetLastError() != cudaSuccess) return AXIOM_ERR_CUDA;
    return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA;
}

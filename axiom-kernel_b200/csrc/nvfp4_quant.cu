// BF16 -> NVFP4 activation quantizer (packed E2M1 codes, one E4M3 scale per 16
// values, FP32 global multiplier).  Arithmetic of the reference quantizers
// (src/axiom_qwen38_nvfp4.cu:57-88, src/axiom_qwen38_nvfp4_mlp.cu:144-223),
// restructured for HBM streaming: every lane owns one 16-byte chunk (8 values,
// half a block), the block maximum is one lane-pair shuffle, and a warp reads
// 4 x 512 contiguous bytes before it converts anything.
#include "runtime.hpp"

namespace axb {

namespace {

constexpr uint32_t kThreads = 256u;
constexpr uint32_t kUnroll = 4u;  // 16-byte loads in flight per lane

__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    x[0] = bf16_lo(v.x); x[1] = bf16_hi(v.x);
    x[2] = bf16_lo(v.y); x[3] = bf16_hi(v.y);
    x[4] = bf16_lo(v.z); x[5] = bf16_hi(v.z);
    x[6] = bf16_lo(v.w); x[7] = bf16_hi(v.w);
}

__device__ __forceinline__ float absmax8(const float (&x)[8]) {
    const float a = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    const float b = fmaxf(fmaxf(fabsf(x[4]), fabsf(x[5])), fmaxf(fabsf(x[6]), fabsf(x[7])));
    return fmaxf(a, b);
}

__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_bf16_kernel(const uint4 *__restrict__ in, uint32_t total_chunks, uint32_t chunks_per_row,
                           float G, uint32_t *__restrict__ codes, uint8_t *__restrict__ scales,
                           uint32_t layout, uint32_t groups, uint32_t inner_tiles) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const uint32_t warps = (gridDim.x * kThreads) >> 5;
    constexpr uint32_t kTile = 32u * kUnroll;
    for (uint64_t tile = warp; tile * kTile < total_chunks; tile += warps) {
        uint4 v[kUnroll];
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            const uint64_t c = tile * kTile + j * 32u + lane;
            v[j] = c < total_chunks ? ld_stream(in + c) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (uint32_t j = 0; j < kUnroll; ++j) {
            const uint64_t c = tile * kTile + j * 32u + lane;
            float x[8];
            unpack8(v[j], x);
            float m = absmax8(x);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, 0.0f);  // an all-NaN block has maximum 0, as a running fmaxf from 0 gives
            uint32_t scale_code;
            const uint32_t packed = nvfp4_quantize8(x, m, G, &scale_code);
            if (c < total_chunks) {
                st_stream(codes + c, packed);
                if ((lane & 1u) == 0u) {
                    uint64_t off = c >> 1;
                    if (layout != AXIOM_SCALE_LAYOUT_CANONICAL) {
                        const uint32_t row = (uint32_t)(c / chunks_per_row);
                        const uint32_t group = ((uint32_t)c - row * chunks_per_row) >> 1;
                        off = scale_offset(row, group, groups, inner_tiles, layout);
                    }
                    scales[off] = (uint8_t)scale_code;
                }
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
    const uint32_t tiles = (total + 32u * kUnroll - 1u) / (32u * kUnroll);
    const uint32_t warps_per_block = kThreads / 32u;
    uint32_t blocks = (tiles + warps_per_block - 1u) / warps_per_block;
    const uint32_t cap = kSmCount * 16u;  // a few waves of resident CTAs, each striding over tiles
    if (blocks > cap) blocks = cap;
    nvfp4_quantize_bf16_kernel<<<blocks, kThreads, 0, stream>>>(
            (const uint4 *)input, total, chunks_per_row, G, (uint32_t *)codes, scales, layout, groups,
            (groups + 3u) / 4u);
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

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

// ---------------------------------------------------------------------------
// Block-per-lane flavour (the one launched for whole tensors).  A lane owns a whole 16-value block: two 16-byte
// loads of 32 contiguous bytes (default caching: the two loads of a warp share their sectors through L1), no lane
// exchange for the block maximum, one scale / table look-up per block, one 8-byte code store and one scale byte per
// lane (a warp writes 256 contiguous code bytes and, in the canonical plane, 32 contiguous scale bytes).  Every
// warp streams one contiguous range of blocks; ranges differ by at most four blocks, so the persistent grid ends
// together.  Loads run kDepth warp tiles (1 KB each) ahead in registers; a tile's registers are refilled as soon as
// it has been converted.  Measured at 4096 x 5120 (canonical / tiled plane): depth 2 with four CTAs per SM 10.9 /
// 11.5 us, depth 3 at 64 registers (spilling) 11.2 / 12.2, depth 3 or 4 with three CTAs 11.2 / 11.6-11.9, depth 2
// with five CTAs 11.2 / 12.6; the chunk-per-lane kernel below 11.5 / 12.5.  At 54 MB per launch the remaining time is
// the dependent-launch floor: first-load latency after the previous kernel has drained, and the drain of the
// last stores (a plain copy of the same bytes takes 12.4 us).  Hinting the first tiles into L2 before the dependency
// wait (cp.async.bulk.prefetch.L2) was measured too and changes nothing: the CTAs of a launch become resident as
// the previous launch's CTAs retire, so there is no earlier moment to hint from; hinting tiles beyond the register
// pipeline from inside the loop makes the kernel 20 % slower.
// ---------------------------------------------------------------------------
#ifndef AXB_Q_DEPTH
#define AXB_Q_DEPTH 2
#endif
#ifndef AXB_Q_CTAS
#define AXB_Q_CTAS 4
#endif
constexpr uint32_t kBlkThreads = 256u;
constexpr uint32_t kDepth = AXB_Q_DEPTH;
constexpr uint32_t kBlkCtasPerSm = AXB_Q_CTAS;

__device__ __forceinline__ uint4 ld_cached(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One block through the exact path, out of line: code words in .x and .y, scale byte in .z (by value: out-pointers
// would force the caller's results into local memory).
static __device__ __noinline__ uint4 quantize_block_exact(uint4 lo, uint4 hi, float G) {
    float x[8], y[8];
    unpack8(lo, x);
    unpack8(hi, y);
    const float m = fmaxf(fmaxf(absmax8_drop_nan(x), absmax8_drop_nan(y)), 0.0f);  // an all-NaN block has maximum 0
    uint32_t sb;
    uint4 out;
    out.x = nvfp4_quantize8_exact(x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], m, G, &sb);
    out.y = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], m, G, &sb);
    out.z = sb;
    out.w = 0u;
    return out;
}

template <bool kTiled>
__global__ void __launch_bounds__(kBlkThreads, kBlkCtasPerSm)
nvfp4_quantize_blocks_kernel(const uint4 *__restrict__ in, uint32_t total_blocks, uint32_t blocks_per_warp, uint32_t groups,
                             float G, uint2 *__restrict__ codes, uint8_t *__restrict__ scales, uint32_t inner_tiles) {
    __shared__ scale_lut_entry lut[128];
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * kBlkThreads + threadIdx.x) >> 5;
    allow_dependents();
    const uint64_t first64 = (uint64_t)warp * blocks_per_warp;
    const uint32_t first = (uint32_t)(first64 < total_blocks ? first64 : total_blocks);
    const uint32_t count = total_blocks - first < blocks_per_warp ? total_blocks - first : blocks_per_warp;
    const bool lut_safe = build_scale_lut(lut, G);  // depends on the scalar argument only
    dependency_wait();
    if (count == 0u) return;
    const uint32_t tiles = (count + 31u) / 32u;

    const uint4 *src = in + 2u * (uint64_t)(first + lane);   // two 16-byte words per block
    uint2 *dst = codes + first + lane;
    uint8_t *sc = scales + first + lane;                      // canonical plane: one byte per block, linear
    uint32_t row = 0u, g = 0u;                                // tiled plane: this lane's block as (row, group)
    if (kTiled) {
        row = (first + lane) / groups;
        g = (first + lane) - row * groups;
    }
    uint4 lo[kDepth], hi[kDepth];
#pragma unroll
    for (uint32_t d = 0; d < kDepth; ++d) {
        lo[d] = hi[d] = make_uint4(0u, 0u, 0u, 0u);
        if (d * 32u + lane < count) {
            lo[d] = ld_cached(src + 64u * d);
            hi[d] = ld_cached(src + 64u * d + 1u);
        }
    }
    for (uint32_t t0 = 0; t0 < tiles; t0 += kDepth) {
#pragma unroll
        for (uint32_t d = 0; d < kDepth; ++d) {
            const uint32_t t = t0 + d;
            if (t >= tiles) break;  // uniform over the warp
            const bool ok = t * 32u + lane < count;
            float x[16];
            {
                float a[8], b[8];
                unpack8(lo[d], a);
                unpack8(hi[d], b);
#pragma unroll
                for (int i = 0; i < 8; ++i) { x[i] = a[i]; x[8 + i] = b[i]; }
            }
            uint32_t scale_byte;
            bool needs_exact = false;
            uint2 packed = nvfp4_quantize16_fast(x, G, lut, &scale_byte, &needs_exact);
            if (!lut_safe || __any_sync(0xffffffffu, needs_exact)) {
                const uint4 redo = quantize_block_exact(lo[d], hi[d], G);
                packed = make_uint2(redo.x, redo.y);
                scale_byte = redo.z;
            }
            // refill this stage with the tile kDepth ahead before the stores go out
            const uint32_t tn = t + kDepth;
            if (tn * 32u + lane < count) {
                lo[d] = ld_cached(src + 64u * tn);
                hi[d] = ld_cached(src + 64u * tn + 1u);
            }
            if (ok) {
                st_stream(dst + 32u * t, packed);
                if (!kTiled) {
                    sc[32u * t] = (uint8_t)scale_byte;
                } else {
                    scales[scale_offset(row, g, groups, inner_tiles, AXIOM_SCALE_LAYOUT_TILED)] = (uint8_t)scale_byte;
                }
            }
            if (kTiled) {
                g += 32u;
                while (g >= groups) { g -= groups; ++row; }
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

// Chunk-per-lane flavour (lane pairs form a block): kept for code buffers that are only 4-byte aligned.
static int launch_nvfp4_quantize_bf16_chunks(const void *input, uint32_t rows, uint32_t cols, float G, uint8_t *codes,
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

int launch_nvfp4_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, float G, uint8_t *codes,
                               uint8_t *scales, uint32_t layout, cudaStream_t stream) {
    const uint32_t groups = cols / kGroup;
    const uint32_t total = rows * groups;  // 16-value blocks (callers bound rows * cols / 8 by 2^32)
    if (reinterpret_cast<uintptr_t>(codes) & 7u) {
        return launch_nvfp4_quantize_bf16_chunks(input, rows, cols, G, codes, scales, layout, stream);  // 4-byte aligned codes only
    }
    const uint32_t warps_per_block = kBlkThreads / 32u;
    // persistent grid: four CTAs of 256 threads per SM (64 registers), or fewer when there is little to do
    uint32_t blocks = kSmCount * kBlkCtasPerSm;
    const uint32_t min_blocks_per_warp = 64u;
    const uint32_t needed = (total + min_blocks_per_warp * warps_per_block - 1u) / (min_blocks_per_warp * warps_per_block);
    if (blocks > needed) blocks = needed;
    const uint32_t warps = blocks * warps_per_block;
    uint32_t per_warp = (total + warps - 1u) / warps;
    per_warp = (per_warp + 3u) & ~3u;  // ranges start on 128-byte boundaries of the input
    if (layout == AXIOM_SCALE_LAYOUT_TILED) {
        launch_chained(nvfp4_quantize_blocks_kernel<true>, dim3(blocks), dim3(kBlkThreads), 0, stream, (const uint4 *)input, total,
                       per_warp, groups, G, (uint2 *)codes, scales, (groups + 3u) / 4u);
    } else {
        launch_chained(nvfp4_quantize_blocks_kernel<false>, dim3(blocks), dim3(kBlkThreads), 0, stream, (const uint4 *)input, total,
                       per_warp, groups, G, (uint2 *)codes, scales, (groups + 3u) / 4u);
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

// Harness around the reference's own NVFP4 activation-quantizer kernels.
// TEST INFRASTRUCTURE: compiled only where the reference tree is present, from
// the reference source where it lies (included below, never copied), into
// oracle/_ref/.  The kernels live in an anonymous namespace of that file, so
// the launchers must be part of the same translation unit.
#include "src/axiom_qwen38_nvfp4_mlp.cu"

namespace {
int ref_done() { return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3; }
}

// input F32 [columns][cols]; codes [columns][cols/2]; scales in the tiled VEC16_UE4M3 plane (pre-zeroed by the caller)
extern "C" int ref_quantize_batch_to_tc(const float *input, float G, uint8_t *codes, uint8_t *scales_tc,
                                        uint32_t cols, uint32_t columns, int warp_variant) {
    const uint32_t groups = cols / 16u, inner_tiles = (groups + 3u) / 4u;
    if (warp_variant) {
        const uint32_t total = groups * columns;
        quantize_batch_to_tc_warp_kernel<<<(total + 15u) / 16u, 256>>>(input, G, codes, scales_tc, cols, groups, inner_tiles, columns);
    } else {
        for (uint32_t c0 = 0; c0 < columns; c0 += 32768u) {
            const uint32_t n = columns - c0 < 32768u ? columns - c0 : 32768u;
            // the kernel addresses the scale plane by absolute column, so shift the base pointers only for whole tiles
            quantize_batch_to_tc_kernel<<<dim3((groups + 127u) / 128u, n), 128>>>(
                    input + (size_t)c0 * cols, G, codes + (size_t)c0 * (cols / 2u),
                    scales_tc + (size_t)(c0 / 128u) * inner_tiles * 512u, cols, groups, inner_tiles, n);
        }
    }
    return ref_done();
}

// gate_up F32 [columns][2*rows] (gate first); codes [columns][rows/2]
extern "C" int ref_silu_mul_quantize_batch_to_tc(const float *gate_up, float G, uint8_t *codes, uint8_t *scales_tc,
                                                 uint32_t rows, uint32_t columns, int warp_variant) {
    const uint32_t groups = rows / 16u, inner_tiles = (groups + 3u) / 4u;
    if (warp_variant) {
        const uint32_t total = groups * columns;
        silu_mul_quantize_batch_to_tc_warp_kernel<<<(total + 15u) / 16u, 256>>>(gate_up, G, codes, scales_tc, rows, groups, inner_tiles, columns);
    } else {
        for (uint32_t c0 = 0; c0 < columns; c0 += 32768u) {
            const uint32_t n = columns - c0 < 32768u ? columns - c0 : 32768u;
            silu_mul_quantize_batch_to_tc_kernel<<<dim3((groups + 127u) / 128u, n), 128>>>(
                    gate_up + (size_t)c0 * rows * 2u, G, codes + (size_t)c0 * (rows / 2u),
                    scales_tc + (size_t)(c0 / 128u) * inner_tiles * 512u, rows, groups, inner_tiles, n);
        }
    }
    return ref_done();
}

extern "C" int ref_silu_mul_batch(const float *gate, const float *up, float *out, uint32_t count) {
    silu_mul_batch_kernel<<<(count + 255u) / 256u, 256>>>(gate, up, out, count);
    return ref_done();
}

// Enqueue-only twins for the timing loops of ref_bench.cu: one launch of the reference's default (warp) kernel
// on the legacy stream, no synchronisation — the way the reference issues it per M = 8 batch
// (projection_run, src/axiom_qwen38_nvfp4_mlp.cu:1347-1381).
extern "C" void ref_enqueue_quantize_to_tc_warp(const float *input, float G, uint8_t *codes, uint8_t *scales_tc,
                                                uint32_t cols, uint32_t columns) {
    const uint32_t groups = cols / 16u, inner_tiles = (groups + 3u) / 4u, total = groups * columns;
    quantize_batch_to_tc_warp_kernel<<<(total + 15u) / 16u, 256>>>(input, G, codes, scales_tc, cols, groups, inner_tiles, columns);
}

extern "C" void ref_enqueue_silu_mul_batch(const float *gate, const float *up, float *out, uint32_t count) {
    silu_mul_batch_kernel<<<(count + 255u) / 256u, 256>>>(gate, up, out, count);
}

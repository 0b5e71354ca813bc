// Timing loops over the reference's own kernels, issued the way the reference issues them: 8 token columns per
// launch (its fixed batch, src/axiom_qwen38_model.cu:34), one launch per fused step, F32 tensors holding BF16
// values, all on the legacy stream.  TEST / BENCHMARK INFRASTRUCTURE: this is the "reference GPU" baseline the
// benchmark reports beside the product's numbers; nothing of the product links it.  The kernels themselves live
// in anonymous namespaces of the reference's units, so each unit's launcher file exports an enqueue-only twin
// and the loops sit here.  Every function returns 0 and the average milliseconds per pass over all rows.
#include <cuda_runtime.h>

#include <cstdint>

extern "C" void ref_enqueue_add_bf16_rmsnorm8(float *residual, const float *addend, const float *weight, float *norm);
extern "C" void ref_enqueue_quantize_to_tc_warp(const float *input, float G, uint8_t *codes, uint8_t *scales_tc,
                                                uint32_t cols, uint32_t columns);
extern "C" void ref_enqueue_silu_mul_batch(const float *gate, const float *up, float *out, uint32_t count);
extern "C" void ref_enqueue_quantize_columns_e4m3(const float *input, uint8_t *codes, float *scales, uint32_t cols, uint32_t n);

namespace {

template <typename Pass>
int timed(uint32_t warmup, uint32_t reps, float *ms_per_pass, Pass pass) {
    cudaEvent_t t0, t1;
    if (cudaEventCreate(&t0) != cudaSuccess || cudaEventCreate(&t1) != cudaSuccess) return 3;
    for (uint32_t r = 0; r < warmup; ++r) pass();
    cudaDeviceSynchronize();
    cudaEventRecord(t0, 0);
    for (uint32_t r = 0; r < reps; ++r) pass();
    cudaEventRecord(t1, 0);
    const bool ok = cudaEventSynchronize(t1) == cudaSuccess && cudaGetLastError() == cudaSuccess;
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, t0, t1);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    *ms_per_pass = reps ? ms / (float)reps : 0.0f;
    return ok ? 0 : 3;
}

constexpr uint32_t kHidden = 5120u, kBatch = 8u;

}  // namespace

// Layer step of the reference at hidden 5120: residual add + RMSNorm (qwen38_add_bf16_rmsnorm8_kernel), then the
// NVFP4 activation quantizer of the MLP that follows it (quantize_batch_to_tc_warp_kernel), per 8 rows.
// residual / addend / norm: F32 [rows][5120]; codes [rows][2560]; scale_planes: rows/8 planes of 80 * 512 bytes
// (every launch writes the tiled plane of its own 8-column batch).  rows % 8 == 0.
extern "C" int ref_time_add_rmsnorm_then_quantize(float *residual, const float *addend, const float *weight, float *norm,
                                                  float G, uint8_t *codes, uint8_t *scale_planes, uint32_t rows,
                                                  uint32_t warmup, uint32_t reps, float *ms_per_pass, uint32_t *launches_per_pass) {
    if (rows % kBatch) return 1;
    const uint32_t plane = ((kHidden / 16u + 3u) / 4u) * 512u;
    *launches_per_pass = 2u * (rows / kBatch);
    return timed(warmup, reps, ms_per_pass, [&] {
        for (uint32_t c0 = 0; c0 < rows; c0 += kBatch) {
            const size_t at = (size_t)c0 * kHidden;
            ref_enqueue_add_bf16_rmsnorm8(residual + at, addend + at, weight, norm + at);
            ref_enqueue_quantize_to_tc_warp(norm + at, G, codes + at / 2u, scale_planes + (size_t)(c0 / kBatch) * plane, kHidden, kBatch);
        }
    });
}

// The activation quantizer alone (configuration 1): input F32 [rows][cols], 8 rows per launch.
extern "C" int ref_time_quantize(const float *input, float G, uint8_t *codes, uint8_t *scale_planes, uint32_t rows,
                                 uint32_t cols, uint32_t warmup, uint32_t reps, float *ms_per_pass, uint32_t *launches_per_pass) {
    if (rows % kBatch || cols % 16u) return 1;
    const uint32_t plane = ((cols / 16u + 3u) / 4u) * 512u;
    *launches_per_pass = rows / kBatch;
    return timed(warmup, reps, ms_per_pass, [&] {
        for (uint32_t c0 = 0; c0 < rows; c0 += kBatch) {
            ref_enqueue_quantize_to_tc_warp(input + (size_t)c0 * cols, G, codes + (size_t)c0 * (cols / 2u),
                                            scale_planes + (size_t)(c0 / kBatch) * plane, cols, kBatch);
        }
    });
}

// FP8 MLP middle (configuration 4): silu(gate) * up into the layer's F32 `mid` buffer (silu_mul_batch_kernel), then
// the per-token E4M3 quantizer of the down projection (quantize_columns_e4m3_kernel), per 8 rows
// (src/axiom_qwen38_fp8_mlp.cu:111-128).  gate, up: F32 [rows][width]; mid: F32 [8][width], reused like the layer's.
extern "C" int ref_time_swiglu_then_fp8(const float *gate, const float *up, float *mid, uint8_t *codes, float *scales,
                                        uint32_t rows, uint32_t width, uint32_t warmup, uint32_t reps, float *ms_per_pass,
                                        uint32_t *launches_per_pass) {
    if (rows % kBatch) return 1;
    *launches_per_pass = 2u * (rows / kBatch);
    return timed(warmup, reps, ms_per_pass, [&] {
        for (uint32_t c0 = 0; c0 < rows; c0 += kBatch) {
            const size_t at = (size_t)c0 * width;
            ref_enqueue_silu_mul_batch(gate + at, up + at, mid, width * kBatch);
            ref_enqueue_quantize_columns_e4m3(mid, codes + at, scales + c0, width, kBatch);
        }
    });
}

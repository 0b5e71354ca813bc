// Harness around the reference's per-token FP8 E4M3 quantizer kernel (test infrastructure, see ref_nvfp4_mlp.cu).
#include "src/axiom_qwen38_fp8.cu"

// input F32 [columns][cols]; the kernel handles at most AXIOM_QWEN38_FP8_BATCH (8) columns per launch
extern "C" int ref_quantize_columns_e4m3(const float *input, uint8_t *codes, float *scales, uint32_t cols, uint32_t columns) {
    for (uint32_t c0 = 0; c0 < columns; c0 += AXIOM_QWEN38_FP8_BATCH) {
        const uint32_t n = columns - c0 < AXIOM_QWEN38_FP8_BATCH ? columns - c0 : AXIOM_QWEN38_FP8_BATCH;
        quantize_columns_e4m3_kernel<<<n, kThreads>>>(input + (size_t)c0 * cols, codes + (size_t)c0 * cols, scales + c0, cols);
    }
    return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// out F32 [8][rows] raw accumulators, scaled and rounded in place: out = bf16((out * weight_scale[row]) * input_scale[column])
extern "C" int ref_fp8_group_row_scale_bf16_epilogue(float *out, const uint16_t *weight_scale, const float *input_scale, uint32_t rows) {
    const uint64_t count = (uint64_t)rows * AXIOM_QWEN38_FP8_BATCH;
    fp8_group_row_scale_bf16_epilogue_kernel<<<(uint32_t)((count + kThreads - 1u) / kThreads), kThreads>>>(out, weight_scale, input_scale, rows);
    return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Enqueue-only twin for ref_bench.cu: one launch over n <= 8 columns, no synchronisation (quantize_input, src/axiom_qwen38_fp8.cu:830-846).
extern "C" void ref_enqueue_quantize_columns_e4m3(const float *input, uint8_t *codes, float *scales, uint32_t cols, uint32_t n) {
    quantize_columns_e4m3_kernel<<<n, kThreads>>>(input, codes, scales, cols);
}

// Static-scale flavour (the ModelOpt branch of quantize_input): input F32 [columns][cols], 8 columns per launch.
extern "C" int ref_quantize_columns_static_e4m3(const float *input, uint8_t *codes, float scale, uint32_t cols, uint32_t columns) {
    for (uint32_t c0 = 0; c0 < columns; c0 += AXIOM_QWEN38_FP8_BATCH) {
        const uint32_t n = columns - c0 < AXIOM_QWEN38_FP8_BATCH ? columns - c0 : AXIOM_QWEN38_FP8_BATCH;
        quantize_columns_static_e4m3_kernel<<<dim3((cols + kThreads - 1u) / kThreads, n), kThreads>>>(
                input + (size_t)c0 * cols, codes + (size_t)c0 * cols, scale, cols);
    }
    return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3;
}

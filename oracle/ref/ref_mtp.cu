// Harness around the reference's BF16-input FP8 row quantizer (test infrastructure, see ref_nvfp4_mlp.cu).
#include "src/axiom_qwen38_mtp_compute.cu"

extern "C" int ref_quantize_bf16_rows_e4m3(const uint16_t *input, uint8_t *codes, float *scales, uint32_t rows,
                                           uint32_t cols, uint32_t *status) {
    quantize_bf16_rows_e4m3_kernel<<<rows, kThreads>>>(input, codes, scales, rows, cols, status);
    return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3;
}

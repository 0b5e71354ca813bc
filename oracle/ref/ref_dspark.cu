// Harness around the reference's BF16-convention (draft / SGLang) q/k kernel and its BF16 rounding pass
// (test infrastructure, see ref_nvfp4_mlp.cu).  Geometry is the draft's own: head_dim 128, full-head NeoX
// rotation, cos/sin read from a caller-supplied FP32 table [positions][cos(64) | sin(64)].
#include "src/axiom_qwen38_dspark_compute.cu"

// x: F32 [columns][heads][128] holding BF16 values, normalised, rounded, rotated and rounded again in place
// (launch_qk_norm_rope + launch_round_bf16, the two steps of the layer sequence at
// src/axiom_qwen38_dspark_compute.cu:1816-1825); token c is at position first_position + c.
extern "C" int ref_dspark_qk_norm_rope_round(const uint16_t *weight, float *x, const float *rope_cache,
                                             uint32_t rope_cache_positions, uint32_t heads, uint32_t columns,
                                             uint32_t first_position) {
    int rc = launch_qk_norm_rope(weight, x, rope_cache, rope_cache_positions, heads, columns, first_position, nullptr, 0);
    if (rc == AXIOM_OK) rc = launch_round_bf16(x, (uint64_t)heads * kHeadDim * columns, 0);
    if (rc != AXIOM_OK) return rc;
    return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3;
}

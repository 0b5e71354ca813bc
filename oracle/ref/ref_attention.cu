// Harness around the reference's attention pre-processing kernels (test infrastructure, see
// ref_nvfp4_mlp.cu).  Geometry is the reference's own: 24 q / 4 kv heads x 256, rope_dim 64,
// theta 1e7, YaRN x4 over 262144, 8 token columns.
#include "src/axiom_qwen38_attention.cu"

namespace {
int ref_done() { return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3; }
}

__global__ void ref_yarn_inv_frequency_kernel(float *out) {
    if (threadIdx.x < kRopeDim / 2u) out[threadIdx.x] = qwen38_yarn_inv_frequency(threadIdx.x);
}

extern "C" int ref_yarn_inv_frequency(float *out32) {
    ref_yarn_inv_frequency_kernel<<<1, 32>>>(out32);
    return ref_done();
}

// q F32 [8][24][256], k F32 [8][4][256], v F32 [8][4][256]; token t is at position base + t;
// k_cache_reference / v_cache_reference F32 [max_context][1024]; the E4M3 caches are u8 of the same shape.
extern "C" int ref_qk_norm_partial_rope_cache_temporal8(float *q, float *k, const float *q_weight, const float *k_weight,
                                                        const float *v, uint8_t *k_cache, uint8_t *v_cache,
                                                        float *k_cache_reference, float *v_cache_reference,
                                                        uint32_t base_position, uint32_t max_context, int yarn) {
    qwen38_qk_norm_partial_rope_cache_temporal8_kernel<<<dim3(kHeads + kKvHeads, kBatch), kThreads>>>(
            q, k, q_weight, k_weight, v, k_cache, v_cache, k_cache_reference, v_cache_reference, base_position, nullptr,
            max_context, yarn != 0, nullptr);
    return ref_done();
}

// all 8 columns at the same position (the batch-lane kernel); cache_columns lanes of [max_context][1024]
extern "C" int ref_qk_norm_partial_rope_cache8(float *q, float *k, const float *q_weight, const float *k_weight,
                                               const float *v, uint8_t *k_cache, uint8_t *v_cache,
                                               float *k_cache_reference, float *v_cache_reference,
                                               uint32_t cache_columns, uint32_t max_context, uint32_t position, int yarn) {
    qwen38_qk_norm_partial_rope_cache8_kernel<<<dim3(kHeads + kKvHeads, kBatch), kThreads>>>(
            q, k, q_weight, k_weight, v, k_cache, v_cache, k_cache_reference, v_cache_reference, cache_columns,
            max_context, position, yarn != 0, nullptr);
    return ref_done();
}

// attention, gate, out: F32 [8][6144] holding BF16 values (the reference's fixed batch of 8 token columns)
extern "C" int ref_sigmoid_gate8(const float *attention, const float *gate, float *out) {
    const uint64_t count = static_cast<uint64_t>(kQDim) * kBatch;
    qwen38_sigmoid_gate_kernel<<<static_cast<uint32_t>((count + kThreads - 1u) / kThreads), kThreads>>>(attention, gate, out);
    return ref_done();
}

// the attention block's input norm: weight F32 [kHidden], input / out F32 [8][kHidden] (kHidden = 5120)
extern "C" int ref_attention_rmsnorm8(const float *weight, const float *input, float *out) {
    qwen38_attention_rmsnorm8_kernel<<<kBatch, kThreads>>>(weight, input, out);
    return ref_done();
}

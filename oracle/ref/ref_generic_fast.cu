// Harness around the reference's generic single-row F32 kernels (test infrastructure, see
// ref_nvfp4_mlp.cu).  Built WITH --use_fast_math, as the reference builds this unit.
#include "src/axiom_cuda.cu"

static int ref_done() { return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3; }

extern "C" int ref_rmsnorm_f32(const float *w, const float *in, float *out, uint32_t count, float eps, int variant) {
    if (variant == 0) axiom_rmsnorm_f32_device_kernel<<<1, 256>>>(w, in, out, count, eps);
    else if (variant == 1) axiom_rmsnorm_f32_hp_device_kernel<<<1, 256>>>(w, in, out, count, eps);
    else axiom_rmsnorm_f32_b1_device_kernel<<<1, 256>>>(w, in, out, count, eps);
    return ref_done();
}

extern "C" int ref_rmsnorm_f32_dual(const float *w, const float *in0, float *out0, const float *in1, float *out1, uint32_t count, float eps) {
    axiom_rmsnorm_f32_dual_device_kernel<<<2, 256>>>(w, in0, out0, in1, out1, count, eps);
    return ref_done();
}

extern "C" int ref_head_rmsnorm_f32(float *x, uint32_t heads, uint32_t head_dim, float eps) {
    axiom_head_rmsnorm_f32_device_kernel<<<heads, 256>>>(x, head_dim, eps);
    return ref_done();
}

extern "C" int ref_qk_rmsnorm_w_f32(float *x, const float *w, uint32_t heads, uint32_t head_dim, float eps) {
    axiom_qwen_qk_rmsnorm_w_f32_kernel<<<heads, 256>>>(x, w, head_dim, eps);
    return ref_done();
}

extern "C" int ref_add_f32(const float *a, const float *b, float *out, uint32_t count) {
    axiom_add_f32_device_kernel<<<(count + 255u) / 256u, 256>>>(a, b, out, count);
    return ref_done();
}

extern "C" int ref_silu_mul_f32(const float *gate, const float *up, float *out, uint32_t count, float clamp_abs) {
    axiom_silu_mul_f32_kernel<<<(count + 255u) / 256u, 256>>>(gate, up, out, count, clamp_abs);
    return ref_done();
}

extern "C" int ref_kv_pool_store_paged_f32(const float *k_stage, const float *v_stage, float *kpool, float *vpool,
                                           const int32_t *tables, const uint32_t *pos, uint32_t active, uint32_t tbl_stride,
                                           uint32_t NL, uint32_t L, uint32_t BT, uint32_t pool_stride, uint32_t kv_dim) {
    axiom_kv_pool_store_paged_f32_kernel<<<dim3((kv_dim + 255u) / 256u, active), 256>>>(
            k_stage, v_stage, kpool, vpool, tables, pos, tbl_stride, NL, L, BT, pool_stride, kv_dim);
    return ref_done();
}

extern "C" int ref_q8_0_embedding_gather_f32(const uint8_t *embedding, float *out, uint32_t token_id, uint32_t token_count,
                                             uint32_t hidden) {
    axiom_q8_0_embedding_gather_f32_kernel<<<(hidden + 255u) / 256u, 256>>>(embedding, out, token_id, token_count, hidden);
    return ref_done();
}

extern "C" int ref_q8_0_embedding_gather_token_f32(const uint8_t *embedding, const uint32_t *token_id, float *out,
                                                   uint32_t token_count, uint32_t hidden) {
    axiom_q8_0_embedding_gather_token_f32_kernel<<<(hidden + 255u) / 256u, 256>>>(embedding, token_id, out, token_count, hidden);
    return ref_done();
}

extern "C" int ref_f16_embedding_streams(const uint16_t *embedding, float *out, uint32_t token_id, uint32_t hidden, uint32_t streams) {
    const uint64_t total = (uint64_t)hidden * streams;
    axiom_f16_embedding_streams_device_kernel<<<(uint32_t)((total + 255u) / 256u), 256>>>(embedding, out, token_id, hidden, streams);
    return ref_done();
}

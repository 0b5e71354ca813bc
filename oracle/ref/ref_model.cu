// Harness around the reference's layer-glue kernels: BF16-boundary residual add, fused add + RMSNorm,
// RMSNorm, embedding gather (test infrastructure, see ref_nvfp4_mlp.cu).  Geometry is the reference's
// own: hidden 5120, 8 token columns per launch, vocabulary 248320.
#include "src/axiom_qwen38_model.cu"

namespace {
int ref_done() { return cudaDeviceSynchronize() == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 3; }
}

extern "C" uint32_t ref_model_hidden() { return kHidden; }
extern "C" uint32_t ref_model_vocab() { return kVocab; }

extern "C" int ref_add_bf16_inplace(float *dst, const float *addend, uint64_t count) {
    qwen38_add_bf16_inplace_kernel<<<(uint32_t)((count + kThreads - 1u) / kThreads), kThreads>>>(dst, addend, count);
    return ref_done();
}

// residual/addend/norm F32 [columns][5120]; columns is processed 8 at a time (a short last launch reads
// and writes only whole 8-column groups, so the caller pads to a multiple of 8)
extern "C" int ref_add_bf16_rmsnorm8(float *residual, const float *addend, const float *weight, float *norm, uint32_t columns) {
    if (columns % kBatch) return 1;
    for (uint32_t c0 = 0; c0 < columns; c0 += kBatch) {
        qwen38_add_bf16_rmsnorm8_kernel<<<kBatch, kThreads>>>(residual + (size_t)c0 * kHidden, addend + (size_t)c0 * kHidden,
                                                              weight, norm + (size_t)c0 * kHidden);
    }
    return ref_done();
}

extern "C" int ref_rmsnorm_bf16_8(const float *weight, const float *input, float *out, uint32_t columns) {
    if (columns % kBatch) return 1;
    for (uint32_t c0 = 0; c0 < columns; c0 += kBatch) {
        qwen38_rmsnorm_bf16_8_kernel<<<kBatch, kThreads>>>(weight, input + (size_t)c0 * kHidden, out + (size_t)c0 * kHidden);
    }
    return ref_done();
}

extern "C" int ref_embedding_gather_columns(const uint16_t *embedding, const uint32_t *token_ids, float *out, uint32_t columns) {
    qwen38_embedding_gather_columns_kernel<<<columns, kThreads>>>(embedding, token_ids, out, columns);
    return ref_done();
}

// logits F32 [8][248320]; partials: 8 x 256 results of 12 bytes; results: 8 x 12 bytes.  hierarchical != 0 takes the
// two-stage path, else the single-kernel one.
extern "C" int ref_top1_8(const float *logits, void *partials, void *results, int hierarchical) {
    if (hierarchical) {
        qwen38_top1_8_stage1_kernel<<<dim3(kTop1Blocks, kBatch), kThreads>>>(logits, (qwen38_top1_result *)partials);
        qwen38_top1_8_stage2_kernel<<<kBatch, kThreads>>>((const qwen38_top1_result *)partials, (qwen38_top1_result *)results);
    } else {
        qwen38_top1_8_kernel<<<kBatch, kThreads>>>(logits, (qwen38_top1_result *)results);
    }
    return ref_done();
}

// Enqueue-only twin for ref_bench.cu: one 8-column launch, no synchronisation (src/axiom_qwen38_model.cu:1371-1373).
extern "C" void ref_enqueue_add_bf16_rmsnorm8(float *residual, const float *addend, const float *weight, float *norm) {
    qwen38_add_bf16_rmsnorm8_kernel<<<kBatch, kThreads>>>(residual, addend, weight, norm);
}

// taps: F32 [tap_count][8][5120]; copies the 8 hidden columns into slot tap_index (qwen38_capture_tap8_kernel)
extern "C" int ref_capture_tap8(const float *hidden, float *taps, uint32_t tap_index) {
    const uint64_t count = (uint64_t)kHidden * kBatch;
    qwen38_capture_tap8_kernel<<<(uint32_t)((count + kThreads - 1u) / kThreads), kThreads>>>(hidden, taps, tap_index);
    return ref_done();
}

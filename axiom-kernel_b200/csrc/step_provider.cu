// Family provider for the reference's step engine: the forward_step hook of axiom_engine_family_ops
// (include/axiom/axiom_engine.h:218-225) with every elementwise stage of the decode forward taken from this
// library and every contraction delegated to the integrator's hooks.  Stage order of one layer as in the
// reference's forward (src/axiom_qwen38_model.cu:1357-1401, attention block src/axiom_qwen38_attention.cu:3482-3687):
//   input norm -> [q/k/v projections] -> q/k norm + RoPE + paged-KV write at the sequence's position
//   -> [attention core + output projection] -> residual add + post norm + NVFP4 -> [gate_up] -> SwiGLU + NVFP4
//   -> [down] -> residual add + next layer's input norm (or the final norm) -> ... -> [LM head] -> logits to the host.
// Paged addressing comes from the engine's device view: block tables d_tbl [cap][tbl_stride], positions at byte
// cap*4 of d_meta, pools d_kpool / d_vpool with element offset (((pb*n_layers+L)*BT+slot)*kv_dim) (:183-198,282-283).
#include "axiom_b200_engine.h"

#include <cstring>
#include <new>

#include "runtime.hpp"

using namespace axb;

struct axiom_b200_step_provider {
    axiom_runtime *runtime = nullptr;
    axiom_b200_step_provider_config cfg{};
    cudaStream_t stream = nullptr;
    uint8_t *arena = nullptr;          // one device allocation holding every scratch tensor
    uint32_t *ids_host = nullptr;      // pinned [max_batch]
    float *logits_host = nullptr;      // pinned [max_batch][vocab]
    uint32_t *status_host = nullptr;   // pinned [1]
    // scratch tensors (device)
    void *residual = nullptr, *norm = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *mixer_out = nullptr;
    uint8_t *in_codes = nullptr, *in_scales = nullptr, *mid_codes = nullptr, *mid_scales = nullptr;
    void *gate_up = nullptr, *mlp_out = nullptr;
    float *logits = nullptr;
    uint32_t *ids = nullptr, *status = nullptr;
    uint64_t in_plane = 0, mid_plane = 0;
};

namespace {

uint64_t align256(uint64_t v) { return (v + 255u) & ~255ull; }

bool config_ok(const axiom_b200_step_provider_config *c) {
    if (!c || c->abi_version != AXIOM_ABI_VERSION || c->struct_size != sizeof(*c)) return false;
    if (c->n_layers == 0u || c->hidden == 0u || (c->hidden % kGroup) != 0u || c->hidden > 16384u || c->ffn == 0u ||
        (c->ffn % kGroup) != 0u || c->ffn > 36864u || c->k_heads == 0u || c->q_heads == 0u ||
        (c->head_dim != 64u && c->head_dim != 128u && c->head_dim != 256u) || c->rope_dim > c->head_dim ||
        c->vocab == 0u || c->max_batch == 0u || c->max_batch > 65535u || c->kv_block_tokens == 0u || c->kv_nphys == 0u ||
        c->kv_dim < c->k_heads * c->head_dim || (c->kv_dim % 8u) != 0u) {
        return false;
    }
    if (!(c->eps > 0.0f) || !std::isfinite(c->eps) || !std::isfinite(c->mscale) || !valid_scale(c->gate_up_input_scale) ||
        !valid_scale(c->down_input_scale)) {
        return false;
    }
    if (!c->embedding || !c->input_norm_gamma || !c->post_norm_gamma || !c->final_norm_gamma || !c->q_norm_gamma ||
        !c->k_norm_gamma || (c->rope_dim != 0u && !c->inv_freq)) {
        return false;
    }
    const axiom_b200_contraction_hooks &h = c->hooks;
    return h.qkv_projection && h.attention_output && h.gate_up_projection && h.down_projection && h.lm_head;
}

}  // namespace

extern "C" void axiom_b200_step_provider_destroy(axiom_b200_step_provider *p) {
    if (!p) return;
    if (p->runtime) (void)cudaSetDevice((int)p->runtime->device);
    if (p->stream) {
        (void)cudaStreamSynchronize(p->stream);
        (void)cudaStreamDestroy(p->stream);
    }
    if (p->arena) (void)cudaFree(p->arena);
    if (p->ids_host) (void)cudaFreeHost(p->ids_host);
    if (p->logits_host) (void)cudaFreeHost(p->logits_host);
    if (p->status_host) (void)cudaFreeHost(p->status_host);
    delete p;
}

extern "C" int axiom_b200_step_provider_create(axiom_runtime *runtime, const axiom_b200_step_provider_config *config,
                                               axiom_b200_step_provider **out) {
    if (out) *out = nullptr;
    if (!runtime || !out || !config_ok(config)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (runtime->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    int rc = select_device((int)runtime->device);
    if (rc != AXIOM_OK) return rc;
    axiom_b200_step_provider *p = new (std::nothrow) axiom_b200_step_provider();
    if (!p) return AXIOM_ERR_RUNTIME;
    p->runtime = runtime;
    p->cfg = *config;
    const axiom_b200_step_provider_config &c = p->cfg;
    const uint64_t n = c.max_batch;
    p->in_plane = axiom_nvfp4_scale_plane_bytes(c.max_batch, c.hidden / kGroup, AXIOM_SCALE_LAYOUT_TILED);
    p->mid_plane = axiom_nvfp4_scale_plane_bytes(c.max_batch, c.ffn / kGroup, AXIOM_SCALE_LAYOUT_TILED);
    const uint64_t sizes[] = {
            n * c.hidden * 2u,                    // residual
            n * c.hidden * 2u,                    // norm
            n * c.q_heads * c.head_dim * 2u,      // q
            n * c.k_heads * c.head_dim * 2u,      // k
            n * c.k_heads * c.head_dim * 2u,      // v
            n * c.hidden * 2u,                    // mixer_out
            n * c.hidden / 2u, p->in_plane,       // mlp_in codes, scales
            n * c.ffn * 4u,                       // gate_up
            n * c.ffn / 2u, p->mid_plane,         // mlp_mid codes, scales
            n * c.hidden * 2u,                    // mlp_out
            n * c.vocab * 4u,                     // logits
            n * 4u, 4u,                           // ids, status word
    };
    uint64_t total = 0;
    for (uint64_t s : sizes) total += align256(s);
    cudaError_t err = cudaMalloc(&p->arena, (size_t)total);
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaHostAlloc(&p->ids_host, (size_t)n * 4u, cudaHostAllocDefault);
    if (err == cudaSuccess) err = cudaHostAlloc(&p->logits_host, (size_t)(n * c.vocab * 4u), cudaHostAllocDefault);
    if (err == cudaSuccess) err = cudaHostAlloc(&p->status_host, 4u, cudaHostAllocDefault);
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        axiom_b200_step_provider_destroy(p);
        return cuda_to_status(err);
    }
    uint8_t *at = p->arena;
    auto take = [&](uint64_t bytes) {
        uint8_t *ptr = at;
        at += align256(bytes);
        return ptr;
    };
    p->residual = take(sizes[0]); p->norm = take(sizes[1]); p->q = take(sizes[2]); p->k = take(sizes[3]); p->v = take(sizes[4]);
    p->mixer_out = take(sizes[5]); p->in_codes = take(sizes[6]); p->in_scales = take(sizes[7]); p->gate_up = take(sizes[8]);
    p->mid_codes = take(sizes[9]); p->mid_scales = take(sizes[10]); p->mlp_out = take(sizes[11]);
    p->logits = (float *)take(sizes[12]); p->ids = (uint32_t *)take(sizes[13]); p->status = (uint32_t *)take(sizes[14]);
    // the tiled scale planes are written cell by cell: their padding has to read as zero
    if (cudaMemsetAsync(p->in_scales, 0, (size_t)p->in_plane, p->stream) != cudaSuccess ||
        cudaMemsetAsync(p->mid_scales, 0, (size_t)p->mid_plane, p->stream) != cudaSuccess ||
        axiom_b200_prepare((int)runtime->device) != AXIOM_OK || cudaStreamSynchronize(p->stream) != cudaSuccess) {
        (void)cudaGetLastError();
        axiom_b200_step_provider_destroy(p);
        return AXIOM_ERR_CUDA;
    }
    *out = p;
    return AXIOM_OK;
}

extern "C" void *axiom_b200_step_provider_scratch(axiom_b200_step_provider *p, uint32_t which) {
    if (!p) return nullptr;
    void *const table[] = {p->residual, p->norm, p->q, p->k, p->v, p->mixer_out, p->in_codes, p->in_scales, p->gate_up,
                           p->mid_codes, p->mid_scales, p->mlp_out, p->logits};
    return which < sizeof(table) / sizeof(table[0]) ? table[which] : nullptr;
}

extern "C" int axiom_b200_step_provider_forward_step(void *fam, axiom_engine_seq *const *active, int n_active,
                                                     const axiom_engine_dev *dev) {
    axiom_b200_step_provider *p = static_cast<axiom_b200_step_provider *>(fam);
    if (!p || !active || n_active <= 0 || !dev) return AXIOM_ERR_INVALID_ARGUMENT;
    const axiom_b200_step_provider_config &c = p->cfg;
    const uint32_t n = (uint32_t)n_active;
    if (n > c.max_batch || dev->cap <= 0 || n > (uint32_t)dev->cap || dev->tbl_stride == 0u || !dev->d_kpool || !dev->d_vpool ||
        !dev->d_tbl || !dev->d_meta || !owned_by(p->runtime, dev->d_kpool) || !owned_by(p->runtime, dev->d_vpool) ||
        !owned_by(p->runtime, dev->d_tbl) || !owned_by(p->runtime, dev->d_meta)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    // the spans the kernels will address: pools, block-table matrix, metadata row of positions
    uint64_t pool_rows = 0, pool_bytes = 0;
    if (!mul_ok((uint64_t)c.kv_nphys * c.n_layers, c.kv_block_tokens, &pool_rows) || !mul_ok(pool_rows, (uint64_t)c.kv_dim * 2u, &pool_bytes) ||
        !span_ok(dev->d_kpool, 0u, pool_bytes) || !span_ok(dev->d_vpool, 0u, pool_bytes) ||
        !span_ok(dev->d_tbl, 0u, (uint64_t)dev->cap * dev->tbl_stride * 4u) || !span_ok(dev->d_meta, 0u, (uint64_t)dev->cap * 8u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    for (uint32_t a = 0; a < n; ++a) {
        if (!active[a]) return AXIOM_ERR_INVALID_ARGUMENT;
        p->ids_host[a] = active[a]->next_tok;
    }
    int rc = select_device((int)p->runtime->device);
    if (rc != AXIOM_OK) return rc;
    cudaStream_t s = p->stream;
    const uint32_t hidden = c.hidden, kvw = c.k_heads * c.head_dim;
    const uint8_t *in_gamma = (const uint8_t *)c.input_norm_gamma, *post_gamma = (const uint8_t *)c.post_norm_gamma;
    const uint8_t *q_gamma = (const uint8_t *)c.q_norm_gamma, *k_gamma = (const uint8_t *)c.k_norm_gamma;
    (void)kvw;

    // embed: the residual stream starts as the embedding rows of next_tok, and the first input norm rides along
    if (cudaMemcpyAsync(p->ids, p->ids_host, (size_t)n * 4u, cudaMemcpyHostToDevice, s) != cudaSuccess ||
        cudaMemsetAsync(p->status, 0, 4u, s) != cudaSuccess ||
        cudaMemsetAsync(p->residual, 0, (size_t)n * hidden * 2u, s) != cudaSuccess) {
        return AXIOM_ERR_CUDA;
    }
    launch_gather_add_rmsnorm_nvfp4_bf16(c.embedding, c.vocab, p->ids, p->residual, in_gamma, c.eps, n, hidden, 1.0f, p->norm,
                                         nullptr, nullptr, AXIOM_SCALE_LAYOUT_CANONICAL, p->status, s);
    const axiom_b200_contraction_hooks &h = c.hooks;
    for (uint32_t layer = 0; layer < c.n_layers; ++layer) {
        if ((rc = h.qkv_projection(h.user, layer, n, p->norm, p->q, p->k, p->v, s)) != 0) break;
        axiom_qk_rope_args qa{};
        qa.abi_version = AXIOM_ABI_VERSION;
        qa.struct_size = sizeof qa;
        qa.tokens = n; qa.q_heads = c.q_heads; qa.k_heads = c.k_heads; qa.head_dim = c.head_dim; qa.rope_dim = c.rope_dim;
        qa.flags = AXIOM_QK_FLAG_PER_TOKEN_TABLE;
        qa.eps = c.eps; qa.mscale = c.mscale;
        qa.block_tokens = c.kv_block_tokens; qa.n_layers = c.n_layers; qa.layer = layer; qa.pool_stride = c.kv_dim;
        qa.tbl_stride = dev->tbl_stride; qa.n_blocks = c.kv_nphys;
        qa.q_bf16 = p->q; qa.k_bf16 = p->k; qa.v_bf16 = p->v;
        qa.q_gamma_bf16 = q_gamma + (size_t)layer * c.head_dim * 2u;
        qa.k_gamma_bf16 = k_gamma + (size_t)layer * c.head_dim * 2u;
        qa.inv_freq = c.inv_freq;
        qa.positions = (const uint32_t *)at(dev->d_meta, (uint64_t)dev->cap * 4u);
        qa.block_tables = (const int32_t *)at(dev->d_tbl, 0u);
        qa.k_pool_bf16 = at(dev->d_kpool, 0u);
        qa.v_pool_bf16 = at(dev->d_vpool, 0u);
        qa.status_word = p->status;
        launch_qk_norm_rope_paged_bf16(&qa, s);
        if ((rc = h.attention_output(h.user, layer, n, p->q, dev, p->mixer_out, s)) != 0) break;
        launch_add_rmsnorm_nvfp4_bf16(p->mixer_out, p->residual, post_gamma + (size_t)layer * hidden * 2u, c.eps, n, hidden,
                                      c.gate_up_input_scale, nullptr, p->in_codes, p->in_scales, AXIOM_SCALE_LAYOUT_TILED, s);
        if ((rc = h.gate_up_projection(h.user, layer, n, p->in_codes, p->in_scales, p->gate_up, s)) != 0) break;
        launch_swiglu_nvfp4_bf16(p->gate_up, n, c.ffn, c.down_input_scale, p->mid_codes, p->mid_scales, AXIOM_SCALE_LAYOUT_TILED, s);
        if ((rc = h.down_projection(h.user, layer, n, p->mid_codes, p->mid_scales, p->mlp_out, s)) != 0) break;
        const void *next_gamma = layer + 1u < c.n_layers ? (const void *)(in_gamma + (size_t)(layer + 1u) * hidden * 2u) : c.final_norm_gamma;
        launch_add_rmsnorm_nvfp4_bf16(p->mlp_out, p->residual, next_gamma, c.eps, n, hidden, 1.0f, p->norm, nullptr, nullptr,
                                      AXIOM_SCALE_LAYOUT_CANONICAL, s);
    }
    if (rc == 0) rc = h.lm_head(h.user, n, p->norm, p->logits, s);
    if (rc != 0) {
        (void)cudaStreamSynchronize(s);  // nothing of the aborted step is left running
        (void)cudaGetLastError();
        return rc;
    }
    if (cudaGetLastError() != cudaSuccess ||
        cudaMemcpyAsync(p->logits_host, p->logits, (size_t)n * c.vocab * 4u, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(p->status_host, p->status, 4u, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        (void)cudaGetLastError();
        return AXIOM_ERR_CUDA;
    }
    for (uint32_t a = 0; a < n; ++a) {
        if (active[a]->seq_logits) memcpy(active[a]->seq_logits, p->logits_host + (size_t)a * c.vocab, (size_t)c.vocab * 4u);
    }
    return *p->status_host == AXIOM_STATUS_WORD_OK ? AXIOM_OK : AXIOM_ERR_RUNTIME;
}

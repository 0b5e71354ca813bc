// axiom_device_buffer flavour and host-I/O flavour of the fused BF16 entry
// points.  Validation follows the reference runtime wrappers: NULLs, zero
// sizes, divisibility, same-runtime, overflow-checked byte counts and span
// checks come before anything is touched (src/axiom_runtime.cpp:3286-3340).
#include <cstdlib>

#include "runtime.hpp"

#include <algorithm>

namespace axb {

int staging_pool::reserve(uint64_t bytes_per_slot, uint64_t aux_need) {
    for (int i = 0; i < kSlots; ++i) {
        if (!stream[i] && cudaStreamCreateWithFlags(&stream[i], cudaStreamNonBlocking) != cudaSuccess) {
            return AXIOM_ERR_CUDA;
        }
    }
    if (!aux_ready && cudaEventCreateWithFlags(&aux_ready, cudaEventDisableTiming) != cudaSuccess) return AXIOM_ERR_CUDA;
    if (bytes_per_slot > slot_bytes) {
        for (int i = 0; i < kSlots; ++i) {
            if (slot[i]) (void)cudaFree(slot[i]);
            slot[i] = nullptr;
        }
        slot_bytes = 0;
        for (int i = 0; i < kSlots; ++i) {
            const cudaError_t err = cudaMalloc(&slot[i], (size_t)bytes_per_slot);
            if (err != cudaSuccess) {
                (void)cudaGetLastError();
                return cuda_to_status(err);
            }
        }
        slot_bytes = bytes_per_slot;
    }
    if (aux_need > aux_bytes) {
        if (aux) (void)cudaFree(aux);
        aux = nullptr;
        aux_bytes = 0;
        const cudaError_t err = cudaMalloc(&aux, (size_t)aux_need);
        if (err != cudaSuccess) {
            (void)cudaGetLastError();
            return cuda_to_status(err);
        }
        aux_bytes = aux_need;
    }
    return AXIOM_OK;
}

void staging_pool::release() {
    for (int i = 0; i < kSlots; ++i) {
        if (slot[i]) (void)cudaFree(slot[i]);
        if (stream[i]) (void)cudaStreamDestroy(stream[i]);
        slot[i] = nullptr;
        stream[i] = nullptr;
    }
    if (aux) (void)cudaFree(aux);
    aux = nullptr;
    if (aux_ready) (void)cudaEventDestroy(aux_ready);
    aux_ready = nullptr;
    slot_bytes = aux_bytes = 0;
}

namespace {

constexpr uint64_t kChunkTargetBytes = 16ull << 20;  // per-slot staging target

inline uint64_t align256(uint64_t v) { return (v + 255u) & ~255ull; }

int runtime_ok(const axiom_runtime *rt) {
    if (!rt) return AXIOM_ERR_INVALID_ARGUMENT;
    return rt->backend == AXIOM_BACKEND_CUDA ? AXIOM_OK : AXIOM_ERR_UNSUPPORTED_BACKEND;
}

// rows per staged chunk: a multiple of `granule` rows, about kChunkTargetBytes
uint32_t chunk_rows_for(uint32_t rows, uint64_t bytes_per_row, uint32_t granule) {
    uint64_t r = kChunkTargetBytes / (bytes_per_row ? bytes_per_row : 1u);
    r = r / granule * granule;
    if (r < granule) r = granule;
    if (r > rows) r = rows;
    return (uint32_t)r;
}

// Device-side address of a host buffer the GPU can reach directly (page-locked and mapped: cudaHostAlloc,
// cudaHostRegister or a framework's pinned allocator under unified addressing); nullptr for pageable memory.
void *mapped_alias(const void *host) {
    // AXIOM_B200_HOST_IO=staged keeps every host buffer on the staged path (for hosts where device access to
    // page-locked memory is slower than the copy engines); read per call, like the reference's launch knobs
    const char *knob = getenv("AXIOM_B200_HOST_IO");
    if (knob && knob[0] == 's') return nullptr;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

int wait_all(staging_pool &p) {
    int rc = AXIOM_OK;
    for (int i = 0; i < staging_pool::kSlots; ++i) {
        if (cudaStreamSynchronize(p.stream[i]) != cudaSuccess) rc = AXIOM_ERR_CUDA;
    }
    return rc;
}

}  // namespace
}  // namespace axb

using namespace axb;

// ------------------------------------------------------------------------
// axiom_device_buffer flavour
// ------------------------------------------------------------------------

extern "C" uint32_t axiom_b200_pipeline_faults(int device) {
    if (select_device(device) != AXIOM_OK) return ~0u;
    if (cudaDeviceSynchronize() != cudaSuccess) return ~0u;
    return add_rmsnorm_fault_word() | swiglu_fault_word() | qk_fault_word();
}

extern "C" int axiom_b200_prepare(int device) {
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    prepare_add_rmsnorm_unit();
    prepare_qk_unit();
    const bool tables = prepare_gated_unit();
    if (cudaDeviceSynchronize() != cudaSuccess || cudaGetLastError() != cudaSuccess) return AXIOM_ERR_CUDA;
    return tables ? AXIOM_OK : AXIOM_ERR_CUDA;
}

extern "C" int axiom_runtime_nvfp4_quantize_bf16_device(
        axiom_runtime *runtime, const axiom_device_buffer *input, uint64_t input_offset, uint32_t rows,
        uint32_t cols, float global_scale, axiom_device_buffer *out_codes, uint64_t codes_offset,
        axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!input || !out_codes || !out_scales || rows == 0u || cols == 0u || (cols % kGroup) != 0u ||
        !valid_scale(global_scale) || scale_layout > AXIOM_SCALE_LAYOUT_TILED) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!owned_by(runtime, input) || !owned_by(runtime, out_codes) || !owned_by(runtime, out_scales)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    uint64_t in_bytes = 0;
    if (!mul_ok((uint64_t)rows * cols, 2u, &in_bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint64_t code_bytes = in_bytes / 4u;
    const uint64_t scale_bytes = axiom_nvfp4_scale_plane_bytes(rows, cols / kGroup, scale_layout);
    if (!span_ok(input, input_offset, in_bytes) || !span_ok(out_codes, codes_offset, code_bytes) ||
        !span_ok(out_scales, scales_offset, scale_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (ranges_overlap(input, input_offset, in_bytes, out_codes, codes_offset, code_bytes) ||
        ranges_overlap(input, input_offset, in_bytes, out_scales, scales_offset, scale_bytes) ||
        ranges_overlap(out_codes, codes_offset, code_bytes, out_scales, scales_offset, scale_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    rc = check_nvfp4_quantize(at(input, input_offset), rows, cols, global_scale, at(out_codes, codes_offset),
                              at(out_scales, scales_offset), scale_layout);
    if (rc != AXIOM_OK) return rc;
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    launch_nvfp4_quantize_bf16(at(input, input_offset), rows, cols, global_scale, at(out_codes, codes_offset),
                               at(out_scales, scales_offset), scale_layout, nullptr);
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_add_rmsnorm_nvfp4_bf16_device(
        axiom_runtime *runtime, const axiom_device_buffer *hidden, uint64_t hidden_offset,
        axiom_device_buffer *residual, uint64_t residual_offset, const axiom_device_buffer *gamma,
        uint64_t gamma_offset, float eps, uint32_t rows, uint32_t cols, float global_scale,
        axiom_device_buffer *norm_out, uint64_t norm_offset, axiom_device_buffer *out_codes,
        uint64_t codes_offset, axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!residual || !gamma || rows == 0u || cols == 0u || (cols % kGroup) != 0u || cols > 16384u ||
        scale_layout > AXIOM_SCALE_LAYOUT_TILED || (out_codes == nullptr) != (out_scales == nullptr) ||
        (!out_codes && !norm_out)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!(eps > 0.0f)) eps = 1.0e-6f;  // the generic wrappers default a non-positive eps (src/axiom_runtime.cpp:3406)
    if (!owned_by(runtime, residual) || !owned_by(runtime, gamma) || (hidden && !owned_by(runtime, hidden)) ||
        (norm_out && !owned_by(runtime, norm_out)) || (out_codes && !owned_by(runtime, out_codes)) ||
        (out_scales && !owned_by(runtime, out_scales))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    uint64_t act_bytes = 0;
    if (!mul_ok((uint64_t)rows * cols, 2u, &act_bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint64_t scale_bytes = axiom_nvfp4_scale_plane_bytes(rows, cols / kGroup, scale_layout);
    if (!span_ok(residual, residual_offset, act_bytes) || !span_ok(gamma, gamma_offset, (uint64_t)cols * 2u) ||
        (hidden && !span_ok(hidden, hidden_offset, act_bytes)) ||
        (norm_out && !span_ok(norm_out, norm_offset, act_bytes)) ||
        (out_codes && (!span_ok(out_codes, codes_offset, act_bytes / 4u) ||
                       !span_ok(out_scales, scales_offset, scale_bytes)))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((hidden && ranges_overlap(hidden, hidden_offset, act_bytes, residual, residual_offset, act_bytes)) ||
        (norm_out && ranges_overlap(norm_out, norm_offset, act_bytes, residual, residual_offset, act_bytes)) ||
        (out_codes && ranges_overlap(out_codes, codes_offset, act_bytes / 4u, residual, residual_offset, act_bytes)) ||
        (out_codes && ranges_overlap(out_codes, codes_offset, act_bytes / 4u, out_scales, scales_offset, scale_bytes))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((hidden_offset | residual_offset | gamma_offset | norm_offset) & 15u || (codes_offset & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    launch_add_rmsnorm_nvfp4_bf16(hidden ? at(hidden, hidden_offset) : nullptr, at(residual, residual_offset),
                                  at(gamma, gamma_offset), eps, rows, cols, global_scale,
                                  norm_out ? at(norm_out, norm_offset) : nullptr,
                                  out_codes ? at(out_codes, codes_offset) : nullptr,
                                  out_scales ? at(out_scales, scales_offset) : nullptr, scale_layout, nullptr);
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_swiglu_fp8_bf16_device(
        axiom_runtime *runtime, const axiom_device_buffer *gate_up, uint64_t gate_up_offset, uint32_t rows,
        uint32_t width, axiom_device_buffer *out_codes, uint64_t codes_offset, axiom_device_buffer *out_scales,
        uint64_t scales_offset) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!gate_up || !out_codes || !out_scales || rows == 0u || width == 0u || (width % 8u) != 0u || width > 36864u ||
        !owned_by(runtime, gate_up) || !owned_by(runtime, out_codes) || !owned_by(runtime, out_scales)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    uint64_t in_bytes = 0;
    if (!mul_ok((uint64_t)rows * width, 4u, &in_bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint64_t code_bytes = (uint64_t)rows * width;
    if (!span_ok(gate_up, gate_up_offset, in_bytes) || !span_ok(out_codes, codes_offset, code_bytes) ||
        !span_ok(out_scales, scales_offset, (uint64_t)rows * 4u) || (gate_up_offset & 15u) || (codes_offset & 7u) ||
        (scales_offset & 3u) ||
        ranges_overlap(gate_up, gate_up_offset, in_bytes, out_codes, codes_offset, code_bytes) ||
        ranges_overlap(gate_up, gate_up_offset, in_bytes, out_scales, scales_offset, (uint64_t)rows * 4u) ||
        ranges_overlap(out_codes, codes_offset, code_bytes, out_scales, scales_offset, (uint64_t)rows * 4u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    rc = launch_swiglu_fp8_bf16(at(gate_up, gate_up_offset), rows, width, at(out_codes, codes_offset),
                                (float *)at(out_scales, scales_offset), nullptr);
    return rc != AXIOM_OK ? rc : finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_swiglu_nvfp4_bf16_device(
        axiom_runtime *runtime, const axiom_device_buffer *gate_up, uint64_t gate_up_offset, uint32_t rows,
        uint32_t width, float global_scale, axiom_device_buffer *out_codes, uint64_t codes_offset,
        axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!gate_up || !out_codes || !out_scales || rows == 0u || width == 0u || (width % kGroup) != 0u ||
        !valid_scale(global_scale) || scale_layout > AXIOM_SCALE_LAYOUT_TILED || !owned_by(runtime, gate_up) ||
        !owned_by(runtime, out_codes) || !owned_by(runtime, out_scales) ||
        (uint64_t)rows * (width / 8u) > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    uint64_t in_bytes = 0;
    if (!mul_ok((uint64_t)rows * width, 4u, &in_bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    const uint64_t code_bytes = (uint64_t)rows * width / 2u;
    const uint64_t scale_bytes = axiom_nvfp4_scale_plane_bytes(rows, width / kGroup, scale_layout);
    if (!span_ok(gate_up, gate_up_offset, in_bytes) || !span_ok(out_codes, codes_offset, code_bytes) ||
        !span_ok(out_scales, scales_offset, scale_bytes) || (gate_up_offset & 15u) || (codes_offset & 3u) ||
        ranges_overlap(gate_up, gate_up_offset, in_bytes, out_codes, codes_offset, code_bytes) ||
        ranges_overlap(gate_up, gate_up_offset, in_bytes, out_scales, scales_offset, scale_bytes) ||
        ranges_overlap(out_codes, codes_offset, code_bytes, out_scales, scales_offset, scale_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    launch_swiglu_nvfp4_bf16(at(gate_up, gate_up_offset), rows, width, global_scale, at(out_codes, codes_offset),
                             at(out_scales, scales_offset), scale_layout, nullptr);
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_qknorm_rope_yarn_paged_bf16_device(
        axiom_runtime *runtime, const axiom_paged_kv_view *view, uint32_t layer, uint32_t n_active, uint32_t flags,
        axiom_device_buffer *q, uint64_t q_offset, const axiom_device_buffer *k, uint64_t k_offset,
        const axiom_device_buffer *v, uint64_t v_offset, const axiom_device_buffer *q_gamma, uint64_t q_gamma_offset,
        const axiom_device_buffer *k_gamma, uint64_t k_gamma_offset, const axiom_device_buffer *inv_freq,
        uint64_t inv_freq_offset, uint32_t q_heads, uint32_t k_heads, uint32_t head_dim, uint32_t rope_dim, float eps,
        float mscale, axiom_device_buffer *status_word, uint64_t status_offset) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!view || view->abi_version != AXIOM_ABI_VERSION || view->struct_size != sizeof(axiom_paged_kv_view)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (n_active == 0u || n_active > 65535u || n_active > view->cap || k_heads == 0u || !k || !k_gamma ||
        (flags & ~AXIOM_QK_FLAG_CACHE_E4M3) != 0u || (head_dim != 64u && head_dim != 128u && head_dim != 256u) ||
        view->tbl_stride == 0u || view->block_tokens == 0u || view->n_layers == 0u || layer >= view->n_layers ||
        view->kv_nphys == 0u || view->kv_dim < k_heads * head_dim || (view->kv_dim % 8u) != 0u ||
        (uint64_t)(q_heads + k_heads) * head_dim > (1u << 20) || (q_heads != 0u && (!q || !q_gamma)) ||
        (rope_dim != 0u && !inv_freq) || (v == nullptr) != (view->d_vpool == nullptr)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!owned_by(runtime, view->d_kpool) || !owned_by(runtime, view->d_tbl) || !owned_by(runtime, view->d_meta) ||
        !owned_by(runtime, k) || !owned_by(runtime, k_gamma) || (v && (!owned_by(runtime, v) || !owned_by(runtime, view->d_vpool))) ||
        (q_heads && (!owned_by(runtime, q) || !owned_by(runtime, q_gamma))) || (rope_dim && !owned_by(runtime, inv_freq)) ||
        (status_word && !owned_by(runtime, status_word))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    const uint64_t cell = (flags & AXIOM_QK_FLAG_CACHE_E4M3) ? 1u : 2u;
    uint64_t pool_rows = 0, pool_bytes = 0, tbl_bytes = 0;
    if (!mul_ok((uint64_t)view->kv_nphys * view->n_layers, view->block_tokens, &pool_rows) ||
        !mul_ok(pool_rows, (uint64_t)view->kv_dim * cell, &pool_bytes) ||
        !mul_ok((uint64_t)view->cap * view->tbl_stride, 4u, &tbl_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    const uint64_t q_bytes = (uint64_t)n_active * q_heads * head_dim * 2u, k_bytes = (uint64_t)n_active * k_heads * head_dim * 2u;
    if (!span_ok(view->d_kpool, 0u, pool_bytes) || (v && !span_ok(view->d_vpool, 0u, pool_bytes)) ||
        !span_ok(view->d_tbl, 0u, tbl_bytes) || !span_ok(view->d_meta, 0u, (uint64_t)view->cap * 8u) ||
        !span_ok(k, k_offset, k_bytes) || (k_offset & 15u) || (v && (!span_ok(v, v_offset, k_bytes) || (v_offset & 15u))) ||
        (q_heads && (!span_ok(q, q_offset, q_bytes) || (q_offset & 15u) ||
                     !span_ok(q_gamma, q_gamma_offset, (uint64_t)head_dim * 2u) || (q_gamma_offset & 1u))) ||
        !span_ok(k_gamma, k_gamma_offset, (uint64_t)head_dim * 2u) || (k_gamma_offset & 1u) ||
        (rope_dim && (!span_ok(inv_freq, inv_freq_offset, (uint64_t)(rope_dim / 2u) * 4u) || (inv_freq_offset & 3u))) ||
        (status_word && (!span_ok(status_word, status_offset, 4u) || (status_offset & 3u)))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    axiom_qk_rope_args a{};
    a.abi_version = AXIOM_ABI_VERSION;
    a.struct_size = sizeof a;
    a.tokens = n_active; a.q_heads = q_heads; a.k_heads = k_heads; a.head_dim = head_dim; a.rope_dim = rope_dim;
    a.flags = flags | AXIOM_QK_FLAG_PER_TOKEN_TABLE;
    a.eps = eps; a.mscale = mscale;
    a.block_tokens = view->block_tokens; a.n_layers = view->n_layers; a.layer = layer; a.pool_stride = view->kv_dim;
    a.tbl_stride = view->tbl_stride; a.n_blocks = view->kv_nphys;
    a.q_bf16 = q_heads ? at(q, q_offset) : nullptr;
    a.k_bf16 = at(k, k_offset);
    a.v_bf16 = v ? at(v, v_offset) : nullptr;
    a.q_gamma_bf16 = q_heads ? at(q_gamma, q_gamma_offset) : nullptr;
    a.k_gamma_bf16 = at(k_gamma, k_gamma_offset);
    a.inv_freq = rope_dim ? (const float *)at(inv_freq, inv_freq_offset) : nullptr;
    a.positions = (const uint32_t *)at(view->d_meta, (uint64_t)view->cap * 4u);
    a.block_tables = (const int32_t *)at(view->d_tbl, 0u);
    a.k_pool_bf16 = at(view->d_kpool, 0u);
    a.v_pool_bf16 = v ? at(view->d_vpool, 0u) : nullptr;
    a.status_word = status_word ? (uint32_t *)at(status_word, status_offset) : nullptr;
    rc = axiom_qwen38_fused_qk_norm_rope_paged_bf16_device((int)runtime->device, &a, nullptr);
    return rc != AXIOM_OK ? rc : finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_embedding_gather_bf16_device(
        axiom_runtime *runtime, const axiom_device_buffer *table, uint64_t table_offset, uint32_t vocab,
        uint32_t hidden, const axiom_device_buffer *token_ids, uint64_t ids_offset, uint32_t tokens,
        axiom_device_buffer *out, uint64_t out_offset) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!table || !token_ids || !out || vocab == 0u || hidden == 0u || (hidden % 8u) != 0u || tokens == 0u ||
        !owned_by(runtime, table) || !owned_by(runtime, token_ids) || !owned_by(runtime, out)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    uint64_t table_bytes = 0, out_bytes = 0;
    if (!mul_ok((uint64_t)vocab * hidden, 2u, &table_bytes) || !mul_ok((uint64_t)tokens * hidden, 2u, &out_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!span_ok(table, table_offset, table_bytes) || !span_ok(token_ids, ids_offset, (uint64_t)tokens * 4u) ||
        !span_ok(out, out_offset, out_bytes) || (table_offset & 15u) || (out_offset & 15u) || (ids_offset & 3u) ||
        ranges_overlap(table, table_offset, table_bytes, out, out_offset, out_bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    launch_embedding_gather_bf16(at(table, table_offset), vocab, hidden, (const uint32_t *)at(token_ids, ids_offset),
                                 tokens, at(out, out_offset), nullptr, nullptr);
    return finish_after_launch(nullptr);
}

// ------------------------------------------------------------------------
// host-I/O flavour: rows stream through three staging slots, each on its own
// stream, so upload / kernel / download of neighbouring chunks overlap.
// ------------------------------------------------------------------------

extern "C" int axiom_runtime_nvfp4_quantize_bf16(
        axiom_runtime *runtime, const void *input_bf16_host, uint32_t rows, uint32_t cols, float global_scale,
        uint8_t *out_codes_host, uint8_t *out_scales_host) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!input_bf16_host || !out_codes_host || !out_scales_host || rows == 0u || cols == 0u ||
        (cols % kGroup) != 0u || !valid_scale(global_scale)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    const uint64_t in_row = (uint64_t)cols * 2u, code_row = cols / 2u, scale_row = cols / kGroup;
    const uint32_t chunk = chunk_rows_for(rows, in_row + code_row + scale_row, 1u);
    const uint64_t off_codes = align256((uint64_t)chunk * in_row);
    const uint64_t off_scales = off_codes + align256((uint64_t)chunk * code_row);
    staging_pool &p = runtime->staging;
    if ((rc = p.reserve(0u, 0u)) != AXIOM_OK) return rc;  // the streams only: the mapped path stages nothing
    {   // page-locked, mapped buffers: the kernel reads and writes them itself (see the add+RMSNorm entry below).
        // One launch covers the tensor, so the launcher's 32-bit chunk count has to hold; larger inputs are staged
        // (the staged loop launches per chunk of rows).
        void *in_dev = mapped_alias(input_bf16_host), *codes_dev = mapped_alias(out_codes_host), *scales_dev = mapped_alias(out_scales_host);
        if (in_dev && codes_dev && scales_dev && aligned16(in_dev) && !(reinterpret_cast<uintptr_t>(codes_dev) & 3u) &&
            (uint64_t)rows * (cols / 8u) <= 0xffffffffull) {
            launch_nvfp4_quantize_bf16(in_dev, rows, cols, global_scale, (uint8_t *)codes_dev, (uint8_t *)scales_dev,
                                       AXIOM_SCALE_LAYOUT_CANONICAL, p.stream[0]);
            if (cudaStreamSynchronize(p.stream[0]) != cudaSuccess) return AXIOM_ERR_CUDA;
            return cudaGetLastError() == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA;
        }
    }
    if ((rc = p.reserve(off_scales + align256((uint64_t)chunk * scale_row), 0u)) != AXIOM_OK) return rc;
    uint32_t slot = 0;
    for (uint32_t r0 = 0; r0 < rows; r0 += chunk, slot = (slot + 1u) % staging_pool::kSlots) {
        const uint32_t n = std::min(chunk, rows - r0);
        uint8_t *dev = (uint8_t *)p.slot[slot];
        cudaStream_t s = p.stream[slot];
        cudaMemcpyAsync(dev, (const uint8_t *)input_bf16_host + (uint64_t)r0 * in_row, (size_t)n * in_row, cudaMemcpyHostToDevice, s);
        launch_nvfp4_quantize_bf16(dev, n, cols, global_scale, dev + off_codes, dev + off_scales, AXIOM_SCALE_LAYOUT_CANONICAL, s);
        cudaMemcpyAsync(out_codes_host + (uint64_t)r0 * code_row, dev + off_codes, (size_t)n * code_row, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(out_scales_host + (uint64_t)r0 * scale_row, dev + off_scales, (size_t)n * scale_row, cudaMemcpyDeviceToHost, s);
    }
    rc = wait_all(p);
    return cudaGetLastError() == cudaSuccess ? rc : AXIOM_ERR_CUDA;
}

extern "C" int axiom_runtime_add_rmsnorm_nvfp4_bf16(
        axiom_runtime *runtime, const void *hidden_bf16_host, void *residual_bf16_host,
        const void *gamma_bf16_host, float eps, uint32_t rows, uint32_t cols, float global_scale,
        uint8_t *out_codes_host, uint8_t *out_scales_host) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!hidden_bf16_host || !residual_bf16_host || !gamma_bf16_host || !out_codes_host || !out_scales_host ||
        rows == 0u || cols == 0u || (cols % kGroup) != 0u || cols > 16384u || !valid_scale(global_scale)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!(eps > 0.0f)) eps = 1.0e-6f;
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    const uint64_t act_row = (uint64_t)cols * 2u, code_row = cols / 2u, scale_row = cols / kGroup;
    const uint32_t chunk = chunk_rows_for(rows, 2u * act_row + code_row + scale_row, 1u);
    const uint64_t off_res = align256((uint64_t)chunk * act_row);
    const uint64_t off_codes = off_res + align256((uint64_t)chunk * act_row);
    const uint64_t off_scales = off_codes + align256((uint64_t)chunk * code_row);
    staging_pool &p = runtime->staging;
    if ((rc = p.reserve(0u, align256(act_row))) != AXIOM_OK) return rc;  // streams and the gamma buffer; slots only when staging
    // gamma is resident for the whole call.  It is uploaded on slot stream 0 and the other slot streams wait for the
    // event behind it: the slot streams are non-blocking, so nothing else orders them after the copy.
    if (cudaMemcpyAsync(p.aux, gamma_bf16_host, (size_t)act_row, cudaMemcpyHostToDevice, p.stream[0]) != cudaSuccess ||
        cudaEventRecord(p.aux_ready, p.stream[0]) != cudaSuccess) {
        return AXIOM_ERR_CUDA;
    }
    for (int i = 1; i < staging_pool::kSlots; ++i) {
        if (cudaStreamWaitEvent(p.stream[i], p.aux_ready, 0) != cudaSuccess) return AXIOM_ERR_CUDA;
    }
    // Page-locked, mapped host buffers are read and written by the kernel itself: one launch whose bulk copies cross
    // the bus in both directions at once, with no staging and no per-chunk copy set-up (about 8 us of idle link per
    // copy on the engines).  Rows must be 16-byte multiples for the bulk copies; anything else is staged.
    void *hidden_dev = mapped_alias(hidden_bf16_host), *res_dev = mapped_alias(residual_bf16_host);
    void *codes_dev = mapped_alias(out_codes_host), *scales_dev = mapped_alias(out_scales_host);
    if (hidden_dev && res_dev && codes_dev && scales_dev && aligned16(hidden_dev) && aligned16(res_dev) &&
        !(reinterpret_cast<uintptr_t>(codes_dev) & 3u)) {
        cudaStream_t s = p.stream[0];
        launch_add_rmsnorm_nvfp4_bf16(hidden_dev, res_dev, p.aux, eps, rows, cols, global_scale, nullptr, (uint8_t *)codes_dev,
                                      (uint8_t *)scales_dev, AXIOM_SCALE_LAYOUT_CANONICAL, s);
        if (cudaStreamSynchronize(s) != cudaSuccess) return AXIOM_ERR_CUDA;
        return cudaGetLastError() == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA;
    }
    if ((rc = p.reserve(off_scales + align256((uint64_t)chunk * scale_row), align256(act_row))) != AXIOM_OK) {
        (void)wait_all(p);  // the gamma upload is still in flight
        return rc;
    }
    uint32_t slot = 0;
    for (uint32_t r0 = 0; r0 < rows; r0 += chunk, slot = (slot + 1u) % staging_pool::kSlots) {
        const uint32_t n = std::min(chunk, rows - r0);
        uint8_t *dev = (uint8_t *)p.slot[slot];
        cudaStream_t s = p.stream[slot];
        uint8_t *res_host = (uint8_t *)residual_bf16_host + (uint64_t)r0 * act_row;
        cudaMemcpyAsync(dev, (const uint8_t *)hidden_bf16_host + (uint64_t)r0 * act_row, (size_t)n * act_row, cudaMemcpyHostToDevice, s);
        cudaMemcpyAsync(dev + off_res, res_host, (size_t)n * act_row, cudaMemcpyHostToDevice, s);
        launch_add_rmsnorm_nvfp4_bf16(dev, dev + off_res, p.aux, eps, n, cols, global_scale, nullptr, dev + off_codes,
                                      dev + off_scales, AXIOM_SCALE_LAYOUT_CANONICAL, s);
        cudaMemcpyAsync(res_host, dev + off_res, (size_t)n * act_row, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(out_codes_host + (uint64_t)r0 * code_row, dev + off_codes, (size_t)n * code_row, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(out_scales_host + (uint64_t)r0 * scale_row, dev + off_scales, (size_t)n * scale_row, cudaMemcpyDeviceToHost, s);
    }
    rc = wait_all(p);
    return cudaGetLastError() == cudaSuccess ? rc : AXIOM_ERR_CUDA;
}

extern "C" int axiom_runtime_swiglu_fp8_bf16(
        axiom_runtime *runtime, const void *gate_up_bf16_host, uint32_t rows, uint32_t width,
        uint8_t *out_codes_host, float *out_scales_host) {
    int rc = runtime_ok(runtime);
    if (rc != AXIOM_OK) return rc;
    if (!gate_up_bf16_host || !out_codes_host || !out_scales_host || rows == 0u || width == 0u ||
        (width % 8u) != 0u || width > 36864u) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((rc = select_device((int)runtime->device)) != AXIOM_OK) return rc;
    const uint64_t in_row = (uint64_t)width * 4u, code_row = width;
    const uint32_t chunk = chunk_rows_for(rows, in_row + code_row + 4u, 1u);
    const uint64_t off_codes = align256((uint64_t)chunk * in_row);
    const uint64_t off_scales = off_codes + align256((uint64_t)chunk * code_row);
    staging_pool &p = runtime->staging;
    if ((rc = p.reserve(0u, 0u)) != AXIOM_OK) return rc;  // the streams only: the mapped path stages nothing
    {   // page-locked, mapped buffers: the kernel reads and writes them itself
        void *in_dev = mapped_alias(gate_up_bf16_host), *codes_dev = mapped_alias(out_codes_host), *scales_dev = mapped_alias(out_scales_host);
        if (in_dev && codes_dev && scales_dev && aligned16(in_dev) && !(reinterpret_cast<uintptr_t>(codes_dev) & 7u)) {
            rc = launch_swiglu_fp8_bf16(in_dev, rows, width, (uint8_t *)codes_dev, (float *)scales_dev, p.stream[0]);
            if (cudaStreamSynchronize(p.stream[0]) != cudaSuccess) return AXIOM_ERR_CUDA;
            return cudaGetLastError() == cudaSuccess ? rc : AXIOM_ERR_CUDA;
        }
    }
    if ((rc = p.reserve(off_scales + align256((uint64_t)chunk * 4u), 0u)) != AXIOM_OK) return rc;
    uint32_t slot = 0;
    for (uint32_t r0 = 0; r0 < rows; r0 += chunk, slot = (slot + 1u) % staging_pool::kSlots) {
        const uint32_t n = std::min(chunk, rows - r0);
        uint8_t *dev = (uint8_t *)p.slot[slot];
        cudaStream_t s = p.stream[slot];
        cudaMemcpyAsync(dev, (const uint8_t *)gate_up_bf16_host + (uint64_t)r0 * in_row, (size_t)n * in_row, cudaMemcpyHostToDevice, s);
        launch_swiglu_fp8_bf16(dev, n, width, dev + off_codes, (float *)(dev + off_scales), s);
        cudaMemcpyAsync(out_codes_host + (uint64_t)r0 * code_row, dev + off_codes, (size_t)n * code_row, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(out_scales_host + r0, dev + off_scales, (size_t)n * 4u, cudaMemcpyDeviceToHost, s);
    }
    rc = wait_all(p);
    return cudaGetLastError() == cudaSuccess ? rc : AXIOM_ERR_CUDA;
}

// Private handle layouts and host-side helpers shared by the ABI translation units.
#pragma once

#include "common.cuh"

namespace axb {

// Device staging for the host-I/O entry points: a ring of `kSlots` chunk
// buffers, each with its own stream, grown on demand and kept by the runtime so
// steady-state calls allocate nothing.
struct staging_pool {
    static constexpr int kSlots = 3;
    void *slot[kSlots] = {nullptr, nullptr, nullptr};
    uint64_t slot_bytes = 0;
    cudaStream_t stream[kSlots] = {nullptr, nullptr, nullptr};
    void *aux = nullptr;       // small resident operands (gamma, tables)
    uint64_t aux_bytes = 0;
    cudaEvent_t aux_ready = nullptr;  // recorded on stream[0] after an upload into aux; the other slot streams wait on it

    int reserve(uint64_t bytes_per_slot, uint64_t aux_need);
    void release();
};

}  // namespace axb

struct axiom_runtime {
    axiom_backend backend = AXIOM_BACKEND_CUDA;
    uint32_t device = 0;
    uint32_t sm_count = 0;
    axb::staging_pool staging;
};

struct axiom_device_buffer {
    axiom_runtime *runtime = nullptr;
    void *ptr = nullptr;
    uint32_t device = 0;
    uint64_t bytes = 0;
};

namespace axb {

bool span_ok(const axiom_device_buffer *buffer, uint64_t offset, uint64_t bytes);
bool mul_ok(uint64_t a, uint64_t b, uint64_t *out);
bool ranges_overlap(const axiom_device_buffer *a, uint64_t a_off, uint64_t a_bytes,
                    const axiom_device_buffer *b, uint64_t b_off, uint64_t b_bytes);

inline bool owned_by(const axiom_runtime *rt, const axiom_device_buffer *b) { return b && b->runtime == rt; }

inline uint8_t *at(const axiom_device_buffer *b, uint64_t offset) { return (uint8_t *)b->ptr + offset; }

// ---- launchers implemented next to their kernels (all asynchronous on `stream`) ----
int launch_nvfp4_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, float G, uint8_t *codes,
                               uint8_t *scales, uint32_t layout, cudaStream_t stream);
int launch_nvfp4_quantize_f32_row(const float *input, float G, uint8_t *codes, uint8_t *scales, uint32_t cols,
                                  cudaStream_t stream);
int launch_add_bf16(const void *a, const void *b, void *out, uint64_t count, cudaStream_t stream);
int launch_add_rmsnorm_nvfp4_bf16(const void *hidden, void *residual, const void *gamma, float eps, uint32_t rows,
                                  uint32_t cols, float G, void *norm_out, uint8_t *codes, uint8_t *scales,
                                  uint32_t layout, cudaStream_t stream);
int launch_add_rmsnorm_tap_nvfp4_bf16(const void *hidden, void *residual, const void *gamma, float eps, uint32_t rows,
                                      uint32_t cols, float G, void *norm_out, uint8_t *codes, uint8_t *scales,
                                      uint32_t layout, void *tap, cudaStream_t stream);
int launch_gather_add_rmsnorm_nvfp4_bf16(const void *table, uint32_t vocab, const uint32_t *token_ids, void *residual,
                                         const void *gamma, float eps, uint32_t rows, uint32_t cols, float G,
                                         void *norm_out, uint8_t *codes, uint8_t *scales, uint32_t layout,
                                         uint32_t *status_word, cudaStream_t stream);
int launch_swiglu_fp8_bf16(const void *gate_up, uint32_t rows, uint32_t width, uint8_t *codes, float *scales,
                           cudaStream_t stream);
int launch_swiglu_nvfp4_bf16(const void *gate_up, uint32_t rows, uint32_t width, float G, uint8_t *codes,
                             uint8_t *scales, uint32_t layout, cudaStream_t stream);
int launch_sigmoid_gate_nvfp4_bf16(const void *attention, const void *gate, uint32_t rows, uint32_t width, float G,
                                   void *out_bf16, uint8_t *codes, uint8_t *scales, uint32_t layout, cudaStream_t stream);
int launch_sigmoid_gate_heads_nvfp4_bf16(const void *attention, const void *q_gate, uint32_t rows, uint32_t heads,
                                         uint32_t head_dim, float G, void *out_bf16, uint8_t *codes, uint8_t *scales,
                                         uint32_t layout, cudaStream_t stream);
int launch_fp8_quantize_bf16(const void *input, uint32_t rows, uint32_t cols, uint8_t *codes, float *scales,
                             uint32_t *status_word, cudaStream_t stream);
int launch_embedding_gather_bf16(const void *table, uint32_t vocab, uint32_t hidden, const uint32_t *ids,
                                 uint32_t tokens, void *out, uint32_t *status_word, cudaStream_t stream);
int launch_yarn_inv_freq(const axiom_rope_config *config, float *out, cudaStream_t stream);
int launch_qk_norm_rope_paged_bf16(const axiom_qk_rope_args *args, cudaStream_t stream);

// bounded-wait fault words of the pipelined kernels (read-and-clear, synchronising)
unsigned int add_rmsnorm_fault_word();
unsigned int swiglu_fault_word();
unsigned int qk_fault_word();
// one-time set-up of each unit on the current device (axiom_b200_prepare)
void prepare_add_rmsnorm_unit();
void prepare_qk_unit();
bool prepare_gated_unit();

// argument validation shared by the raw, buffer and host flavours
int check_nvfp4_quantize(const void *input, uint32_t rows, uint32_t cols, float G, const void *codes,
                         const void *scales, uint32_t layout);

}  // namespace axb

// Token-embedding gather and the BF16 residual add.
//   gather: qwen38_embedding_gather_columns_kernel (src/axiom_qwen38_model.cu:321-341),
//           BF16 rows copied as BF16; an id at or beyond the vocabulary gives a zero row.
//   add:    qwen38_add_bf16_inplace_kernel (src/axiom_qwen38_model.cu:175-184).
#include "runtime.hpp"

namespace axb {

namespace {

constexpr uint32_t kThreads = 256u;

__global__ void __launch_bounds__(kThreads)
embedding_gather_bf16_kernel(const uint4 *__restrict__ table, uint32_t vocab, uint32_t chunks_per_row,
                             const uint32_t *__restrict__ ids, uint32_t tokens, uint4 *__restrict__ out,
                             uint32_t *__restrict__ status_word) {
    allow_dependents();
    dependency_wait();
    const uint64_t total = (uint64_t)tokens * chunks_per_row;
    for (uint64_t c = (uint64_t)blockIdx.x * kThreads + threadIdx.x; c < total; c += (uint64_t)gridDim.x * kThreads) {
        const uint32_t token = (uint32_t)(c / chunks_per_row);
        const uint32_t q = (uint32_t)(c - (uint64_t)token * chunks_per_row);
        const uint32_t id = ids[token];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (id < vocab) {
            v = ld_stream(table + (uint64_t)id * chunks_per_row + q);
        } else if (q == 0u && status_word) {
            atomicCAS(status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
        }
        st_stream(out + c, v);
    }
}

__global__ void __launch_bounds__(kThreads)
add_bf16_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ out, uint64_t chunks,
                const uint16_t *a_tail, const uint16_t *b_tail, uint16_t *out_tail, uint32_t tail) {
    allow_dependents();
    dependency_wait();
    for (uint64_t c = (uint64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (uint64_t)gridDim.x * kThreads) {
        const uint4 x = ld_stream(a + c), y = ld_stream(b + c);
        uint4 r;
        r.x = pack_bf16x2(__fadd_rn(bf16_lo(x.x), bf16_lo(y.x)), __fadd_rn(bf16_hi(x.x), bf16_hi(y.x)));
        r.y = pack_bf16x2(__fadd_rn(bf16_lo(x.y), bf16_lo(y.y)), __fadd_rn(bf16_hi(x.y), bf16_hi(y.y)));
        r.z = pack_bf16x2(__fadd_rn(bf16_lo(x.z), bf16_lo(y.z)), __fadd_rn(bf16_hi(x.z), bf16_hi(y.z)));
        r.w = pack_bf16x2(__fadd_rn(bf16_lo(x.w), bf16_lo(y.w)), __fadd_rn(bf16_hi(x.w), bf16_hi(y.w)));
        st_stream(out + c, r);
    }
    if (blockIdx.x == 0u && threadIdx.x < tail) {
        const float s = __fadd_rn(__uint_as_float((uint32_t)a_tail[threadIdx.x] << 16),
                                  __uint_as_float((uint32_t)b_tail[threadIdx.x] << 16));
        out_tail[threadIdx.x] = (uint16_t)(pack_bf16x2(s, 0.0f) & 0xffffu);
    }
}

uint32_t grid_for(uint64_t work_items) {
    uint64_t blocks = (work_items + kThreads - 1u) / kThreads;
    const uint64_t cap = (uint64_t)kSmCount * 16u;
    if (blocks > cap) blocks = cap;
    return blocks ? (uint32_t)blocks : 1u;
}

}  // namespace

int launch_embedding_gather_bf16(const void *table, uint32_t vocab, uint32_t hidden, const uint32_t *ids,
                                 uint32_t tokens, void *out, uint32_t *status_word, cudaStream_t stream) {
    const uint32_t chunks_per_row = hidden / 8u;
    launch_chained(embedding_gather_bf16_kernel, dim3(grid_for((uint64_t)tokens * chunks_per_row)), dim3(kThreads), 0, stream, 
            (const uint4 *)table, vocab, chunks_per_row, ids, tokens, (uint4 *)out, status_word);
    note_launch();
    return AXIOM_OK;
}

int launch_add_bf16(const void *a, const void *b, void *out, uint64_t count, cudaStream_t stream) {
    const uint64_t chunks = count / 8u;
    const uint32_t tail = (uint32_t)(count - chunks * 8u);
    launch_chained(add_bf16_kernel, dim3(grid_for(chunks)), dim3(kThreads), 0, stream, 
            (const uint4 *)a, (const uint4 *)b, (uint4 *)out, chunks, (const uint16_t *)a + chunks * 8u,
            (const uint16_t *)b + chunks * 8u, (uint16_t *)out + chunks * 8u, tail);
    note_launch();
    return AXIOM_OK;
}

}  // namespace axb

using namespace axb;

extern "C" int axiom_qwen38_fused_embedding_gather_bf16_device(
        int device, const void *table_bf16, uint32_t vocab, uint32_t hidden, const uint32_t *token_ids,
        uint32_t tokens, void *out_bf16, uint32_t *status_word, void *stream) {
    if (!table_bf16 || !token_ids || !out_bf16 || vocab == 0u || hidden == 0u || (hidden % 8u) != 0u ||
        tokens == 0u || !aligned16(table_bf16) || !aligned16(out_bf16)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_embedding_gather_bf16(table_bf16, vocab, hidden, token_ids, tokens, out_bf16, status_word, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_add_bf16_device(int device, const void *a_bf16, const void *b_bf16,
                                                  void *out_bf16, uint64_t count, void *stream) {
    if (!a_bf16 || !b_bf16 || !out_bf16 || count == 0u || !aligned16(a_bf16) || !aligned16(b_bf16) ||
        !aligned16(out_bf16)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_bf16(a_bf16, b_bf16, out_bf16, count, (cudaStream_t)stream);
    return launch_status();
}

// Generic single-row F32 RoPE / fused qk-norm + RoPE ops of the runtime ABI,
// precise unit (no fast-math, as the reference builds its precise unit:
// reference Makefile:73).
//   NeoX RoPE, full and partial      src/axiom_cuda_precise.cu:39-97
//   per-head RMSNorm x weight + RoPE src/axiom_cuda_precise.cu:105-235
// freq = powf(theta, -2*i/n_rot), angle = (float)pos * freq, pairs (i, i+n_rot/2),
// FP64 sum of squares through a power-of-two tree, no BF16 rounding, no YaRN.
#include "runtime.hpp"

namespace axb {
namespace {

__device__ __forceinline__ void rotate_pair(float *row, uint32_t i, uint32_t half, uint32_t n_rot, float a, float b,
                                            uint32_t pos, float theta) {
    const float freq = powf(theta, -2.0f * (float)i / (float)n_rot);
    const float ang = (float)pos * freq;
    const float c = cosf(ang), s = sinf(ang);
    row[i] = a * c - b * s;
    row[i + half] = a * s + b * c;
}

__global__ void rope_neox_kernel(float *x, uint32_t head_dim, uint32_t n_rot, uint32_t pos, float theta) {
    float *row = x + (uint64_t)blockIdx.x * head_dim;
    const uint32_t half = n_rot / 2u;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) rotate_pair(row, i, half, n_rot, row[i], row[i + half], pos, theta);
}

// grid = q_heads + k_heads (k part may be empty), block = head_dim threads,
// dynamic shared = head_dim doubles + head_dim floats.
__global__ void qknorm_rope_kernel(float *q, const float *qw, float *k, const float *kw, uint32_t q_heads,
                                   uint32_t head_dim, uint32_t pos_value, const uint32_t *pos_ptr, float theta,
                                   float eps) {
    extern __shared__ double cell[];
    float *normed = reinterpret_cast<float *>(cell + head_dim);
    const uint32_t tid = threadIdx.x;
    const bool is_q = blockIdx.x < q_heads;
    float *row = is_q ? q + (uint64_t)blockIdx.x * head_dim : k + (uint64_t)(blockIdx.x - q_heads) * head_dim;
    const float *w = is_q ? qw : kw;
    const uint32_t pos = pos_ptr ? pos_ptr[0] : pos_value;
    const float v = row[tid];
    cell[tid] = (double)v * (double)v;
    __syncthreads();
    for (uint32_t stride = head_dim >> 1; stride > 0u; stride >>= 1u) {
        if (tid < stride) cell[tid] += cell[tid + stride];
        __syncthreads();
    }
    const float inv = (float)(1.0 / sqrt(cell[0] / (double)head_dim + (double)eps));
    normed[tid] = v * inv * w[tid];
    __syncthreads();
    const uint32_t half = head_dim >> 1;
    if (tid < half) rotate_pair(row, tid, half, head_dim, normed[tid], normed[tid + half], pos, theta);
}

bool f32_span(const axiom_device_buffer *b, uint64_t off, uint64_t count) {
    uint64_t bytes = 0;
    return mul_ok(count, sizeof(float), &bytes) && span_ok(b, off, bytes);
}

bool pow2_le_1024(uint32_t v) { return v != 0u && (v & (v - 1u)) == 0u && v <= 1024u; }

int rope_entry(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, uint32_t heads, uint32_t head_dim,
               uint32_t n_rot, uint32_t pos, float theta) {
    if (!rt || !x || heads == 0u || head_dim == 0u || (head_dim & 1u) || n_rot == 0u || (n_rot & 1u) || n_rot > head_dim) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA || !owned_by(rt, x) || !f32_span(x, x_off, (uint64_t)heads * head_dim)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device((int)rt->device);
    if (rc != AXIOM_OK) return rc;
    rope_neox_kernel<<<heads, 256>>>((float *)at(x, x_off), head_dim, n_rot, pos, theta);
    note_launch();
    return finish_after_launch(nullptr);
}

int qknorm_entry(axiom_runtime *rt, axiom_device_buffer *q, uint64_t q_off, const axiom_device_buffer *qw, uint64_t qw_off,
                 axiom_device_buffer *k, uint64_t k_off, const axiom_device_buffer *kw, uint64_t kw_off,
                 const axiom_device_buffer *pos, uint64_t pos_off, uint32_t pos_value, uint32_t q_heads,
                 uint32_t k_heads, uint32_t head_dim, float theta, float eps) {
    if (!rt || !q || !qw || q_heads == 0u || head_dim == 0u || eps <= 0.0f) return AXIOM_ERR_INVALID_ARGUMENT;
    if (rt->backend != AXIOM_BACKEND_CUDA || !owned_by(rt, q) || !owned_by(rt, qw) || (pos && !owned_by(rt, pos)) ||
        (k && (!owned_by(rt, k) || !kw || !owned_by(rt, kw)))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!f32_span(q, q_off, (uint64_t)q_heads * head_dim) || !f32_span(qw, qw_off, head_dim) ||
        (k && (!f32_span(k, k_off, (uint64_t)k_heads * head_dim) || !f32_span(kw, kw_off, head_dim))) ||
        (pos && !span_ok(pos, pos_off, sizeof(uint32_t)))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!pow2_le_1024(head_dim)) return AXIOM_ERR_INVALID_ARGUMENT;  // src/axiom_cuda.cu:15274-15276
    int rc = select_device((int)rt->device);
    if (rc != AXIOM_OK) return rc;
    const size_t shared = (size_t)head_dim * (sizeof(double) + sizeof(float));
    qknorm_rope_kernel<<<q_heads + (k ? k_heads : 0u), head_dim, shared>>>(
            (float *)at(q, q_off), (const float *)at(qw, qw_off), k ? (float *)at(k, k_off) : nullptr,
            k ? (const float *)at(kw, kw_off) : nullptr, q_heads, head_dim, pos_value,
            pos ? (const uint32_t *)at(pos, pos_off) : nullptr, theta, eps);
    note_launch();
    return finish_after_launch(nullptr);
}

}  // namespace
}  // namespace axb

using namespace axb;

extern "C" int axiom_runtime_rope_neox_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, uint32_t heads, uint32_t head_dim, uint32_t pos, float theta) {
    return rope_entry(rt, x, x_off, heads, head_dim, head_dim, pos, theta);
}

extern "C" int axiom_runtime_rope_neox_partial_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, uint32_t heads, uint32_t head_dim, uint32_t n_rot, uint32_t pos, float theta) {
    return rope_entry(rt, x, x_off, heads, head_dim, n_rot, pos, theta);
}

extern "C" int axiom_runtime_qknorm_rope_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, const axiom_device_buffer *w, uint64_t w_off, uint32_t heads, uint32_t head_dim, uint32_t pos, float theta, float eps) {
    return qknorm_entry(rt, x, x_off, w, w_off, nullptr, 0, nullptr, 0, nullptr, 0, pos, heads, 0u, head_dim, theta, eps);
}

extern "C" int axiom_runtime_qknorm_rope_pos_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, const axiom_device_buffer *w, uint64_t w_off, const axiom_device_buffer *pos, uint64_t pos_off, uint32_t heads, uint32_t head_dim, float theta, float eps) {
    if (!pos) return AXIOM_ERR_INVALID_ARGUMENT;
    return qknorm_entry(rt, x, x_off, w, w_off, nullptr, 0, nullptr, 0, pos, pos_off, 0u, heads, 0u, head_dim, theta, eps);
}

extern "C" int axiom_runtime_qknorm_rope_pos_dual_f32_device(axiom_runtime *rt, axiom_device_buffer *q, uint64_t q_off, const axiom_device_buffer *qw, uint64_t qw_off, axiom_device_buffer *k, uint64_t k_off, const axiom_device_buffer *kw, uint64_t kw_off, const axiom_device_buffer *pos, uint64_t pos_off, uint32_t q_heads, uint32_t k_heads, uint32_t head_dim, float theta, float eps) {
    if (!k || !kw || !pos || k_heads == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    return qknorm_entry(rt, q, q_off, qw, qw_off, k, k_off, kw, kw_off, pos, pos_off, 0u, q_heads, k_heads, head_dim, theta, eps);
}

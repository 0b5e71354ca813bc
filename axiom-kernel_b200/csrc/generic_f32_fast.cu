// Generic single-row F32 device ops of the runtime ABI, fast-math unit.
//
// The reference builds its generic backend with --use_fast_math
// (reference Makefile:17), so these kernels are compiled with the same flag:
// products feeding sums contract to FMA, x/y and rsqrtf are the approximate
// forms, denormals flush.  Expressions keep the reference's operand order:
//   rmsnorm      src/axiom_cuda.cu:14530-14551   float partials, 256-wide tree
//   rmsnorm hp   src/axiom_cuda.cu:14556-14577   double partials
//   rmsnorm b1   src/axiom_cuda.cu:14583-14655   float4 + shuffle
//   rmsnorm dual src/axiom_cuda.cu:14657-14685   two rows
//   head norm    src/axiom_cuda.cu:15119-15141   weightless, in place
//   qk norm w    src/axiom_cuda.cu:15347-15366   double partials, weight
//   add          src/axiom_cuda.cu:15803-15810
//   silu*up      src/axiom_cuda.cu:17278-17293   optional clamp
//   paged store  src/axiom_cuda.cu:16954-16969
// All launch on the legacy default stream and then follow the
// finish-after-launch convention.
#include "runtime.hpp"

#include <cuda_fp16.h>

namespace axb {
namespace {

constexpr uint32_t kT = 256u;

// Tree over 256 shared cells, every level through shared memory; result in cell[0].
template <typename T>
__device__ __forceinline__ void tree256(T *cell, uint32_t tid) {
    __syncthreads();
    for (uint32_t stride = kT / 2u; stride > 0u; stride >>= 1u) {
        if (tid < stride) cell[tid] += cell[tid + stride];
        __syncthreads();
    }
}

enum class sum_kind { f32, f64 };

template <sum_kind K>
__device__ __forceinline__ float inverse_rms(const float *x, uint32_t count, float eps, uint32_t tid) {
    if (K == sum_kind::f32) {
        __shared__ float cell[kT];
        float ss = 0.0f;
        for (uint32_t i = tid; i < count; i += kT) ss += x[i] * x[i];
        cell[tid] = ss;
        tree256(cell, tid);
        return rsqrtf(cell[0] / (float)count + eps);
    }
    __shared__ double dcell[kT];
    double ss = 0.0;
    for (uint32_t i = tid; i < count; i += kT) {
        const double v = (double)x[i];
        ss += v * v;
    }
    dcell[tid] = ss;
    tree256(dcell, tid);
    return (float)(1.0 / sqrt(dcell[0] / (double)count + (double)eps));
}

// grid.x rows: row r reads in[r], writes out[r]; w == nullptr means weightless.
template <sum_kind K>
__global__ void __launch_bounds__(kT)
rmsnorm_rows_kernel(const float *w, const float *in0, float *out0, const float *in1, float *out1,
                    uint64_t row_stride, uint32_t count, float eps) {
    const uint32_t tid = threadIdx.x;
    const float *in = in1 ? (blockIdx.x == 0u ? in0 : in1) : in0 + blockIdx.x * row_stride;
    float *out = in1 ? (blockIdx.x == 0u ? out0 : out1) : out0 + blockIdx.x * row_stride;
    const float inv = inverse_rms<K>(in, count, eps, tid);
    if (w) {
        for (uint32_t i = tid; i < count; i += kT) out[i] = in[i] * inv * w[i];
    } else {
        for (uint32_t i = tid; i < count; i += kT) out[i] = in[i] * inv;
    }
}

__global__ void __launch_bounds__(kT)
rmsnorm_b1_kernel(const float *w, const float *in, float *out, uint32_t count, float eps) {
    __shared__ float warp_sum[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t vec = count >> 2, tail = vec << 2;
    const bool in_vec = (reinterpret_cast<uintptr_t>(in) & 15u) == 0u;
    const bool all_vec = in_vec && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0u;
    float ss = 0.0f;
    if (in_vec) {
        const float4 *in4 = reinterpret_cast<const float4 *>(in);
        for (uint32_t i = tid; i < vec; i += kT) {
            const float4 v = in4[i];
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
        for (uint32_t i = tail + tid; i < count; i += kT) ss = fmaf(in[i], in[i], ss);
    } else {
        for (uint32_t i = tid; i < count; i += kT) ss = fmaf(in[i], in[i], ss);
    }
#pragma unroll
    for (uint32_t off = 16u; off > 0u; off >>= 1u) ss += __shfl_down_sync(0xffffffffu, ss, off);
    if (lane == 0u) warp_sum[warp] = ss;
    __syncthreads();
    ss = (warp == 0u && lane < 8u) ? warp_sum[lane] : 0.0f;
    if (warp == 0u) {
#pragma unroll
        for (uint32_t off = 16u; off > 0u; off >>= 1u) ss += __shfl_down_sync(0xffffffffu, ss, off);
        if (lane == 0u) warp_sum[0] = ss;
    }
    __syncthreads();
    const float inv = rsqrtf(warp_sum[0] / (float)count + eps);
    if (all_vec) {
        const float4 *in4 = reinterpret_cast<const float4 *>(in);
        const float4 *w4 = reinterpret_cast<const float4 *>(w);
        float4 *out4 = reinterpret_cast<float4 *>(out);
        for (uint32_t i = tid; i < vec; i += kT) {
            const float4 v = in4[i], g = w4[i];
            out4[i] = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
        }
        for (uint32_t i = tail + tid; i < count; i += kT) out[i] = in[i] * inv * w[i];
        return;
    }
    for (uint32_t i = tid; i < count; i += kT) out[i] = in[i] * inv * w[i];
}

__global__ void add_kernel(const float *a, const float *b, float *out, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = a[i] + b[i];
}

__global__ void silu_mul_kernel(const float *gate, const float *up, float *out, uint32_t count, float clamp_abs) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float g = gate[i], u = up[i];
    if (clamp_abs > 1.0e-6f) {
        g = fminf(g, clamp_abs);
        u = fminf(fmaxf(u, -clamp_abs), clamp_abs);
    }
    out[i] = (g / (1.0f + expf(-g))) * u;
}

__global__ void kv_store_paged_kernel(const float *k_stage, const float *v_stage, float *k_pool, float *v_pool,
                                      const int32_t *tables, const uint32_t *pos, uint32_t tbl_stride,
                                      uint32_t n_layers, uint32_t layer, uint32_t block_tokens,
                                      uint32_t pool_stride, uint32_t kv_dim) {
    const uint32_t seq = blockIdx.y;
    const uint32_t p = pos[seq];
    const uint32_t block = (uint32_t)tables[(uint64_t)seq * tbl_stride + p / block_tokens];
    const uint64_t dst = (((uint64_t)block * n_layers + layer) * block_tokens + p % block_tokens) * pool_stride;
    const uint64_t src = (uint64_t)seq * kv_dim;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < kv_dim; i += gridDim.x * blockDim.x) {
        k_pool[dst + i] = k_stage[src + i];
        v_pool[dst + i] = v_stage[src + i];
    }
}

int begin(axiom_runtime *rt) {
    if (!rt) return AXIOM_ERR_INVALID_ARGUMENT;
    return select_device((int)rt->device);
}

bool f32_span(const axiom_device_buffer *b, uint64_t off, uint64_t count) {
    uint64_t bytes = 0;
    return mul_ok(count, sizeof(float), &bytes) && span_ok(b, off, bytes);
}

const float *cf(const axiom_device_buffer *b, uint64_t off) { return (const float *)at(b, off); }
float *mf(axiom_device_buffer *b, uint64_t off) { return (float *)at(b, off); }

enum class norm_variant { plain, hp, b1 };

int rmsnorm_entry(norm_variant variant, axiom_runtime *rt, const axiom_device_buffer *w, uint64_t w_off,
                  const axiom_device_buffer *in, uint64_t in_off, axiom_device_buffer *out, uint64_t out_off,
                  uint32_t count, float eps) {
    if (count == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!rt || !w || !in || !out || !owned_by(rt, w) || !owned_by(rt, in) || !owned_by(rt, out) ||
        !f32_span(w, w_off, count) || !f32_span(in, in_off, count) || !f32_span(out, out_off, count)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    const float e = eps > 0.0f ? eps : 1.0e-6f;
    switch (variant) {
    case norm_variant::plain:
        rmsnorm_rows_kernel<sum_kind::f32><<<1, kT>>>(cf(w, w_off), cf(in, in_off), mf(out, out_off), nullptr, nullptr, 0, count, e);
        break;
    case norm_variant::hp:
        rmsnorm_rows_kernel<sum_kind::f64><<<1, kT>>>(cf(w, w_off), cf(in, in_off), mf(out, out_off), nullptr, nullptr, 0, count, e);
        break;
    case norm_variant::b1:
        rmsnorm_b1_kernel<<<1, kT>>>(cf(w, w_off), cf(in, in_off), mf(out, out_off), count, e);
        break;
    }
    note_launch();
    return finish_after_launch(nullptr);
}

}  // namespace
}  // namespace axb

using namespace axb;

extern "C" int axiom_runtime_rmsnorm_f32_device(axiom_runtime *rt, const axiom_device_buffer *w, uint64_t w_off, const axiom_device_buffer *in, uint64_t in_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count, float eps) {
    return rmsnorm_entry(norm_variant::plain, rt, w, w_off, in, in_off, out, out_off, count, eps);
}

extern "C" int axiom_runtime_rmsnorm_f32_hp_device(axiom_runtime *rt, const axiom_device_buffer *w, uint64_t w_off, const axiom_device_buffer *in, uint64_t in_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count, float eps) {
    return rmsnorm_entry(norm_variant::hp, rt, w, w_off, in, in_off, out, out_off, count, eps);
}

extern "C" int axiom_runtime_rmsnorm_f32_b1_device(axiom_runtime *rt, const axiom_device_buffer *w, uint64_t w_off, const axiom_device_buffer *in, uint64_t in_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count, float eps) {
    return rmsnorm_entry(norm_variant::b1, rt, w, w_off, in, in_off, out, out_off, count, eps);
}

extern "C" int axiom_runtime_rmsnorm_f32_dual_device(axiom_runtime *rt, const axiom_device_buffer *w, uint64_t w_off, const axiom_device_buffer *in0, uint64_t in0_off, axiom_device_buffer *out0, uint64_t out0_off, const axiom_device_buffer *in1, uint64_t in1_off, axiom_device_buffer *out1, uint64_t out1_off, uint32_t count, float eps) {
    if (!rt || !w || !in0 || !out0 || !in1 || !out1 || count == 0u) return AXIOM_ERR_INVALID_ARGUMENT;
    if (rt->backend != AXIOM_BACKEND_CUDA || !owned_by(rt, w) || !owned_by(rt, in0) || !owned_by(rt, out0) ||
        !owned_by(rt, in1) || !owned_by(rt, out1)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!f32_span(w, w_off, count) || !f32_span(in0, in0_off, count) || !f32_span(out0, out0_off, count) ||
        !f32_span(in1, in1_off, count) || !f32_span(out1, out1_off, count)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    rmsnorm_rows_kernel<sum_kind::f32><<<2, kT>>>(cf(w, w_off), cf(in0, in0_off), mf(out0, out0_off), cf(in1, in1_off),
                                                  mf(out1, out1_off), 0, count, eps > 0.0f ? eps : 1.0e-6f);
    note_launch();
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_head_rmsnorm_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, uint32_t heads, uint32_t head_dim, float eps) {
    if (!rt || !x || heads == 0u || head_dim == 0u || eps <= 0.0f) return AXIOM_ERR_INVALID_ARGUMENT;
    if (rt->backend != AXIOM_BACKEND_CUDA || !owned_by(rt, x) || !f32_span(x, x_off, (uint64_t)heads * head_dim)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    rmsnorm_rows_kernel<sum_kind::f32><<<heads, kT>>>(nullptr, cf(x, x_off), mf(x, x_off), nullptr, nullptr, head_dim, head_dim, eps);
    note_launch();
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_qk_rmsnorm_w_f32_device(axiom_runtime *rt, axiom_device_buffer *x, uint64_t x_off, const axiom_device_buffer *w, uint64_t w_off, uint32_t heads, uint32_t head_dim, float eps) {
    if (!rt || !x || !w || heads == 0u || head_dim == 0u || eps <= 0.0f) return AXIOM_ERR_INVALID_ARGUMENT;
    if (rt->backend != AXIOM_BACKEND_CUDA || !owned_by(rt, x) || !owned_by(rt, w) ||
        !f32_span(x, x_off, (uint64_t)heads * head_dim) || !f32_span(w, w_off, head_dim)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    rmsnorm_rows_kernel<sum_kind::f64><<<heads, kT>>>(cf(w, w_off), cf(x, x_off), mf(x, x_off), nullptr, nullptr, head_dim, head_dim, eps);
    note_launch();
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_add_f32_device(axiom_runtime *rt, const axiom_device_buffer *a, uint64_t a_off, const axiom_device_buffer *b, uint64_t b_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count) {
    if (!rt || !a || !b || !out || count == 0u || !owned_by(rt, a) || !owned_by(rt, b) || !owned_by(rt, out)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    if (!f32_span(a, a_off, count) || !f32_span(b, b_off, count) || !f32_span(out, out_off, count)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    add_kernel<<<(count + 255u) / 256u, 256>>>(cf(a, a_off), cf(b, b_off), mf(out, out_off), count);
    note_launch();
    return finish_after_launch(nullptr);
}

static int silu_entry(axiom_runtime *rt, const axiom_device_buffer *gate, uint64_t gate_off, const axiom_device_buffer *up, uint64_t up_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count, float clamp_abs) {
    if (!rt || !gate || !up || !out || count == 0u || !owned_by(rt, gate) || !owned_by(rt, up) || !owned_by(rt, out)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    if (!f32_span(gate, gate_off, count) || !f32_span(up, up_off, count) || !f32_span(out, out_off, count)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    silu_mul_kernel<<<(count + 255u) / 256u, 256>>>(cf(gate, gate_off), cf(up, up_off), mf(out, out_off), count, clamp_abs);
    note_launch();
    return finish_after_launch(nullptr);
}

extern "C" int axiom_runtime_silu_mul_f32_device(axiom_runtime *rt, const axiom_device_buffer *gate, uint64_t gate_off, const axiom_device_buffer *up, uint64_t up_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count) {
    return silu_entry(rt, gate, gate_off, up, up_off, out, out_off, count, 0.0f);
}

extern "C" int axiom_runtime_silu_mul_clamp_f32_device(axiom_runtime *rt, const axiom_device_buffer *gate, uint64_t gate_off, const axiom_device_buffer *up, uint64_t up_off, axiom_device_buffer *out, uint64_t out_off, uint32_t count, float clamp_abs) {
    return silu_entry(rt, gate, gate_off, up, up_off, out, out_off, count, clamp_abs);
}

extern "C" int axiom_runtime_kv_pool_store_paged_f32_device(axiom_runtime *rt, const axiom_device_buffer *k_stage, uint64_t k_stage_off, const axiom_device_buffer *v_stage, uint64_t v_stage_off, axiom_device_buffer *k_pool, uint64_t k_pool_off, axiom_device_buffer *v_pool, uint64_t v_pool_off, const axiom_device_buffer *tables, uint64_t tbl_off, const axiom_device_buffer *pos, uint64_t pos_off, uint32_t active, uint32_t tbl_stride, uint32_t n_layers, uint32_t layer, uint32_t block_tokens, uint32_t pool_stride, uint32_t kv_dim) {
    if (!rt || !k_stage || !v_stage || !k_pool || !v_pool || !tables || !pos || active == 0u || tbl_stride == 0u ||
        n_layers == 0u || layer >= n_layers || block_tokens == 0u || kv_dim == 0u || pool_stride < kv_dim) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    if (!owned_by(rt, k_stage) || !owned_by(rt, v_stage) || !owned_by(rt, k_pool) || !owned_by(rt, v_pool) ||
        !owned_by(rt, tables) || !owned_by(rt, pos)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (active > 65535u) return AXIOM_ERR_INVALID_ARGUMENT;  // grid.y bound (src/axiom_cuda.cu:16982-16987)
    if (!f32_span(k_stage, k_stage_off, (uint64_t)active * kv_dim) || !f32_span(v_stage, v_stage_off, (uint64_t)active * kv_dim) ||
        !span_ok(tables, tbl_off, (uint64_t)active * tbl_stride * sizeof(int32_t)) ||
        !span_ok(pos, pos_off, (uint64_t)active * sizeof(uint32_t)) || !span_ok(k_pool, k_pool_off, 0) ||
        !span_ok(v_pool, v_pool_off, 0)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    kv_store_paged_kernel<<<dim3((kv_dim + 255u) / 256u, active), 256>>>(
            cf(k_stage, k_stage_off), cf(v_stage, v_stage_off), mf(k_pool, k_pool_off), mf(v_pool, v_pool_off),
            (const int32_t *)at(tables, tbl_off), (const uint32_t *)at(pos, pos_off), tbl_stride, n_layers, layer,
            block_tokens, pool_stride, kv_dim);
    note_launch();
    return finish_after_launch(nullptr);
}

// ------------------------------------------------------------------------
// Generic single-token embedding gathers (src/axiom_cuda.cu:2213-2256, 14458-14469; runtime
// wrappers src/axiom_runtime.cpp:4656-4752).  Q8_0 rows are blocks of 34 bytes: a little-endian
// F16 scale followed by 32 signed bytes; value = scale * q.  F16 rows are widened and replicated
// into `streams` copies.  One 16-byte-free scalar path is enough: a row is a few KB.
// ------------------------------------------------------------------------
namespace axb {
namespace {

__device__ __forceinline__ float q8_0_value(const uint8_t *row, uint32_t idx) {
    const uint8_t *blk = row + (uint64_t)(idx >> 5) * 34u;
    const uint16_t bits = (uint16_t)blk[0] | ((uint16_t)blk[1] << 8);
    const float d = __half2float(__ushort_as_half(bits));
    return d * (float)((const int8_t *)(blk + 2u))[idx & 31u];
}

__global__ void q8_0_embedding_gather_kernel(const uint8_t *__restrict__ embedding, const uint32_t *__restrict__ token_ptr,
                                             uint32_t token_value, float *__restrict__ out, uint32_t token_count,
                                             uint32_t hidden) {
    const uint32_t tok = token_ptr ? token_ptr[0] : token_value;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= hidden) return;
    if (tok >= token_count) {
        out[i] = 0.0f;
        return;
    }
    out[i] = q8_0_value(embedding + (uint64_t)tok * (hidden / 32u) * 34u, i);
}

__global__ void f16_embedding_streams_kernel(const uint16_t *__restrict__ embedding, float *__restrict__ out, uint32_t token_id,
                                             uint32_t hidden, uint32_t streams) {
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)hidden * streams) return;
    out[idx] = __half2float(__ushort_as_half(embedding[(uint64_t)token_id * hidden + (uint32_t)(idx % hidden)]));
}

int q8_0_gather_entry(axiom_runtime *rt, const axiom_device_buffer *emb, uint64_t emb_off, const axiom_device_buffer *tok,
                      uint64_t tok_off, uint32_t token_value, axiom_device_buffer *out, uint64_t out_off, uint32_t token_count,
                      uint32_t hidden) {
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    const uint64_t emb_bytes = (uint64_t)(hidden / 32u) * 34u * token_count;
    if (!span_ok(emb, emb_off, emb_bytes) || !f32_span(out, out_off, hidden) || (tok && !span_ok(tok, tok_off, sizeof(uint32_t)))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    q8_0_embedding_gather_kernel<<<(hidden + 255u) / 256u, 256>>>(at(emb, emb_off), tok ? (const uint32_t *)at(tok, tok_off) : nullptr,
                                                                 token_value, mf(out, out_off), token_count, hidden);
    note_launch();
    return finish_after_launch(nullptr);
}

}  // namespace
}  // namespace axb

extern "C" int axiom_runtime_q8_0_embedding_gather_f32_device(axiom_runtime *rt, const axiom_device_buffer *embedding_q8, uint64_t embedding_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t token_id, uint32_t token_count, uint32_t hidden) {
    if (!rt || !embedding_q8 || !out || token_count == 0u || hidden == 0u || (hidden % 32u) != 0u || token_id >= token_count ||
        !owned_by(rt, embedding_q8) || !owned_by(rt, out)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    return q8_0_gather_entry(rt, embedding_q8, embedding_offset, nullptr, 0u, token_id, out, out_offset, token_count, hidden);
}

extern "C" int axiom_runtime_q8_0_embedding_gather_token_f32_device(axiom_runtime *rt, const axiom_device_buffer *embedding_q8, uint64_t embedding_offset, const axiom_device_buffer *token_id, uint64_t token_id_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t token_count, uint32_t hidden) {
    if (!rt || !embedding_q8 || !token_id || !out || token_count == 0u || hidden == 0u || (hidden % 32u) != 0u ||
        !owned_by(rt, embedding_q8) || !owned_by(rt, token_id) || !owned_by(rt, out) || (token_id_offset & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    return q8_0_gather_entry(rt, embedding_q8, embedding_offset, token_id, token_id_offset, 0u, out, out_offset, token_count, hidden);
}

extern "C" int axiom_runtime_f16_embedding_streams_device(axiom_runtime *rt, const axiom_device_buffer *embedding_f16, uint64_t embedding_offset, axiom_device_buffer *out_streams, uint64_t out_offset, uint32_t token_id, uint32_t hidden, uint32_t streams) {
    if (!rt || !embedding_f16 || !out_streams || hidden == 0u || streams == 0u || !owned_by(rt, embedding_f16) ||
        !owned_by(rt, out_streams) || (embedding_offset & 1u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (rt->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    uint64_t row_end = 0, out_count = 0;
    if (!mul_ok((uint64_t)token_id + 1u, (uint64_t)hidden * sizeof(uint16_t), &row_end) || !mul_ok(hidden, streams, &out_count) ||
        out_count > 0xffffffffull || !span_ok(embedding_f16, embedding_offset, row_end) ||
        !f32_span(out_streams, out_offset, (uint32_t)out_count)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = begin(rt);
    if (rc != AXIOM_OK) return rc;
    f16_embedding_streams_kernel<<<(uint32_t)((out_count + 255u) / 256u), 256>>>((const uint16_t *)at(embedding_f16, embedding_offset),
                                                                                mf(out_streams, out_offset), token_id, hidden, streams);
    note_launch();
    return finish_after_launch(nullptr);
}

// Greedy next-token selection: per row of logits the largest finite value, the smallest id
// among equal values, and a flag that is raised when any logit of the row is not finite.
//
// Result rule of qwen38_top1_select / qwen38_top1_8_kernel (src/axiom_qwen38_model.cu:408-455,
// 483-493): value > best, or value == best and id < best id; non-finite logits never win and
// set `invalid`.  The rule is an order-independent reduction, so any partition of the row
// gives the reference's result.  The reference's hierarchical path (stage 1 into a global
// `partials` array, stage 2 over it, :510-600) becomes one launch: a thread-block cluster of
// eight CTAs owns a row, every CTA reduces its eighth of the vocabulary with 16-byte loads, and
// the eight partial results meet in the first CTA's shared memory over the cluster's
// distributed shared memory — no global scratch, no second kernel.  With more rows there are enough CTAs with
// smaller clusters, and from 256 rows on without splitting a row at all: the launcher picks 8, 4, 2 or 1 CTAs per row.
#include "runtime.hpp"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace cg = cooperative_groups;

namespace axb {
namespace {

constexpr uint32_t kTop1Threads = 512u;

struct top1_candidate {
    float value;
    uint32_t id;
    uint32_t invalid;
};

__device__ __forceinline__ void top1_take(float value, uint32_t id, top1_candidate *best) {
    if (value > best->value || (value == best->value && id < best->id)) {
        best->value = value;
        best->id = id;
    }
}

__device__ __forceinline__ void top1_see(float value, uint32_t id, top1_candidate *best) {
    if ((__float_as_uint(value) & 0x7f800000u) == 0x7f800000u) best->invalid = 1u;  // infinity or NaN
    else top1_take(value, id, best);
}

__device__ __forceinline__ void top1_warp(top1_candidate *best) {
#pragma unroll
    for (uint32_t off = 16u; off != 0u; off >>= 1u) {
        const float v = __shfl_xor_sync(0xffffffffu, best->value, off);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, best->id, off);
        best->invalid |= __shfl_xor_sync(0xffffffffu, best->invalid, off);
        top1_take(v, i, best);
    }
}

// kParts: CTAs per row — a cluster of that many, or 1 (no cluster).
template <uint32_t kParts, uint32_t kBatch>
__device__ __forceinline__ void top1_rows_body(const float *__restrict__ logits, uint32_t vocab,
                                               axiom_top1_result *__restrict__ results) {
    __shared__ top1_candidate warp_best[kTop1Threads / 32u];
    __shared__ top1_candidate cluster_best[kParts];
    uint32_t part = 0u;
    if (kParts > 1u) part = cg::this_cluster().block_rank();
    const uint32_t row = blockIdx.x / kParts;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    allow_dependents();
    dependency_wait();
    // First half of a cluster barrier: by the time a CTA has scanned its slice and passes the matching wait
    // below, every CTA of the cluster has started, which the store into rank 0's shared memory requires
    // (distributed shared memory may only be accessed once the owning CTA is running).
    if (kParts > 1u) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // this CTA's slice of the row, in units of four logits when the row allows 16-byte loads
    const float *row_logits = logits + (uint64_t)row * vocab;
    top1_candidate best{-CUDART_INF_F, 0xffffffffu, 0u};
    const bool vector = (vocab % 4u) == 0u && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0u;
    if (vector) {
        const uint32_t quads = vocab / 4u;
        const uint32_t per = (quads + kParts - 1u) / kParts;
        const uint32_t lo = part * per, hi = lo + per < quads ? lo + per : quads;
        const float4 *src = reinterpret_cast<const float4 *>(row_logits);
        for (uint32_t q0 = lo + tid; q0 < hi; q0 += kBatch * kTop1Threads) {
            float4 v[kBatch];
#pragma unroll
            for (uint32_t b = 0; b < kBatch; ++b) {
                const uint32_t q = q0 + b * kTop1Threads;
                v[b] = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
                if (q < hi) {
                    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                                 : "=f"(v[b].x), "=f"(v[b].y), "=f"(v[b].z), "=f"(v[b].w) : "l"(src + q));
                }
            }
#pragma unroll
            for (uint32_t b = 0; b < kBatch; ++b) {
                const uint32_t q = q0 + b * kTop1Threads;
                if (q < hi) {
                    top1_see(v[b].x, 4u * q, &best);
                    top1_see(v[b].y, 4u * q + 1u, &best);
                    top1_see(v[b].z, 4u * q + 2u, &best);
                    top1_see(v[b].w, 4u * q + 3u, &best);
                }
            }
        }
    } else {
        const uint32_t per = (vocab + kParts - 1u) / kParts;
        const uint32_t lo = part * per, hi = lo + per < vocab ? lo + per : vocab;
        for (uint32_t i = lo + tid; i < hi; i += kTop1Threads) top1_see(row_logits[i], i, &best);
    }
    top1_warp(&best);
    if (lane == 0u) warp_best[warp] = best;
    __syncthreads();
    if (kParts > 1u) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // free once the slice is scanned: all CTAs arrived long ago
    if (warp == 0u) {
        best = lane < kTop1Threads / 32u ? warp_best[lane] : top1_candidate{-CUDART_INF_F, 0xffffffffu, 0u};
        top1_warp(&best);
        if (kParts > 1u && lane == 0u) {
            // deposit this CTA's result in the first CTA's shared memory
            top1_candidate *dst = cg::this_cluster().map_shared_rank(cluster_best, 0);
            dst[part] = best;
        }
    }
    if (kParts > 1u) cg::this_cluster().sync();
    if (part == 0u && warp == 0u) {
        if (kParts > 1u) {
            best = lane < kParts ? cluster_best[lane] : top1_candidate{-CUDART_INF_F, 0xffffffffu, 0u};
            top1_warp(&best);
        }
        if (lane == 0u) {
            results[row].value = best.value;
            results[row].token_id = best.id;
            results[row].invalid = best.invalid;
        }
    }
}

// kBatch = 16-byte loads in flight per thread
template <uint32_t kParts, uint32_t kBatch>
__global__ void __cluster_dims__(kParts, 1, 1) __launch_bounds__(kTop1Threads)
top1_rows_kernel(const float *__restrict__ logits, uint32_t vocab, axiom_top1_result *__restrict__ results) {
    top1_rows_body<kParts, kBatch>(logits, vocab, results);
}

template <uint32_t kBatch>
__global__ void __launch_bounds__(kTop1Threads)
top1_whole_rows_kernel(const float *__restrict__ logits, uint32_t vocab, axiom_top1_result *__restrict__ results) {
    top1_rows_body<1u, kBatch>(logits, vocab, results);
}

template <uint32_t kParts, uint32_t kBatch>
void launch_top1(const float *logits, uint32_t rows, uint32_t vocab, axiom_top1_result *results, cudaStream_t stream) {
    if constexpr (kParts == 1u) launch_chained(top1_whole_rows_kernel<kBatch>, dim3(rows), dim3(kTop1Threads), 0, stream, logits, vocab, results);
    else launch_chained(top1_rows_kernel<kParts, kBatch>, dim3(rows * kParts), dim3(kTop1Threads), 0, stream, logits, vocab, results);
}

}  // namespace
}  // namespace axb

using namespace axb;

extern "C" int axiom_qwen38_fused_top1_f32_device(int device, const float *logits, uint32_t rows, uint32_t vocab,
                                                  axiom_top1_result *results, void *stream) {
    if (!logits || !results || rows == 0u || vocab == 0u || rows > 65535u || (reinterpret_cast<uintptr_t>(logits) & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // CTAs per row: about 256 CTAs in all (a little under two per SM), at most a cluster of eight per row and at
    // least one CTA per row.  Measured at vocab 151 936 (us, best of parts 8/4/2/1): 8 rows 5.8 (8), 32 rows 7.1 (8),
    // 64 rows 12.5 (4; 15.2 with 8), 128 rows 19.3 (2; 23.9 with 8), 256 rows 32.1 (1; 42.9 with 8), 1024 rows 97.6
    // (1; 154.9 with 8).  Eight loads in flight per thread while all CTAs are resident at once, four beyond that.
    uint32_t parts = 8u;
    while (parts > 1u && rows * parts > 256u) parts >>= 1;
    const bool deep = rows * parts <= 2u * kSmCount;
    if (parts == 8u) launch_top1<8, 8>(logits, rows, vocab, results, st);
    else if (parts == 4u) launch_top1<4, 8>(logits, rows, vocab, results, st);
    else if (parts == 2u) launch_top1<2, 8>(logits, rows, vocab, results, st);
    else if (deep) launch_top1<1, 8>(logits, rows, vocab, results, st);
    else launch_top1<1, 4>(logits, rows, vocab, results, st);
    note_launch();
    return launch_status();
}

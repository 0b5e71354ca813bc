// Residual add + RMSNorm (+ NVFP4 quantize) in one pass over HBM.
//
// Arithmetic of qwen38_add_bf16_rmsnorm8_kernel / qwen38_rmsnorm_bf16_8_kernel
// (src/axiom_qwen38_model.cu:190-292) followed by the activation quantizer
// (src/axiom_qwen38_nvfp4_mlp.cu:144-223), including the reference's FP32
// summation order: 256 partial sums over features (c + 256*k) accumulated with
// fmaf in k order, then the tree 128/64/32/16/8/4/2/1.
//
// Streaming kernel (add_rmsnorm_stream_kernel, two rows per SM and more): persistent CTAs, one
// per SM, made of up to eight independent 4-warp teams.  A team owns one shared-memory slot (more
// when rows are narrow); its first thread fills the slot with one row (addend | residual) through
// 1-D bulk copies that complete on the slot's mbarrier and no arithmetic warp issues a global
// load.  The kernel is bound by instruction issue, so resident warps matter more than prefetch
// depth: while a team waits for its next row the others compute, and the addend half of the next
// row is requested as soon as sweep 1 has consumed the current one.  Sweep 1 (merge + sum of
// squares) gives thread t the feature pairs 256k + 2t, 2t+1: those are partial sums 2t and 2t+1
// of the reference order, so the fmaf chains run along k in registers; the 256 partials meet in
// shared memory and every warp runs the reference tree as a shuffle butterfly.  The merged row is
// written back into the slot (it is BF16-valued by construction), leaves for HBM as one bulk
// store, and sweep 2 (normalise + quantize) re-reads it in 16-byte chunks, lane pairs forming the
// 16-value NVFP4 blocks.
//
// Wide-row kernel (add_rmsnorm_wide_row_kernel, decode shapes and the gathered-addend flavour): one
// CTA per row, one thread per 16-byte chunk, one global round trip per row.
#include "pipeline.cuh"
#include "runtime.hpp"

namespace axb {

namespace {

__device__ __forceinline__ void unpack8(const uint4 &v, float (&x)[8]) {
    const float2 a = bf16x2_widen_fma(v.x), b = bf16x2_widen_fma(v.y), c = bf16x2_widen_fma(v.z), d = bf16x2_widen_fma(v.w);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}

struct norm_args {
    const uint4 *hidden;    // may be null
    uint4 *residual;        // read; rewritten when hidden != null
    const uint16_t *gamma;
    uint4 *norm_out;        // may be null
    uint32_t *codes;        // may be null
    uint8_t *scales;
    float eps;
    float G;
    uint32_t rows;
    uint32_t cols;
    uint32_t chunks_per_row;
    uint32_t layout;
    uint32_t groups;
    uint32_t inner_tiles;
    uint32_t ring_slots;    // stream kernel: shared-memory slots per warp
    // wide-row kernel only: the addend of row r is row token_ids[r] of an embedding table
    const uint4 *table;     // may be null
    const uint32_t *token_ids;
    uint32_t vocab;
    uint32_t *status_word;  // may be null
    uint4 *tap;             // may be null: second copy of the updated residual rows (layer tap)
    // scaled-F32 addend (kScaledF32): raw FP8-GEMM accumulators with their per-feature and per-token scales
    const float *hidden_f32;        // [rows x cols]
    const uint16_t *weight_scale;   // [cols] BF16
    const float *input_scale;       // [rows]
    // test hook (axiom_b200_test_arm_wait_timeout): the first row of team 0 of CTA 0 announces this many bytes more
    // than its copies deliver, so its barrier never completes, and waits give up after spin_limit polls (0 = default)
    uint32_t inject_tx;
    uint32_t spin_limit;
};

// What is added to the residual before the norm.
//   kBf16:      a BF16 tensor (or, in the wide-row kernel, rows gathered from a BF16 table)
//   kScaledF32: bf16((raw * weight_scale[feature]) * input_scale[token]) of raw F32 accumulators — the FP8 GEMM's
//               scale epilogue (fp8_group_row_scale_bf16_epilogue_kernel, src/axiom_qwen38_fp8.cu:250-262) evaluated
//               in this kernel's prologue instead of in a pass of its own
enum addend_kind : int { kNone = 0, kBf16 = 1, kScaledF32 = 2 };

// Second sweep over one row held in shared memory as BF16: n = bf16((r * inv) * gamma), optional
// BF16 copy out, NVFP4 quantize.  Thread t takes the 16-byte chunks t + 128k; lane pairs form
// the 16-value blocks.  kExact recomputes every chunk with IEEE divisions and the reference's
// NaN-dropping maximum (taken only when the straight-line pass flagged a block).  kFull: the
// row is a whole number of 128-chunk steps, so no bounds predicate is needed.
template <bool kExact, bool kFull>
__device__ __forceinline__ void norm_quant_sweep(const norm_args &a, const uint4 *row_sh, const float *gamma_sh,
                                                 const scale_lut_entry *lut, float2 inv2, uint64_t base,
                                                 uint32_t iters, uint32_t t, uint8_t *scale_ptr,
                                                 uint32_t scale_step, bool *needs_exact) {
    const uint4 *src = row_sh + t;
    const float4 *gamma_a = reinterpret_cast<const float4 *>(gamma_sh) + t;
    const float4 *gamma_b = reinterpret_cast<const float4 *>(gamma_sh + (a.cols >> 1)) + t;
    uint4 *norm_dst = a.norm_out ? a.norm_out + base + t : nullptr;
    uint32_t *code_dst = a.codes ? a.codes + base + t : nullptr;
#pragma unroll 5
    for (uint32_t k = 0; k < iters; ++k) {
        const bool ok = kFull || t + 128u * k < a.chunks_per_row;
        uint4 m = make_uint4(0u, 0u, 0u, 0u);
        float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), gb = ga;
        if (ok) {
            m = src[128u * k];
            ga = gamma_a[128u * k];
            gb = gamma_b[128u * k];
        }
        const float2 y0 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m.x), inv2), make_float2(ga.x, ga.y));
        const float2 y1 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m.y), inv2), make_float2(ga.z, ga.w));
        const float2 y2 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m.z), inv2), make_float2(gb.x, gb.y));
        const float2 y3 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m.w), inv2), make_float2(gb.z, gb.w));
        const uint4 nrm = make_uint4(pack_bf16x2(y0.x, y0.y), pack_bf16x2(y1.x, y1.y), pack_bf16x2(y2.x, y2.y), pack_bf16x2(y3.x, y3.y));
        if (!kExact && norm_dst && ok) st_stream(norm_dst + 128u * k, nrm);
        if (code_dst) {
            float y[8];
            unpack8(nrm, y);  // the quantizer sees the BF16-rounded values
            uint32_t scale_byte, packed;
            if (kExact) {
                float mx = absmax8_drop_nan(y);
                mx = fmaxf(fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1)), 0.0f);
                packed = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], mx, a.G, &scale_byte);
            } else {
                float mx = absmax8_nan(y);
                mx = max_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                packed = nvfp4_quantize8_fast(y, mx, a.G, lut, &scale_byte, needs_exact);
            }
            if (ok) {
                st_stream(code_dst + 128u * k, packed);
                if ((t & 1u) == 0u) scale_ptr[(uint64_t)k * scale_step] = (uint8_t)scale_byte;
            }
        }
    }
}

// A row of zeros: the addend of a token whose id lies outside the embedding table (device arrays start zeroed).
static __device__ __align__(16) uint8_t g_zero_row[16384u * 2u];

constexpr uint32_t kTeamThreads = 128u;
constexpr uint32_t kMaxTeams = 8u;
constexpr uint32_t kMaxSlotsPerTeam = 4u;

__device__ __forceinline__ void team_barrier(uint32_t team) {
    asm volatile("bar.sync %0, %1;" ::"r"(team + 1u), "r"(kTeamThreads) : "memory");
}
// The same barrier carrying a vote: true in every thread of the team when any of them passed true.
__device__ __forceinline__ bool team_barrier_any(uint32_t team, bool flag) {
    uint32_t any;
    asm volatile("{\n\t.reg .pred in, out;\n\tsetp.ne.u32 in, %3, 0;\n\tbar.red.or.pred out, %1, %2, in;\n\tselp.u32 %0, 1, 0, out;\n\t}"
                 : "=r"(any) : "r"(team + 1u), "r"(kTeamThreads), "r"((uint32_t)flag) : "memory");
    return any != 0u;
}

// Shared memory: [teams x slots x slot_bytes][gamma F32, two planes][scale table][partials teams x 256][barriers]
// kCols != 0: the row width is a template constant and the CTA has kMaxTeams teams with one slot each (what the
// launcher picks at that width): both sweeps unroll completely, every offset inside a row is an immediate and the
// slot bookkeeping disappears.
template <int kAddend, bool kFull, uint32_t kCols = 0u>
__global__ void __launch_bounds__(kMaxTeams * kTeamThreads, 1)
add_rmsnorm_stream_kernel(const norm_args given) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool kAdd = kAddend != kNone;
    norm_args a = given;
    if (kCols) {
        a.cols = kCols;
        a.chunks_per_row = kCols / 8u;
        a.groups = kCols / kGroup;
        a.inner_tiles = (kCols / kGroup + 3u) / 4u;
        a.ring_slots = 1u;
    }
    const uint32_t teams = kCols ? kMaxTeams : blockDim.x / kTeamThreads;
    const uint32_t spt = a.ring_slots;  // slots per team
    const uint32_t row_bytes = a.cols * 2u;
    const uint32_t addend_bytes = kAddend == kScaledF32 ? 2u * row_bytes : kAddend == kBf16 ? row_bytes : 0u;
    const uint32_t slot_bytes = addend_bytes + row_bytes;
    float *gamma_sh = reinterpret_cast<float *>(smem + (size_t)teams * spt * slot_bytes);
    float *wscale_sh = gamma_sh + a.cols;  // [cols] F32, kScaledF32 only
    scale_lut_entry *lut = reinterpret_cast<scale_lut_entry *>(wscale_sh + (kAddend == kScaledF32 ? a.cols : 0u));
    float *partials = reinterpret_cast<float *>(lut + 128);                      // [teams][256]
    uint64_t *bars = reinterpret_cast<uint64_t *>(partials + teams * 256u);      // [teams][kMaxSlotsPerTeam]

    const uint32_t tid = threadIdx.x, team = tid / kTeamThreads, t = tid % kTeamThreads, lane = tid & 31u;
    const uint32_t warp_in_team = t >> 5;
    uint64_t *my_bars = bars + team * kMaxSlotsPerTeam;
    uint8_t *my_slots = smem + (size_t)team * spt * slot_bytes;
    float *my_partials = partials + team * 256u;
    allow_dependents();
    if (t == 0u) {
        for (uint32_t j = 0; j < spt; ++j) mbar_init(my_bars + j, 1u);
        mbar_init_fence();
    }
    team_barrier(team);
    dependency_wait();
    const uint32_t spin_limit = a.spin_limit ? a.spin_limit : kSpinLimit;

    // rows of this CTA: blockIdx.x + n * gridDim.x; this team takes n = team + teams * i
    const uint32_t cta_rows = blockIdx.x < a.rows ? (a.rows - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;
    const uint32_t my_rows = team < cta_rows ? (cta_rows - team + teams - 1u) / teams : 0u;
    const float count = (float)a.cols;
    const bool stores = kAdd || a.tap != nullptr;  // rows leave shared memory through bulk stores
    const uint32_t k_iters = (a.cols + 255u) / 256u;                      // sweep 1: feature pairs 256k + 2t
    const uint32_t c_iters = (a.chunks_per_row + kTeamThreads - 1u) / kTeamThreads;  // sweep 2: chunks t + 128k

    // A row arrives in two bulk copies that complete on the slot's mbarrier.  The addend half of a
    // slot is dead as soon as sweep 1 has merged it into the residual half, so the NEXT row's
    // addend is requested right then (announced with expect_tx only) and only its residual has
    // to wait until sweep 2 and the bulk store of the merged row are done with the other half.
    // `token` is the row's id when the addend is gathered from an embedding table (ids at or beyond the vocabulary
    // read the row of zeros and raise the status word)
    auto issue_addend = [&](uint32_t i, uint32_t j, uint32_t token) {  // thread 0 of the team; j = i % spt
        const uint64_t row = blockIdx.x + (uint64_t)(team + teams * i) * gridDim.x;
        mbar_expect_tx(my_bars + j, addend_bytes);
        const void *src;
        if (kAddend == kScaledF32) {
            src = a.hidden_f32 + row * a.cols;
        } else if (a.table) {
            if (token < a.vocab) {
                src = a.table + (uint64_t)token * a.chunks_per_row;
            } else {
                src = g_zero_row;
                if (a.status_word) atomicCAS(a.status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
            }
        } else {
            src = a.hidden + row * a.chunks_per_row;
        }
        bulk_load(my_slots + (size_t)j * slot_bytes, src, addend_bytes, my_bars + j);
    };
    auto token_of_row = [&](uint32_t i) -> uint32_t {
        return (kAddend == kBf16 && a.table) ? a.token_ids[blockIdx.x + (team + teams * i) * gridDim.x] : 0u;
    };
    auto issue_residual = [&](uint32_t i, uint32_t j) {
        const uint64_t row = blockIdx.x + (uint64_t)(team + teams * i) * gridDim.x;
        mbar_arrive_expect_tx(my_bars + j, row_bytes + ((blockIdx.x | team | i) == 0u ? a.inject_tx : 0u));
        bulk_load(my_slots + (size_t)j * slot_bytes + addend_bytes, a.residual + row * a.chunks_per_row, row_bytes,
                  my_bars + j);
    };
    auto issue = [&](uint32_t i, uint32_t j) {
        if (kAdd) issue_addend(i, j, token_of_row(i));
        issue_residual(i, j);
    };
    // the first rows are already on their way while the CTA prepares gamma and the scale table
    if (t == 0u) {
        for (uint32_t i = 0; i < spt && i < my_rows; ++i) issue(i, i);
    }
    // gamma as F32 in two planes: plane h holds values 8q+4h .. 8q+4h+3 of every chunk q, so a warp's
    // 16-byte reads are contiguous
    for (uint32_t f = tid; f < a.cols; f += blockDim.x) {
        gamma_sh[((f >> 2) & 1u) * (a.cols >> 1) + (f >> 3) * 4u + (f & 3u)] = __uint_as_float((uint32_t)a.gamma[f] << 16);
    }
    if (kAddend == kScaledF32) {
        for (uint32_t f = tid; f < a.cols; f += blockDim.x) wscale_sh[f] = __uint_as_float((uint32_t)a.weight_scale[f] << 16);
    }
    const bool lut_safe = build_scale_lut(lut, a.codes ? a.G : 1.0f);  // contains the CTA barrier

    uint32_t j = 0u, phase = 0u;  // slot of row i and the parity of its barrier: i % spt, (i / spt) & 1
    for (uint32_t i = 0; i < my_rows; ++i) {
        float token_scale = 1.0f;
        if (kAddend == kScaledF32) token_scale = a.input_scale[blockIdx.x + (team + teams * i) * gridDim.x];
        // the id of the row whose addend is requested after sweep 1 (fetched now: its latency hides behind the sweep)
        uint32_t next_token = 0u;
        if (t == 0u && i + spt < my_rows) {
            next_token = token_of_row(i + spt);
            // the residual half of the slot is refilled only at the end of this row: hint that row into L2 now, so
            // the refill is an L2 hit by the time it is issued (49.7 -> 48.7 us at 8192 x 5120). Hinting the addend
            // as well, or two rows ahead, measured slower (49.8 and 60.9 us): the hints then compete with the loads
            // in flight.
            bulk_prefetch_l2(a.residual + (blockIdx.x + (uint64_t)(team + teams * (i + spt)) * gridDim.x) * a.chunks_per_row,
                             row_bytes);
        }
        // A wait that ran out raises the device's fault word.  The barrier that follows sweep 1 (which only touches
        // shared memory) carries the threads' verdicts as a vote, so the team decides as one: it writes nothing for
        // this row or any later one, waits — bounded again — for the copies it still has in flight, and leaves.
        // Its rows keep their old contents; the caller learns of it from axiom_b200_pipeline_faults().
        const bool gave_up = !mbar_wait(my_bars + j, phase, spin_limit);
        const uint32_t row = blockIdx.x + (team + teams * i) * gridDim.x;
        const uint64_t base = (uint64_t)row * a.chunks_per_row;
        uint8_t *slot = my_slots + (size_t)j * slot_bytes;
        const uint32_t *hid_sh = reinterpret_cast<const uint32_t *>(slot) + t;
        uint32_t *res_sh = reinterpret_cast<uint32_t *>(slot + addend_bytes);
        const float2 *raw_sh = reinterpret_cast<const float2 *>(slot) + t;        // kScaledF32: feature pairs as F32
        const float2 *ws_sh = reinterpret_cast<const float2 *>(wscale_sh) + t;
        const float2 ts2 = make_float2(token_scale, token_scale);

        // sweep 1: merge in place; this thread's two fmaf chains (partials 2t and 2t+1)
        float2 p = make_float2(0.f, 0.f);
        {
            uint32_t *res_w = res_sh + t;
#pragma unroll 5
            for (uint32_t k = 0; k < k_iters; ++k) {
                if (kFull || 256u * k + 2u * t < a.cols) {
                    uint32_t m = res_w[128u * k];
                    if (kAddend == kBf16) {
                        m = add_bf16x2(m, hid_sh[128u * k]);  // bf16(bf16(res) + bf16(add))
                        res_w[128u * k] = m;
                    } else if (kAddend == kScaledF32) {
                        // addend = bf16((raw * weight_scale) * token_scale), the reference's epilogue expression
                        const float2 h = __fmul2_rn(__fmul2_rn(raw_sh[128u * k], ws_sh[128u * k]), ts2);
                        m = add_bf16x2(m, pack_bf16x2(h.x, h.y));
                        res_w[128u * k] = m;
                    }
                    p = bf16x2_square_accumulate(m, p);
                }
            }
        }
        reinterpret_cast<float2 *>(my_partials)[t] = p;
        if (stores) fence_async_shared();
        if (team_barrier_any(team, gave_up)) {
            // rows i+1 .. i+spt-1 were requested in full; nothing later was (the addend of row i+spt is requested below)
            for (uint32_t n = i + 1u; n < i + spt && n < my_rows; ++n) (void)mbar_wait(my_bars + n % spt, (n / spt) & 1u, spin_limit);
            break;
        }
        if (stores && t == 0u) {
            // the merged row leaves as one bulk store (two with a tap); the slot stays in use until it has been read
            if (kAdd) bulk_store(a.residual + base, res_sh, row_bytes);
            if (a.tap) bulk_store(a.tap + base, res_sh, row_bytes);
            bulk_commit();
            if (kAdd && i + spt < my_rows) issue_addend(i + spt, j, next_token);  // every thread is past its reads of the addend half
        }
        // Reference tree over the 256 partials c: strides 128,64,32 then 16,8,4,2,1.  With lane l
        // holding c = 8l + e, strides 128..8 are the lane butterfly 16,8,4,2,1 applied to each e
        // separately; warp w of the team does e = 2w and 2w+1, then the four results meet in
        // shared memory for strides 4,2,1 (e+4, e+2, e+1).
        float s0 = my_partials[8u * lane + 2u * warp_in_team], s1 = my_partials[8u * lane + 2u * warp_in_team + 1u];
#pragma unroll
        for (uint32_t off = 16u; off != 0u; off >>= 1u) {
            s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, off));
            s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, off));
        }
        team_barrier(team);  // everyone has read the partials
        if (lane == 0u) {
            my_partials[2u * warp_in_team] = s0;
            my_partials[2u * warp_in_team + 1u] = s1;
        }
        team_barrier(team);
        const float4 lo = reinterpret_cast<const float4 *>(my_partials)[0], hi = reinterpret_cast<const float4 *>(my_partials)[1];
        const float t0 = __fadd_rn(lo.x, hi.x), t1 = __fadd_rn(lo.y, hi.y), t2 = __fadd_rn(lo.z, hi.z), t3 = __fadd_rn(lo.w, hi.w);
        const float total = __fadd_rn(__fadd_rn(t0, t2), __fadd_rn(t1, t3));
        const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(total, count), a.eps));
        const float2 inv2 = make_float2(inverse, inverse);

        // sweep 2: normalise, round, quantize.  Chunk t + 128k is block (t>>1) + 64k.
        const uint32_t g0 = t >> 1;
        uint8_t *scale_ptr;
        uint32_t scale_step;
        if (a.layout == AXIOM_SCALE_LAYOUT_CANONICAL) {
            scale_ptr = a.scales + (uint64_t)row * a.groups + g0;
            scale_step = 64u;
        } else {
            scale_ptr = a.scales + ((uint64_t)(row >> 7) * a.inner_tiles + (g0 >> 2)) * 512u + (row & 31u) * 16u +
                        ((row & 127u) >> 5) * 4u + (g0 & 3u);
            scale_step = 16u * 512u;
        }
        bool needs_exact = false;
        const uint4 *row_sh = reinterpret_cast<const uint4 *>(res_sh);
        norm_quant_sweep<false, kFull>(a, row_sh, gamma_sh, lut, inv2, base, c_iters, t, scale_ptr, scale_step, &needs_exact);
        if (a.codes && (!lut_safe || __any_sync(0xffffffffu, needs_exact))) {
            norm_quant_sweep<true, kFull>(a, row_sh, gamma_sh, lut, inv2, base, c_iters, t, scale_ptr, scale_step, &needs_exact);
        }
        // the whole team is done with the slot: refill it with the row that comes spt rows later
        team_barrier(team);
        if (t == 0u) {
            if (stores) bulk_wait_read_all();
            if (i + spt < my_rows) issue_residual(i + spt, j);
        }
        if (++j == spt) {
            j = 0u;
            phase ^= 1u;
        }
    }
    if (stores && t == 0u) bulk_wait_read_all();
}

// ---------------------------------------------------------------------------
// Few rows (decode shapes): one CTA per row with one thread per 16-byte chunk, so a row costs
// one global round trip: every thread loads its chunk of hidden, residual and gamma at once,
// merges, stores the residual chunk and parks the merged chunk in shared memory; 128 threads
// then run the reference's 256 fmaf chains from shared memory (20 dependent FMAs each at 5120
// columns), one warp runs the reference tree, and every thread normalises and quantizes the
// chunk it still holds in registers.
// ---------------------------------------------------------------------------
constexpr uint32_t kWideMaxChunksPerThread = 2u;  // 16384 columns = 2048 chunks over 1024 threads

template <int kAddend>
__global__ void __launch_bounds__(1024, 1)
add_rmsnorm_wide_row_kernel(const norm_args a) {
    constexpr bool kAdd = kAddend != kNone;
    extern __shared__ __align__(128) uint8_t smem[];
    uint4 *merged_sh = reinterpret_cast<uint4 *>(smem);  // [chunks_per_row]
    __shared__ scale_lut_entry lut[128];
    __shared__ __align__(16) float partials[256];
    __shared__ float total_sh;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint4 *gamma16 = reinterpret_cast<const uint4 *>(a.gamma);
    allow_dependents();
    // the divisor table depends on a scalar argument only: it is built while the previous kernel on the stream drains
    const bool lut_safe = build_scale_lut(lut, a.codes ? a.G : 1.0f);
    dependency_wait();

    for (uint32_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
        const uint64_t base = (uint64_t)row * a.chunks_per_row;
        uint32_t token_id = 0u;
        float token_scale = 1.0f;
        if (kAddend == kScaledF32) token_scale = a.input_scale[row];
        if (kAddend == kBf16 && a.table) {
            token_id = a.token_ids[row];
            if (token_id >= a.vocab && tid == 0u && a.status_word) {
                atomicCAS(a.status_word, AXIOM_STATUS_WORD_OK, AXIOM_STATUS_WORD_BAD_ADDRESS);
            }
        }
        uint4 m[kWideMaxChunksPerThread], gam[kWideMaxChunksPerThread];
#pragma unroll
        for (uint32_t c = 0; c < kWideMaxChunksPerThread; ++c) {
            const uint32_t q = tid + c * blockDim.x;
            m[c] = make_uint4(0u, 0u, 0u, 0u);
            gam[c] = m[c];
            if (q < a.chunks_per_row) {
                m[c] = ld_stream(a.residual + base + q);
                uint4 h = make_uint4(0u, 0u, 0u, 0u);
                if (kAddend == kBf16) {
                    if (a.table) {  // gathered addend: id >= vocab gives a zero row and raises the status word
                        if (token_id < a.vocab) h = ld_stream(a.table + (uint64_t)token_id * a.chunks_per_row + q);
                    } else {
                        h = ld_stream(a.hidden + base + q);
                    }
                } else if (kAddend == kScaledF32) {
                    // addend = bf16((raw * weight_scale) * token_scale), the reference's epilogue expression
                    const float4 *raw = reinterpret_cast<const float4 *>(a.hidden_f32 + (uint64_t)row * a.cols) + 2u * q;
                    const float4 r0 = raw[0], r1 = raw[1];
                    const uint4 w = reinterpret_cast<const uint4 *>(a.weight_scale)[q];
                    const float2 ts2 = make_float2(token_scale, token_scale);
                    const float2 h0 = __fmul2_rn(__fmul2_rn(make_float2(r0.x, r0.y), bf16x2_widen_fma(w.x)), ts2);
                    const float2 h1 = __fmul2_rn(__fmul2_rn(make_float2(r0.z, r0.w), bf16x2_widen_fma(w.y)), ts2);
                    const float2 h2 = __fmul2_rn(__fmul2_rn(make_float2(r1.x, r1.y), bf16x2_widen_fma(w.z)), ts2);
                    const float2 h3 = __fmul2_rn(__fmul2_rn(make_float2(r1.z, r1.w), bf16x2_widen_fma(w.w)), ts2);
                    h = make_uint4(pack_bf16x2(h0.x, h0.y), pack_bf16x2(h1.x, h1.y), pack_bf16x2(h2.x, h2.y), pack_bf16x2(h3.x, h3.y));
                }
                gam[c] = gamma16[q];
                if (kAdd) {
                    m[c].x = add_bf16x2(m[c].x, h.x); m[c].y = add_bf16x2(m[c].y, h.y);
                    m[c].z = add_bf16x2(m[c].z, h.z); m[c].w = add_bf16x2(m[c].w, h.w);
                    st_stream(a.residual + base + q, m[c]);
                }
                if (a.tap) st_stream(a.tap + base + q, m[c]);
                merged_sh[q] = m[c];
            }
        }
        __syncthreads();  // merged_sh is complete

        // partial sums 2t, 2t+1: features 256k + 2t, 2t+1 in k order (the reference's chains)
        if (tid < 128u) {
            const uint32_t *words = reinterpret_cast<const uint32_t *>(merged_sh) + tid;
            float2 p = make_float2(0.f, 0.f);
            const uint32_t k_iters = (a.cols + 255u) / 256u;
            for (uint32_t k = 0; k < k_iters; ++k) {
                if (256u * k + 2u * tid < a.cols) {
                    const uint32_t w = words[128u * k];
                    p = bf16x2_square_accumulate(w, p);
                }
            }
            reinterpret_cast<float2 *>(partials)[tid] = p;
        }
        __syncthreads();
        if (tid < 32u) {
            // strides 128, 64, 32 through shared memory, then 16..1 as a butterfly (same additions)
            float v = __fadd_rn(__fadd_rn(__fadd_rn(partials[lane], partials[lane + 128u]),
                                          __fadd_rn(partials[lane + 64u], partials[lane + 192u])),
                                __fadd_rn(__fadd_rn(partials[lane + 32u], partials[lane + 160u]),
                                          __fadd_rn(partials[lane + 96u], partials[lane + 224u])));
#pragma unroll
            for (uint32_t off = 16u; off != 0u; off >>= 1u) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
            if (lane == 0u) total_sh = v;
        }
        __syncthreads();
        const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(total_sh, (float)a.cols), a.eps));
        const float2 inv2 = make_float2(inverse, inverse);

#pragma unroll
        for (uint32_t c = 0; c < kWideMaxChunksPerThread; ++c) {
            const uint32_t q = tid + c * blockDim.x;
            if (c * blockDim.x >= a.chunks_per_row) break;  // uniform: no thread has a chunk in this round
            const bool ok = q < a.chunks_per_row;
            const float2 y0 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m[c].x), inv2),
                                         bf16x2_widen_fma(gam[c].x));
            const float2 y1 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m[c].y), inv2),
                                         bf16x2_widen_fma(gam[c].y));
            const float2 y2 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m[c].z), inv2),
                                         bf16x2_widen_fma(gam[c].z));
            const float2 y3 = __fmul2_rn(__fmul2_rn(bf16x2_widen_fma(m[c].w), inv2),
                                         bf16x2_widen_fma(gam[c].w));
            const uint4 nrm = make_uint4(pack_bf16x2(y0.x, y0.y), pack_bf16x2(y1.x, y1.y), pack_bf16x2(y2.x, y2.y),
                                         pack_bf16x2(y3.x, y3.y));
            if (a.norm_out && ok) st_stream(a.norm_out + base + q, nrm);
            if (a.codes) {
                float y[8];
                unpack8(nrm, y);  // the quantizer sees the BF16-rounded values
                float mx = absmax8_nan(y);
                mx = max_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                uint32_t scale_byte;
                bool needs_exact = false;
                uint32_t packed = nvfp4_quantize8_fast(y, mx, a.G, lut, &scale_byte, &needs_exact);
                if (!lut_safe || __any_sync(0xffffffffu, needs_exact)) {
                    mx = absmax8_drop_nan(y);
                    mx = fmaxf(fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1)), 0.0f);
                    packed = nvfp4_quantize8_exact(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7], mx, a.G, &scale_byte);
                }
                if (ok) {
                    st_stream(a.codes + base + q, packed);
                    if ((q & 1u) == 0u) {
                        a.scales[scale_offset(row, q >> 1, a.groups, a.inner_tiles, a.layout)] = (uint8_t)scale_byte;
                    }
                }
            }
        }
        __syncthreads();  // merged_sh, partials and total_sh are rewritten for the next row
    }
}

constexpr size_t kSmemBudget = 227u * 1024u;
// Below this many rows the one-CTA-per-row kernel is used (measured crossover with the streaming kernel).
#ifndef AXB_WIDE_ROW_BELOW_ROWS
#define AXB_WIDE_ROW_BELOW_ROWS (2u * 148u)
#endif
constexpr uint32_t kWideRowBelowRows = AXB_WIDE_ROW_BELOW_ROWS;

size_t stream_fixed_bytes(uint32_t cols, uint32_t teams, int addend = kBf16) {
    return (size_t)cols * sizeof(float) * (addend == kScaledF32 ? 2u : 1u) + 128u * sizeof(scale_lut_entry) +
           (size_t)teams * 256u * sizeof(float) + (size_t)teams * kMaxSlotsPerTeam * sizeof(uint64_t);
}

constexpr uint32_t kModelHidden = 5120u;  // the reference model's hidden size: the BF16-addend kernel is also built for it

template <int kAdd, bool kFull, uint32_t kCols = 0u>
void launch_stream_impl(const norm_args &a, uint32_t teams, size_t smem, cudaStream_t stream) {
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kAdd, kFull, kCols>>(kSmemBudget);
    const uint32_t ctas = a.rows < kSmCount ? a.rows : kSmCount;
    launch_chained(add_rmsnorm_stream_kernel<kAdd, kFull, kCols>, dim3(ctas), dim3(teams * kTeamThreads), smem, stream, a);
}

template <int kAdd>
void launch_stream(const norm_args &a, uint32_t teams, size_t smem, cudaStream_t stream) {
    // 48.7 -> 48.3 us at 8192 x 5120
    if (kAdd == kBf16 && a.cols == kModelHidden && teams == kMaxTeams && a.ring_slots == 1u) {
        launch_stream_impl<kBf16, true, kModelHidden>(a, teams, smem, stream);
        return;
    }
    if (a.cols % 1024u == 0u) launch_stream_impl<kAdd, true>(a, teams, smem, stream);
    else launch_stream_impl<kAdd, false>(a, teams, smem, stream);
}

// One-shot test hook state (axiom_b200_test_arm_wait_timeout): consumed by the next streaming launch.
uint32_t g_armed_inject_tx = 0u, g_armed_spin_limit = 0u;

// Picks the kernel and its shape for a prepared argument block.
int launch_norm(norm_args &a, int addend, cudaStream_t stream) {
    const uint32_t rows = a.rows, cols = a.cols;
    // Stream kernel shape.  The kernel is bound by instruction issue, not by memory, so resident
    // warps count for more than prefetch depth: eight teams with one slot each (while a team
    // waits for its next row the other seven compute) beat five double-buffered teams at 5120
    // columns (53.5 us against 56.0 us for 8192 rows).  Narrow rows get both: up to eight
    // teams and as many slots per team as fit.
    const size_t slot_bytes = (size_t)cols * 2u * (addend == kScaledF32 ? 3u : addend == kBf16 ? 2u : 1u);
    auto teams_that_fit = [&](uint32_t slots) {
        uint32_t t = kMaxTeams;
        while (t != 0u && stream_fixed_bytes(cols, t, addend) + (size_t)t * slots * slot_bytes > kSmemBudget) --t;
        return t;
    };
    const uint32_t single = teams_that_fit(1u), dual = teams_that_fit(2u);
    uint32_t teams = single >= dual + 2u ? single : dual;
    uint32_t spt = 0u;
    if (teams != 0u) {
        spt = (uint32_t)((kSmemBudget - stream_fixed_bytes(cols, teams, addend)) / (teams * slot_bytes));
        if (spt > kMaxSlotsPerTeam) spt = kMaxSlotsPerTeam;
    }
    // Few rows (latency matters more than streaming), or rows too wide for one slot: one wide CTA per row.
    if (rows < kWideRowBelowRows || teams == 0u || spt == 0u) {
        uint32_t threads = (a.chunks_per_row + 31u) & ~31u;
        if (threads > 1024u) threads = 1024u;
        if (threads < 128u) threads = 128u;  // the 256 partial sums are produced by the first 128 threads
        const size_t row_smem = (size_t)a.chunks_per_row * sizeof(uint4);
        const uint32_t ctas = rows < kSmCount * 8u ? rows : kSmCount * 8u;
        if (addend == kScaledF32) launch_chained(add_rmsnorm_wide_row_kernel<kScaledF32>, dim3(ctas), dim3(threads), row_smem, stream, a);
        else if (addend == kBf16) launch_chained(add_rmsnorm_wide_row_kernel<kBf16>, dim3(ctas), dim3(threads), row_smem, stream, a);
        else launch_chained(add_rmsnorm_wide_row_kernel<kNone>, dim3(ctas), dim3(threads), row_smem, stream, a);
        note_launch();
        return AXIOM_OK;
    }
    a.ring_slots = spt;
    a.inject_tx = g_armed_inject_tx;
    a.spin_limit = g_armed_spin_limit;
    g_armed_inject_tx = g_armed_spin_limit = 0u;
    const size_t smem = stream_fixed_bytes(cols, teams, addend) + (size_t)teams * spt * slot_bytes;
    if (addend == kScaledF32) launch_stream<kScaledF32>(a, teams, smem, stream);
    else if (addend == kBf16) launch_stream<kBf16>(a, teams, smem, stream);
    else launch_stream<kNone>(a, teams, smem, stream);
    note_launch();
    return AXIOM_OK;
}

}  // namespace

unsigned int add_rmsnorm_fault_word() { return read_and_clear_pipeline_fault(); }

// Everything a first launch would set up lazily, for axiom_b200_prepare().
void prepare_add_rmsnorm_unit() {
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kNone, true>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kNone, false>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kBf16, true>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kBf16, false>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kBf16, true, kModelHidden>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kScaledF32, true>>(kSmemBudget);
    allow_dynamic_smem<add_rmsnorm_stream_kernel<kScaledF32, false>>(kSmemBudget);
}

int launch_gather_add_rmsnorm_nvfp4_bf16(const void *table, uint32_t vocab, const uint32_t *token_ids, void *residual,
                                         const void *gamma, float eps, uint32_t rows, uint32_t cols, float G,
                                         void *norm_out, uint8_t *codes, uint8_t *scales, uint32_t layout,
                                         uint32_t *status_word, cudaStream_t stream) {
    norm_args a{};
    a.table = (const uint4 *)table;
    a.token_ids = token_ids;
    a.vocab = vocab;
    a.status_word = status_word;
    a.residual = (uint4 *)residual;
    a.gamma = (const uint16_t *)gamma;
    a.norm_out = (uint4 *)norm_out;
    a.codes = (uint32_t *)codes;
    a.scales = scales;
    a.eps = eps;
    a.G = G;
    a.rows = rows;
    a.cols = cols;
    a.chunks_per_row = cols / 8u;
    a.layout = layout;
    a.groups = cols / kGroup;
    a.inner_tiles = (a.groups + 3u) / 4u;
    return launch_norm(a, kBf16, stream);
}

int launch_add_rmsnorm_nvfp4_bf16(const void *hidden, void *residual, const void *gamma, float eps, uint32_t rows,
                                  uint32_t cols, float G, void *norm_out, uint8_t *codes, uint8_t *scales,
                                  uint32_t layout, cudaStream_t stream) {
    return launch_add_rmsnorm_tap_nvfp4_bf16(hidden, residual, gamma, eps, rows, cols, G, norm_out, codes, scales, layout,
                                             nullptr, stream);
}

int launch_add_rmsnorm_tap_nvfp4_bf16(const void *hidden, void *residual, const void *gamma, float eps, uint32_t rows,
                                      uint32_t cols, float G, void *norm_out, uint8_t *codes, uint8_t *scales,
                                      uint32_t layout, void *tap, cudaStream_t stream) {
    norm_args a{};
    a.tap = (uint4 *)tap;
    a.hidden = (const uint4 *)hidden;
    a.residual = (uint4 *)residual;
    a.gamma = (const uint16_t *)gamma;
    a.norm_out = (uint4 *)norm_out;
    a.codes = (uint32_t *)codes;
    a.scales = scales;
    a.eps = eps;
    a.G = G;
    a.rows = rows;
    a.cols = cols;
    a.chunks_per_row = cols / 8u;
    a.layout = layout;
    a.groups = cols / kGroup;
    a.inner_tiles = (a.groups + 3u) / 4u;

    return launch_norm(a, hidden ? kBf16 : kNone, stream);
}

int launch_fp8_epilogue_add_rmsnorm_nvfp4(const float *gemm_out, const void *weight_scale, const float *input_scale,
                                          void *residual, const void *gamma, float eps, uint32_t rows, uint32_t cols,
                                          float G, void *norm_out, uint8_t *codes, uint8_t *scales, uint32_t layout,
                                          cudaStream_t stream) {
    norm_args a{};
    a.hidden_f32 = gemm_out;
    a.weight_scale = (const uint16_t *)weight_scale;
    a.input_scale = input_scale;
    a.residual = (uint4 *)residual;
    a.gamma = (const uint16_t *)gamma;
    a.norm_out = (uint4 *)norm_out;
    a.codes = (uint32_t *)codes;
    a.scales = scales;
    a.eps = eps;
    a.G = G;
    a.rows = rows;
    a.cols = cols;
    a.chunks_per_row = cols / 8u;
    a.layout = layout;
    a.groups = cols / kGroup;
    a.inner_tiles = (a.groups + 3u) / 4u;
    return launch_norm(a, kScaledF32, stream);
}

}  // namespace axb

using namespace axb;

extern "C" int axiom_b200_test_arm_wait_timeout(uint32_t extra_bytes, uint32_t spin_limit) {
    if ((extra_bytes % 16u) != 0u || extra_bytes > (1u << 19) || spin_limit > (1u << 20)) return AXIOM_ERR_INVALID_ARGUMENT;
    g_armed_inject_tx = extra_bytes;
    g_armed_spin_limit = spin_limit;
    return AXIOM_OK;
}

extern "C" int axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device(
        int device, const void *hidden_bf16, void *residual_bf16, const void *gamma_bf16, float eps,
        uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes,
        uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!residual_bf16 || !gamma_bf16 || rows == 0u || cols == 0u || (cols % kGroup) != 0u || cols > 16384u ||
        scale_layout > AXIOM_SCALE_LAYOUT_TILED || !(eps > 0.0f) || !std::isfinite(eps)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !norm_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!aligned16(residual_bf16) || !aligned16(gamma_bf16) || (hidden_bf16 && !aligned16(hidden_bf16)) ||
        (norm_out_bf16 && !aligned16(norm_out_bf16)) || (reinterpret_cast<uintptr_t>(out_codes) & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_rmsnorm_nvfp4_bf16(hidden_bf16, residual_bf16, gamma_bf16, eps, rows, cols, global_scale,
                                  norm_out_bf16, out_codes, out_scales, scale_layout, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_gather_add_rmsnorm_nvfp4_bf16_device(
        int device, const void *table_bf16, uint32_t vocab, const uint32_t *token_ids, void *residual_bf16,
        const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16,
        uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, uint32_t *status_word, void *stream) {
    if (!table_bf16 || !token_ids || vocab == 0u || !residual_bf16 || !gamma_bf16 || rows == 0u || cols == 0u ||
        (cols % kGroup) != 0u || cols > 16384u || scale_layout > AXIOM_SCALE_LAYOUT_TILED || !(eps > 0.0f) ||
        !std::isfinite(eps)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !norm_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!aligned16(table_bf16) || !aligned16(residual_bf16) || !aligned16(gamma_bf16) || (norm_out_bf16 && !aligned16(norm_out_bf16)) ||
        (out_codes && (reinterpret_cast<uintptr_t>(out_codes) & 3u))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_gather_add_rmsnorm_nvfp4_bf16(table_bf16, vocab, token_ids, residual_bf16, gamma_bf16, eps, rows, cols,
                                         out_codes ? global_scale : 1.0f, norm_out_bf16, out_codes, out_scales, scale_layout,
                                         status_word, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_add_rmsnorm_nvfp4_tap_bf16_device(
        int device, const void *hidden_bf16, void *residual_bf16, const void *gamma_bf16, float eps, uint32_t rows,
        uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes, uint8_t *out_scales,
        uint32_t scale_layout, void *tap_out_bf16, void *stream) {
    if (!tap_out_bf16 || !aligned16(tap_out_bf16) || tap_out_bf16 == residual_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!residual_bf16 || !gamma_bf16 || rows == 0u || cols == 0u || (cols % kGroup) != 0u || cols > 16384u ||
        scale_layout > AXIOM_SCALE_LAYOUT_TILED || !(eps > 0.0f) || !std::isfinite(eps)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !norm_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if ((hidden_bf16 && !aligned16(hidden_bf16)) || !aligned16(residual_bf16) || !aligned16(gamma_bf16) ||
        (norm_out_bf16 && !aligned16(norm_out_bf16)) || (out_codes && (reinterpret_cast<uintptr_t>(out_codes) & 3u))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_rmsnorm_tap_nvfp4_bf16(hidden_bf16, residual_bf16, gamma_bf16, eps, rows, cols, out_codes ? global_scale : 1.0f,
                                      norm_out_bf16, out_codes, out_scales, scale_layout, tap_out_bf16, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_fp8_epilogue_add_rmsnorm_nvfp4_device(
        int device, const float *gemm_out_f32, const void *weight_scale_bf16, const float *input_scale, void *residual_bf16,
        const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16,
        uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream) {
    if (!gemm_out_f32 || !weight_scale_bf16 || !input_scale || !residual_bf16 || !gamma_bf16 || rows == 0u || cols == 0u ||
        (cols % kGroup) != 0u || cols > 16384u || scale_layout > AXIOM_SCALE_LAYOUT_TILED || !(eps > 0.0f) ||
        !std::isfinite(eps)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if ((out_codes == nullptr) != (out_scales == nullptr)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!out_codes && !norm_out_bf16) return AXIOM_ERR_INVALID_ARGUMENT;
    if (out_codes && !valid_scale(global_scale)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (!aligned16(gemm_out_f32) || !aligned16(weight_scale_bf16) || (reinterpret_cast<uintptr_t>(input_scale) & 3u) ||
        !aligned16(residual_bf16) || !aligned16(gamma_bf16) || (norm_out_bf16 && !aligned16(norm_out_bf16)) ||
        (out_codes && (reinterpret_cast<uintptr_t>(out_codes) & 3u))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_fp8_epilogue_add_rmsnorm_nvfp4(gemm_out_f32, weight_scale_bf16, input_scale, residual_bf16, gamma_bf16, eps, rows, cols,
                                          out_codes ? global_scale : 1.0f, norm_out_bf16, out_codes, out_scales, scale_layout,
                                          (cudaStream_t)stream);
    return launch_status();
}

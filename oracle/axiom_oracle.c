/*
 * CPU oracle — plain C restatement of the reference kernels' arithmetic.
 * TEST INFRASTRUCTURE ONLY (see axiom_oracle.h).  Build with
 *   gcc -O2 -std=c11 -fopenmp -ffp-contract=off -fPIC -shared
 * (-ffp-contract=off matters: every fused multiply-add below is an explicit
 * fmaf(), every other product/sum is separately rounded, as on the device).
 *
 * Citations are relative to the reference project root.
 */
#include "axiom_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define AXO_OK 0
#define AXO_INVALID 1

static int g_threads = 0;

void axo_set_threads(int threads) { g_threads = threads > 0 ? threads : 0; }

int axo_get_threads(void) {
#ifdef _OPENMP
    return g_threads > 0 ? g_threads : omp_get_max_threads();
#else
    return 1;
#endif
}

#ifdef _OPENMP
#define AXO_PARALLEL_FOR _Pragma("omp parallel for schedule(static) num_threads(axo_get_threads())")
#else
#define AXO_PARALLEL_FOR
#endif

/* ------------------------------------------------------------------ */
/* scalar primitives                                                   */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* IEEE round-to-nearest-even F32 -> BF16; the finite path is the integer
 * trick of host_round_bf16 (src/axiom_qwen38_model.cu:393-401) and
 * float_host_to_bf16 (src/axiom_qwen38_mtp_compute.cu:132-137).  NaN is kept a
 * quiet NaN as __float2bfloat16_rn does (0x7fff). */
uint16_t axo_f32_to_bf16(float value) {
    uint32_t bits = f32_bits(value);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

float axo_bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

float axo_bf16_round(float value) { return axo_bf16_to_f32(axo_f32_to_bf16(value)); }

/* E4M3FN decode: src/axiom_qwen38_nvfp4.cu:36-46 (same table in
 * src/axiom_qwen38_fp8.cu:41-51). */
float axo_e4m3_decode(uint8_t code) {
    if ((code & 0x7fu) == 0x7fu) return NAN;
    const uint32_t exponent = (code >> 3) & 0x0fu;
    const uint32_t mantissa = code & 0x07u;
    const float magnitude = exponent == 0u
            ? ldexpf((float)mantissa, -9)
            : ldexpf(1.0f + (float)mantissa * 0.125f, (int)exponent - 7);
    return (code & 0x80u) ? -magnitude : magnitude;
}

/* __nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3) as called at
 * src/axiom_qwen38_fp8.cu:90-91 and src/axiom_qwen38_nvfp4.cu:49-50:
 * round-to-nearest-even onto the E4M3FN grid, everything at or beyond the
 * largest finite value (infinities included) saturates to +-448, NaN -> 0x7f. */
uint8_t axo_e4m3_encode_satfinite(float value) {
    if (isnan(value)) return 0x7fu;
    const uint8_t sign = signbit(value) ? 0x80u : 0u;
    const float a = fabsf(value);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7eu);
    if (a < 0.015625f) {
        /* subnormal grid, spacing 2^-9; 8 rolls over into the first normal code */
        const int q = (int)rintf(a * 512.0f);
        return (uint8_t)(sign | (uint8_t)q);
    }
    int e = ilogbf(a);
    int q = (int)rintf((a / ldexpf(1.0f, e) - 1.0f) * 8.0f);
    if (q == 8) { q = 0; ++e; }
    uint32_t code = ((uint32_t)(e + 7) << 3) | (uint32_t)q;
    if (code > 0x7eu) code = 0x7eu;
    return (uint8_t)(sign | code);
}

/* encode_e4m3fn_scale (src/axiom_qwen38_nvfp4.cu:48-55,
 * src/axiom_qwen38_nvfp4_mlp.cu:133-140): zero magnitude becomes +0.125
 * (0x20), the NaN code is replaced by the largest finite code. */
uint8_t axo_e4m3_encode_scale(float value) {
    const uint8_t code = axo_e4m3_encode_satfinite(value);
    const uint8_t magnitude = code & 0x7fu;
    if (magnitude == 0u) return 0x20u;
    if (magnitude == 0x7fu) return (uint8_t)((code & 0x80u) | 0x7eu);
    return code;
}

/* __nv_cvt_float_to_fp4(value, __NV_E2M1, cudaRoundNearest) as called at
 * src/axiom_qwen38_nvfp4.cu:82-85: RN-even on {0,.5,1,1.5,2,3,4,6} (ties go to
 * the code with an even mantissa bit), saturating, NaN -> +6. */
uint8_t axo_e2m1_encode(float value) {
    if (isnan(value)) return 7u;
    const uint8_t sign = signbit(value) ? 8u : 0u;
    const float a = fabsf(value);
    uint8_t code;
    if (a <= 0.25f) code = 0u;
    else if (a < 0.75f) code = 1u;
    else if (a <= 1.25f) code = 2u;
    else if (a < 1.75f) code = 3u;
    else if (a <= 2.5f) code = 4u;
    else if (a < 3.5f) code = 5u;
    else if (a <= 5.0f) code = 6u;
    else code = 7u;
    return (uint8_t)(sign | code);
}

float axo_e2m1_decode(uint8_t nibble) {
    static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    const float v = grid[nibble & 7u];
    return (nibble & 8u) ? -v : v;
}

/* ------------------------------------------------------------------ */
/* NVFP4 activation quantizer                                          */
/* ------------------------------------------------------------------ */

/* One 16-value group: qwen38_quantize_reference_kernel
 * (src/axiom_qwen38_nvfp4.cu:57-88).  Order of operations kept:
 * (max * (1/6)) * G, then decode(scale)/G as a true division, then x / d. */
static void nvfp4_group(const float *x, float global_scale, uint8_t *packed, uint8_t *scale) {
    float max_abs = 0.0f;
    for (int i = 0; i < 16; ++i) max_abs = fmaxf(max_abs, fabsf(x[i]));
    const float sixth = 1.0f / 6.0f;
    const uint8_t code = axo_e4m3_encode_scale((max_abs * sixth) * global_scale);
    const float local = axo_e4m3_decode(code) / global_scale;
    *scale = code;
    for (int pair = 0; pair < 8; ++pair) {
        const uint8_t lo = axo_e2m1_encode(x[2 * pair] / local) & 0x0fu;
        const uint8_t hi = axo_e2m1_encode(x[2 * pair + 1] / local) & 0x0fu;
        packed[pair] = (uint8_t)(lo | (hi << 4));
    }
}

static int valid_scale(float v) { return isfinite(v) && v > 0.0f; }

/* Argument contract of axiom_qwen38_nvfp4_quantize_reference_f32
 * (src/axiom_qwen38_nvfp4.cu:132-143), extended to many rows. */
int axo_nvfp4_quantize_f32(const float *input, uint32_t rows, uint32_t cols,
                           float global_scale, uint8_t *codes, uint8_t *scales) {
    if (!input || !codes || !scales || rows == 0u || cols == 0u || (cols % 16u) != 0u ||
        !valid_scale(global_scale)) {
        return AXO_INVALID;
    }
    const uint32_t groups = cols / 16u;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const float *row = input + (size_t)r * cols;
        for (uint32_t g = 0; g < groups; ++g) {
            nvfp4_group(row + 16u * g, global_scale, codes + (size_t)r * (cols / 2u) + 8u * g,
                        scales + (size_t)r * groups + g);
        }
    }
    return AXO_OK;
}

int axo_nvfp4_quantize_bf16(const uint16_t *input, uint32_t rows, uint32_t cols,
                            float global_scale, uint8_t *codes, uint8_t *scales) {
    if (!input || !codes || !scales || rows == 0u || cols == 0u || (cols % 16u) != 0u ||
        !valid_scale(global_scale)) {
        return AXO_INVALID;
    }
    const uint32_t groups = cols / 16u;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const uint16_t *row = input + (size_t)r * cols;
        float x[16];
        for (uint32_t g = 0; g < groups; ++g) {
            for (int i = 0; i < 16; ++i) x[i] = axo_bf16_to_f32(row[16u * g + i]);
            nvfp4_group(x, global_scale, codes + (size_t)r * (cols / 2u) + 8u * g,
                        scales + (size_t)r * groups + g);
        }
    }
    return AXO_OK;
}

/* scale_view_bytes / scale_view_offset (src/axiom_qwen38_nvfp4_mlp.cu:95-108):
 * 128 x 4 scale tiles of 512 bytes, the layout cuBLASLt names VEC16_UE4M3. */
uint64_t axo_scale_tiled_bytes(uint32_t outer, uint32_t inner) {
    const uint64_t outer_tiles = ((uint64_t)outer + 127u) / 128u;
    const uint64_t inner_tiles = ((uint64_t)inner + 3u) / 4u;
    return outer_tiles * inner_tiles * 512u;
}

uint64_t axo_scale_tiled_offset(uint32_t outer, uint32_t inner, uint32_t inner_tiles) {
    const uint32_t in_tile = outer % 128u;
    const uint64_t base = ((uint64_t)(outer / 128u) * inner_tiles + inner / 4u) * 512u;
    return base + (in_tile % 32u) * 16u + (in_tile / 32u) * 4u + inner % 4u;
}

/* pack_weight_scales (src/axiom_qwen38_nvfp4_mlp.cu:110-120): padding bytes are zero. */
int axo_scales_canonical_to_tiled(const uint8_t *canonical, uint32_t rows, uint32_t groups,
                                  uint8_t *tiled) {
    if (!canonical || !tiled || rows == 0u || groups == 0u) return AXO_INVALID;
    const uint32_t inner_tiles = (groups + 3u) / 4u;
    memset(tiled, 0, (size_t)axo_scale_tiled_bytes(rows, groups));
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t g = 0; g < groups; ++g) {
            tiled[axo_scale_tiled_offset(r, g, inner_tiles)] = canonical[(size_t)r * groups + g];
        }
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* FP8 E4M3 per-token quantizer                                        */
/* ------------------------------------------------------------------ */

/* quantize_columns_e4m3_kernel (src/axiom_qwen38_fp8.cu:64-94): a "column" is
 * one token's contiguous feature row.  fmaxf is order independent, so the
 * reduction tree does not matter. */
static void fp8_row(const float *x, uint32_t cols, uint8_t *codes, float *scale_out) {
    float m = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) m = fmaxf(m, fabsf(x[c]));
    float scale = m == 0.0f ? 1.0f : m / 448.0f;
    if (!isfinite(scale) || scale <= 0.0f) scale = 1.0f;
    *scale_out = scale;
    for (uint32_t c = 0; c < cols; ++c) codes[c] = axo_e4m3_encode_satfinite(x[c] / scale);
}

int axo_fp8_quantize_f32(const float *input, uint32_t rows, uint32_t cols,
                         uint8_t *codes, float *scales) {
    if (!input || !codes || !scales || rows == 0u || cols == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        fp8_row(input + (size_t)r * cols, cols, codes + (size_t)r * cols, scales + r);
    }
    return AXO_OK;
}

/* Static-scale flavour quantize_columns_static_e4m3_kernel (src/axiom_qwen38_fp8.cu:96-107; the ModelOpt
 * branch of quantize_input, :830-840): code = e4m3_satfinite(x / scale) with a scale given by the caller. */
int axo_fp8_quantize_static_f32(const float *input, uint64_t count, float scale, uint8_t *codes) {
    if (!input || !codes) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t i = 0; i < (int64_t)count; ++i) codes[i] = axo_e4m3_encode_satfinite(input[i] / scale);
    return AXO_OK;
}

/* BF16-input twin quantize_bf16_rows_e4m3_kernel
 * (src/axiom_qwen38_mtp_compute.cu:239-278): non-finite inputs are skipped by
 * the max and raise the status word (4 = runtime error). */
int axo_fp8_quantize_bf16(const uint16_t *input, uint32_t rows, uint32_t cols,
                          uint8_t *codes, float *scales, uint32_t *status) {
    if (!input || !codes || !scales || rows == 0u || cols == 0u) return AXO_INVALID;
    int bad = 0;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const uint16_t *row = input + (size_t)r * cols;
        uint8_t *out = codes + (size_t)r * cols;
        float m = 0.0f;
        for (uint32_t c = 0; c < cols; ++c) {
            const float v = axo_bf16_to_f32(row[c]);
            if (isfinite(v)) m = fmaxf(m, fabsf(v));
            else {
#ifdef _OPENMP
#pragma omp atomic write
#endif
                bad = 1;
            }
        }
        const float scale = m == 0.0f ? 1.0f : m / 448.0f;
        scales[r] = scale;
        for (uint32_t c = 0; c < cols; ++c) {
            out[c] = axo_e4m3_encode_satfinite(axo_bf16_to_f32(row[c]) / scale);
        }
    }
    if (status && bad && *status == 0u) *status = 4u;
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* residual add + RMSNorm                                              */
/* ------------------------------------------------------------------ */

/* qwen38_add_bf16_inplace_kernel (src/axiom_qwen38_model.cu:175-184). */
int axo_add_bf16(const uint16_t *a, const uint16_t *b, uint64_t count, uint16_t *out) {
    if (!a || !b || !out || count == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        out[i] = axo_f32_to_bf16(axo_bf16_to_f32(a[i]) + axo_bf16_to_f32(b[i]));
    }
    return AXO_OK;
}

/* Sum of squares in the reference order (src/axiom_qwen38_model.cu:203-236):
 * 256 strided partial sums (feature = lane + 256*k, fmaf chain in k order), a
 * shared-memory tree 128/64/32 and a shuffle tree 16..1.  Rows whose length is
 * not a multiple of 256 simply have shorter chains in the upper lanes. */
static float sum_squares_tree256(const float *x, uint32_t cols) {
    float partial[256];
    for (uint32_t lane = 0; lane < 256u; ++lane) {
        float s = 0.0f;
        for (uint32_t f = lane; f < cols; f += 256u) s = fmaf(x[f], x[f], s);
        partial[lane] = s;
    }
    for (uint32_t stride = 128u; stride != 0u; stride >>= 1u) {
        for (uint32_t lane = 0; lane < stride; ++lane) partial[lane] = partial[lane] + partial[lane + stride];
    }
    return partial[0];
}

/* rsqrtf() of the device is an approximation (<= 2 ulp); the oracle uses the
 * correctly rounded value and the tests allow the documented tolerance. */
static float rsqrt_f32(float v) { return (float)(1.0 / sqrt((double)v)); }

static void add_rmsnorm_row(const uint16_t *hidden, const uint16_t *residual_in,
                            const uint16_t *gamma, float eps, uint32_t cols,
                            uint16_t *residual_out, float *merged, float *norm) {
    for (uint32_t f = 0; f < cols; ++f) {
        float r = axo_bf16_to_f32(residual_in[f]);
        if (hidden) r = axo_bf16_round(r + axo_bf16_to_f32(hidden[f]));
        merged[f] = r;
        if (residual_out) residual_out[f] = axo_f32_to_bf16(r);
    }
    const float ss = sum_squares_tree256(merged, cols);
    const float inverse = rsqrt_f32(ss / (float)cols + eps);
    for (uint32_t f = 0; f < cols; ++f) {
        norm[f] = axo_bf16_round((merged[f] * inverse) * axo_bf16_to_f32(gamma[f]));
    }
}

/* qwen38_add_bf16_rmsnorm8_kernel / qwen38_rmsnorm_bf16_8_kernel
 * (src/axiom_qwen38_model.cu:190-292) with BF16 storage. */
int axo_add_rmsnorm_bf16(const uint16_t *hidden, const uint16_t *residual_in,
                         const uint16_t *gamma, float eps, uint32_t rows, uint32_t cols,
                         uint16_t *residual_out, uint16_t *norm_out) {
    if (!residual_in || !gamma || !norm_out || rows == 0u || cols == 0u) return AXO_INVALID;
    int failed = 0;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        float *merged = (float *)malloc(sizeof(float) * 2u * cols);
        if (!merged) { failed = 1; continue; }
        float *norm = merged + cols;
        add_rmsnorm_row(hidden ? hidden + (size_t)r * cols : NULL, residual_in + (size_t)r * cols,
                        gamma, eps, cols, residual_out ? residual_out + (size_t)r * cols : NULL,
                        merged, norm);
        for (uint32_t f = 0; f < cols; ++f) norm_out[(size_t)r * cols + f] = axo_f32_to_bf16(norm[f]);
        free(merged);
    }
    return failed ? AXO_INVALID : AXO_OK;
}

/* The fused add + RMSNorm + NVFP4 chain: the reference runs the norm kernel
 * (src/axiom_qwen38_model.cu:1371-1373) and then the activation quantizer on
 * its BF16-valued output (src/axiom_qwen38_nvfp4_mlp.cu:1347-1381). */
int axo_add_rmsnorm_nvfp4_bf16(const uint16_t *hidden, const uint16_t *residual_in,
                               const uint16_t *gamma, float eps, uint32_t rows, uint32_t cols,
                               float global_scale, uint16_t *residual_out, uint16_t *norm_out,
                               uint8_t *codes, uint8_t *scales) {
    if (!residual_in || !gamma || !codes || !scales || rows == 0u || cols == 0u ||
        (cols % 16u) != 0u || !valid_scale(global_scale)) {
        return AXO_INVALID;
    }
    const uint32_t groups = cols / 16u;
    int failed = 0;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        float *merged = (float *)malloc(sizeof(float) * 2u * cols);
        if (!merged) { failed = 1; continue; }
        float *norm = merged + cols;
        add_rmsnorm_row(hidden ? hidden + (size_t)r * cols : NULL, residual_in + (size_t)r * cols,
                        gamma, eps, cols, residual_out ? residual_out + (size_t)r * cols : NULL,
                        merged, norm);
        if (norm_out) {
            for (uint32_t f = 0; f < cols; ++f) norm_out[(size_t)r * cols + f] = axo_f32_to_bf16(norm[f]);
        }
        for (uint32_t g = 0; g < groups; ++g) {
            nvfp4_group(norm + 16u * g, global_scale, codes + (size_t)r * (cols / 2u) + 8u * g,
                        scales + (size_t)r * groups + g);
        }
        free(merged);
    }
    return failed ? AXO_INVALID : AXO_OK;
}

/* ------------------------------------------------------------------ */
/* SwiGLU                                                              */
/* ------------------------------------------------------------------ */

/* silu_mul_batch_kernel (src/axiom_qwen38_fp8_mlp.cu:16-21): FP32, true
 * division, precise expf, product with `up` last, no BF16 rounding. */
float axo_silu_mul(float gate, float up) { return (gate / (1.0f + expf(-gate))) * up; }

int axo_swiglu_f32(const uint16_t *gate_up, uint32_t rows, uint32_t width, float *out) {
    if (!gate_up || !out || rows == 0u || width == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const uint16_t *row = gate_up + (size_t)r * 2u * width;
        for (uint32_t f = 0; f < width; ++f) {
            out[(size_t)r * width + f] = axo_silu_mul(axo_bf16_to_f32(row[f]), axo_bf16_to_f32(row[width + f]));
        }
    }
    return AXO_OK;
}

/* silu_mul_batch_kernel followed by quantize_columns_e4m3_kernel
 * (src/axiom_qwen38_fp8_mlp.cu:111-128, src/axiom_qwen38_fp8.cu:64-94). */
int axo_swiglu_fp8_bf16(const uint16_t *gate_up, uint32_t rows, uint32_t width,
                        uint8_t *codes, float *scales) {
    if (!gate_up || !codes || !scales || rows == 0u || width == 0u) return AXO_INVALID;
    int failed = 0;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        float *y = (float *)malloc(sizeof(float) * width);
        if (!y) { failed = 1; continue; }
        const uint16_t *row = gate_up + (size_t)r * 2u * width;
        for (uint32_t f = 0; f < width; ++f) {
            y[f] = axo_silu_mul(axo_bf16_to_f32(row[f]), axo_bf16_to_f32(row[width + f]));
        }
        fp8_row(y, width, codes + (size_t)r * width, scales + r);
        free(y);
    }
    return failed ? AXO_INVALID : AXO_OK;
}

/* silu_mul_quantize_batch_to_tc_kernel (src/axiom_qwen38_nvfp4_mlp.cu:229-270),
 * canonical scale layout. */
int axo_swiglu_nvfp4_bf16(const uint16_t *gate_up, uint32_t rows, uint32_t width,
                          float global_scale, uint8_t *codes, uint8_t *scales) {
    if (!gate_up || !codes || !scales || rows == 0u || width == 0u || (width % 16u) != 0u ||
        !valid_scale(global_scale)) {
        return AXO_INVALID;
    }
    const uint32_t groups = width / 16u;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const uint16_t *row = gate_up + (size_t)r * 2u * width;
        float y[16];
        for (uint32_t g = 0; g < groups; ++g) {
            for (int i = 0; i < 16; ++i) {
                y[i] = axo_silu_mul(axo_bf16_to_f32(row[16u * g + i]),
                                    axo_bf16_to_f32(row[width + 16u * g + i]));
            }
            nvfp4_group(y, global_scale, codes + (size_t)r * (width / 2u) + 8u * g,
                        scales + (size_t)r * groups + g);
        }
    }
    return AXO_OK;
}

/* Output gate of the attention block followed by the o_proj activation quantizer:
 * y = bf16(attention * (1.0f / (1.0f + expf(-gate)))) (qwen38_sigmoid_gate_kernel, reference
 * src/axiom_qwen38_attention.cu:470-479), then the NVFP4 quantizer on the BF16 values.
 * out_bf16, codes/scales optional (codes and scales together). */
int axo_sigmoid_gate_nvfp4_bf16(const uint16_t *attention, const uint16_t *gate, uint32_t rows,
                                uint32_t width, float global_scale, uint16_t *out_bf16,
                                uint8_t *codes, uint8_t *scales) {
    if (!attention || !gate || rows == 0u || width == 0u || (width % 16u) != 0u ||
        ((codes == NULL) != (scales == NULL)) || (!codes && !out_bf16) ||
        (codes && !valid_scale(global_scale))) {
        return AXO_INVALID;
    }
    const uint32_t groups = width / 16u;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        float y[16];
        for (uint32_t g = 0; g < groups; ++g) {
            for (int i = 0; i < 16; ++i) {
                const size_t at = (size_t)r * width + 16u * g + i;
                const float sig = 1.0f / (1.0f + expf(-axo_bf16_to_f32(gate[at])));
                const uint16_t bits = axo_f32_to_bf16(axo_bf16_to_f32(attention[at]) * sig);
                if (out_bf16) out_bf16[at] = bits;
                y[i] = axo_bf16_to_f32(bits);
            }
            if (codes) {
                nvfp4_group(y, global_scale, codes + (size_t)r * (width / 2u) + 8u * g,
                            scales + (size_t)r * groups + g);
            }
        }
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* YaRN frequencies                                                    */
/* ------------------------------------------------------------------ */

/* 0.1 * ln(factor) + 1 (include/axiom/qwen38_attention.h:29 holds the value
 * for factor 4: 1.138629436111989). */
float axo_yarn_mscale(float factor) {
    if (!(factor > 1.0f)) return 1.0f;
    return (float)(0.1 * log((double)factor) + 1.0);
}

/* qwen38_yarn_inv_frequency (src/axiom_qwen38_attention.cu:98-116): all FP32.
 * The blend is evaluated as fma(inv, 1-ramp, (inv/factor)*ramp). */
int axo_yarn_inv_freq(const axo_rope_params *p, float *inv_freq) {
    if (!p || !inv_freq || p->rope_dim == 0u || (p->rope_dim & 1u) || !(p->theta > 0.0f)) return AXO_INVALID;
    const float dim = (float)p->rope_dim;
    const uint32_t half = p->rope_dim / 2u;
    for (uint32_t pair = 0; pair < half; ++pair) {
        const float exponent = (2.0f * (float)pair) / dim;
        const float inv = 1.0f / powf(p->theta, exponent);
        if (!(p->factor > 1.0f)) { inv_freq[pair] = inv; continue; }
        const float two_pi = 6.283185307179586f;
        const float fast = dim * logf(p->original_context / (p->beta_fast * two_pi)) / (2.0f * logf(p->theta));
        const float slow = dim * logf(p->original_context / (p->beta_slow * two_pi)) / (2.0f * logf(p->theta));
        const float low = floorf(fast < slow ? fast : slow);
        const float high = ceilf(fast > slow ? fast : slow);
        float ramp = high > low ? ((float)pair - low) / (high - low)
                                : ((float)pair >= high ? 1.0f : 0.0f);
        ramp = fminf(1.0f, fmaxf(0.0f, ramp));
        inv_freq[pair] = fmaf(inv, 1.0f - ramp, (inv / p->factor) * ramp);
    }
    return AXO_OK;
}

/* initialize_rope_cache (src/axiom_qwen38_dspark_compute.cu:1470-1498):
 * correction bounds in FP64 and clamped to [0, dim-1]; the blend itself FP32. */
int axo_yarn_inv_freq_host_table(const axo_rope_params *p, float *inv_freq) {
    if (!p || !inv_freq || p->rope_dim == 0u || (p->rope_dim & 1u) || !(p->theta > 0.0f)) return AXO_INVALID;
    const double two_pi = 6.283185307179586476925286766559;
    const double dim = (double)p->rope_dim;
    const uint32_t half = p->rope_dim / 2u;
    const double fast = dim * log((double)p->original_context / ((double)p->beta_fast * two_pi)) /
                        (2.0 * log((double)p->theta));
    const double slow = dim * log((double)p->original_context / ((double)p->beta_slow * two_pi)) /
                        (2.0 * log((double)p->theta));
    const float low = (float)fmax(0.0, floor(fast));
    const float high = (float)fmin(dim - 1.0, ceil(slow));
    for (uint32_t pair = 0; pair < half; ++pair) {
        const float exponent = (float)(2u * pair) / (float)p->rope_dim;
        const float pos_frequency = powf(p->theta, exponent);
        const float extrapolated = 1.0f / pos_frequency;
        if (!(p->factor > 1.0f)) { inv_freq[pair] = extrapolated; continue; }
        const float interpolated = 1.0f / (p->factor * pos_frequency);
        float ramp = high > low ? ((float)pair - low) / (high - low)
                                : ((float)pair >= high ? 1.0f : 0.0f);
        ramp = fminf(1.0f, fmaxf(0.0f, ramp));
        const float mask = 1.0f - ramp;
        inv_freq[pair] = interpolated * (1.0f - mask) + extrapolated * mask;
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* q/k RMSNorm + NeoX RoPE + paged KV write                            */
/* ------------------------------------------------------------------ */

/* Double sum of squares through the power-of-two shared-memory tree of
 * qwen38_qk_norm_partial_rope_cache8_kernel (src/axiom_qwen38_attention.cu:503-513)
 * and axiom_qwen_qknorm_rope_precise_kernel (src/axiom_cuda_precise.cu:113-120). */
static double sum_squares_tree_f64(const float *x, uint32_t n) {
    double cell[1024];
    uint32_t width = 1u;
    while (width < n) width <<= 1u;
    for (uint32_t i = 0; i < width; ++i) cell[i] = i < n ? (double)x[i] * (double)x[i] : 0.0;
    for (uint32_t stride = width >> 1u; stride != 0u; stride >>= 1u) {
        for (uint32_t i = 0; i < stride; ++i) cell[i] += cell[i + stride];
    }
    return cell[0];
}

/* One head: src/axiom_qwen38_attention.cu:514-541.  inv = (float)(1/sqrt(ss/D+eps))
 * in FP64; n = (x*inv)*w in FP32; NeoX pairs (p, p+rope_dim/2); angle =
 * (float)pos * f; cos and sin each multiplied by mscale; a single BF16 rounding
 * at the end.  The two rotation sums are fma(first, c, -(second*s)) and
 * fma(second, c, first*s): the contraction the reference's build applies to
 * `first * cosine - second * sine` and `first * sine + second * cosine`,
 * settled against its kernel on the GPU (the draft kernel below fuses the
 * first product of both sums). */
static void qk_head(const uint16_t *in, const uint16_t *gamma, uint32_t head_dim, uint32_t rope_dim,
                    float eps, const float *cosine, const float *sine, uint16_t *out) {
    float x[1024], n[1024];
    for (uint32_t i = 0; i < head_dim; ++i) x[i] = axo_bf16_to_f32(in[i]);
    const double ss = sum_squares_tree_f64(x, head_dim);
    const float inverse = (float)(1.0 / sqrt(ss / (double)head_dim + (double)eps));
    for (uint32_t i = 0; i < head_dim; ++i) n[i] = (x[i] * inverse) * axo_bf16_to_f32(gamma[i]);
    const uint32_t half = rope_dim / 2u;
    for (uint32_t p = 0; p < half; ++p) {
        const float first = n[p], second = n[p + half];
        out[p] = axo_f32_to_bf16(fmaf(first, cosine[p], -(second * sine[p])));
        out[p + half] = axo_f32_to_bf16(fmaf(second, cosine[p], first * sine[p]));
    }
    for (uint32_t i = rope_dim; i < head_dim; ++i) out[i] = axo_f32_to_bf16(n[i]);
}

/* The BF16 ("draft") rounding convention of the same step: qk_rmsnorm_rope_bf16_kernel followed by
 * round_f32_to_bf16_inplace_kernel (src/axiom_qwen38_dspark_compute.cu:250-300,210-213; layer sequence
 * :1816-1825).  FP32 squares through the kernel's shared-memory tree (strides D/2 .. 1), inv =
 * rsqrtf(ss/D + eps) (restated as 1/sqrtf: the device's rsqrtf is an approximation within 2 ulp, hence the
 * 1-BF16-ulp tolerance of the parity tests), n = bf16((x*inv)*w) rounded BEFORE the rotation, full-head NeoX
 * rotation with cos/sin from the caller's [position][cos(D/2) | sin(D/2)] table, result rounded to BF16.
 * x: [tokens][heads][head_dim] BF16 in place; a token whose position is outside the table is left untouched
 * and reported through *status (the reference kernel returns early). */
int axo_qk_norm_rope_round_after_norm_bf16(uint16_t *x, const uint16_t *gamma, const float *rope_table,
                                           uint32_t table_positions, const uint32_t *positions, uint32_t tokens,
                                           uint32_t heads, uint32_t head_dim, float eps, uint32_t *status) {
    if (!x || !gamma || !rope_table || !positions || head_dim == 0u || head_dim > 1024u || (head_dim & (head_dim - 1u))) {
        return AXO_INVALID;
    }
    const uint32_t half = head_dim / 2u;
    int bad = 0;
    AXO_PARALLEL_FOR
    for (int64_t t = 0; t < (int64_t)tokens; ++t) {
        const uint32_t pos = positions[t];
        if (pos >= table_positions) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
            bad = 1;
            continue;
        }
        const float *cs = rope_table + (size_t)pos * head_dim;
        for (uint32_t h = 0; h < heads; ++h) {
            uint16_t *row = x + ((size_t)t * heads + h) * head_dim;
            float v[1024], cell[1024], n[1024];
            for (uint32_t i = 0; i < head_dim; ++i) {
                v[i] = axo_bf16_to_f32(row[i]);
                cell[i] = v[i] * v[i];
            }
            for (uint32_t stride = half; stride != 0u; stride >>= 1u) {
                for (uint32_t i = 0; i < stride; ++i) cell[i] += cell[i + stride];
            }
            const float inverse = 1.0f / sqrtf(cell[0] / (float)head_dim + eps);
            for (uint32_t i = 0; i < head_dim; ++i) {
                n[i] = axo_bf16_to_f32(axo_f32_to_bf16((v[i] * inverse) * axo_bf16_to_f32(gamma[i])));
            }
            for (uint32_t p = 0; p < half; ++p) {
                const float a = n[p], b = n[p + half], c = cs[p], sn = cs[half + p];
                row[p] = axo_f32_to_bf16(fmaf(a, c, -(b * sn)));
                row[p + half] = axo_f32_to_bf16(fmaf(a, sn, b * c));
            }
        }
    }
    if (status && bad && *status == 0u) *status = 1u;
    return AXO_OK;
}

/* The reference's host-built rotary table of that convention: initialize_rope_cache
 * (src/axiom_qwen38_dspark_compute.cu:1459-1513) with the frequencies of axo_yarn_inv_freq_host_table. */
int axo_rope_table_host(const float *inv_freq, uint32_t head_dim, float mscale, uint32_t positions, float *out) {
    if (!inv_freq || !out || (head_dim & 1u)) return AXO_INVALID;
    const uint32_t half = head_dim / 2u;
    for (uint32_t pos = 0; pos < positions; ++pos) {
        float *row = out + (size_t)pos * head_dim;
        const float t = (float)pos;
        for (uint32_t p = 0; p < half; ++p) {
            const float angle = t * inv_freq[p];
            row[p] = cosf(angle) * mscale;
            row[half + p] = sinf(angle) * mscale;
        }
    }
    return AXO_OK;
}

/* Paged addressing: axiom_kv_pool_store_paged_f32_kernel
 * (src/axiom_cuda.cu:16954-16969), contract include/axiom/axiom.h:615-630;
 * ring indexing of the logical block as in src/axiom_qwen38_attention.cu:629-634. */
int axo_qk_norm_rope_paged_bf16(const axo_qk_params *p, uint16_t *q, const uint16_t *k,
                                const uint16_t *v, const uint16_t *q_gamma,
                                const uint16_t *k_gamma, const float *inv_freq,
                                const uint32_t *positions, const int32_t *block_tables,
                                uint16_t *k_pool, uint16_t *v_pool, uint16_t *k_out,
                                uint32_t *status) {
    if (!p || !positions || !inv_freq || p->tokens == 0u || p->head_dim == 0u ||
        p->head_dim > 1024u || p->rope_dim > p->head_dim || (p->rope_dim & 1u)) {
        return AXO_INVALID;
    }
    if ((p->q_heads && (!q || !q_gamma)) || (p->k_heads && (!k || !k_gamma))) return AXO_INVALID;
    const int paged = k_pool != NULL;
    if (paged && (!block_tables || p->block_tokens == 0u || p->n_layers == 0u ||
                  p->layer >= p->n_layers || p->tbl_stride == 0u ||
                  p->pool_stride < p->k_heads * p->head_dim)) {
        return AXO_INVALID;
    }
    const uint32_t half = p->rope_dim / 2u;
    const uint32_t kv_dim = p->k_heads * p->head_dim;
    int bad = 0;
    AXO_PARALLEL_FOR
    for (int64_t t = 0; t < (int64_t)p->tokens; ++t) {
        float cosine[512], sine[512];
        const uint32_t pos = positions[t];
        for (uint32_t pr = 0; pr < half; ++pr) {
            const float angle = (float)pos * inv_freq[pr];
            cosine[pr] = cosf(angle) * p->mscale;
            sine[pr] = sinf(angle) * p->mscale;
        }
        for (uint32_t h = 0; h < p->q_heads; ++h) {
            uint16_t *row = q + ((size_t)t * p->q_heads + h) * p->head_dim;
            uint16_t tmp[1024];
            qk_head(row, q_gamma, p->head_dim, p->rope_dim, p->eps, cosine, sine, tmp);
            memcpy(row, tmp, sizeof(uint16_t) * p->head_dim);
        }
        uint16_t *dst_k = NULL, *dst_v = NULL;
        if (paged) {
            uint32_t lb = pos / p->block_tokens;
            int ok = 1;
            if (p->ring) lb %= p->tbl_stride;
            else if (lb >= p->tbl_stride) ok = 0;
            int32_t pb = -1;
            if (ok) {
                pb = block_tables[(size_t)(p->per_token_table ? t : 0) * p->tbl_stride + lb];
                if (pb < 0 || (uint32_t)pb >= p->n_blocks) ok = 0;
            }
            if (ok) {
                const uint64_t base = (((uint64_t)pb * p->n_layers + p->layer) * p->block_tokens +
                                       pos % p->block_tokens) * p->pool_stride;
                dst_k = k_pool + base;
                if (v_pool && v) dst_v = v_pool + base;
            } else {
#ifdef _OPENMP
#pragma omp atomic write
#endif
                bad = 1;
            }
        }
        for (uint32_t h = 0; h < p->k_heads; ++h) {
            const uint16_t *row = k + ((size_t)t * p->k_heads + h) * p->head_dim;
            uint16_t tmp[1024];
            qk_head(row, k_gamma, p->head_dim, p->rope_dim, p->eps, cosine, sine, tmp);
            if (dst_k) memcpy(dst_k + (size_t)h * p->head_dim, tmp, sizeof(uint16_t) * p->head_dim);
            if (k_out) memcpy(k_out + ((size_t)t * p->k_heads + h) * p->head_dim, tmp, sizeof(uint16_t) * p->head_dim);
        }
        if (dst_v) memcpy(dst_v, v + (size_t)t * kv_dim, sizeof(uint16_t) * kv_dim);
    }
    if (status && bad && *status == 0u) *status = 1u;
    return AXO_OK;
}

/* E4M3 image of BF16 cache rows at scale 1: qwen38_kv_encode_e4m3fn_scale1
 * (reference src/axiom_qwen38_attention.cu:245-248) applied to BF16-valued floats. */
int axo_bf16_to_e4m3_scale1(const uint16_t *in, uint8_t *out, uint64_t count) {
    if (!in || !out) return AXO_INVALID;
    for (uint64_t i = 0; i < count; ++i) {
        uint32_t bits = (uint32_t)in[i] << 16;
        float f;
        memcpy(&f, &bits, sizeof f);
        out[i] = axo_e4m3_encode_satfinite(f);
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* embedding gather                                                    */
/* ------------------------------------------------------------------ */

/* qwen38_embedding_gather_columns_kernel (src/axiom_qwen38_model.cu:321-341):
 * an id at or beyond the vocabulary yields an all-zero row. */
int axo_embedding_gather_bf16(const uint16_t *table, uint32_t vocab, uint32_t hidden,
                              const uint32_t *ids, uint32_t tokens, uint16_t *out) {
    if (!table || !ids || !out || vocab == 0u || hidden == 0u || tokens == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t t = 0; t < (int64_t)tokens; ++t) {
        uint16_t *dst = out + (size_t)t * hidden;
        if (ids[t] >= vocab) memset(dst, 0, sizeof(uint16_t) * hidden);
        else memcpy(dst, table + (size_t)ids[t] * hidden, sizeof(uint16_t) * hidden);
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* generic single-row F32 ops                                          */
/* ------------------------------------------------------------------ */

/* axiom_rmsnorm_f32_device_kernel (src/axiom_cuda.cu:14530-14551): 256 strided
 * float partial sums + full shared-memory tree; that unit is built with
 * --use_fast_math, so products and sums contract to fma and rsqrt/divide are
 * approximate on the device: comparisons against this use a tolerance. */
int axo_rmsnorm_f32(const float *w, const float *x, float *out, uint32_t count, float eps) {
    if (!w || !x || !out || count == 0u) return AXO_INVALID;
    const float ss = sum_squares_tree256(x, count);
    const float inv = rsqrt_f32(ss / (float)count + eps);
    for (uint32_t i = 0; i < count; ++i) out[i] = (x[i] * inv) * w[i];
    return AXO_OK;
}

/* axiom_rmsnorm_f32_hp_device_kernel (src/axiom_cuda.cu:14556-14577). */
int axo_rmsnorm_f32_hp(const float *w, const float *x, float *out, uint32_t count, float eps) {
    if (!w || !x || !out || count == 0u) return AXO_INVALID;
    double partial[256];
    for (uint32_t lane = 0; lane < 256u; ++lane) {
        double s = 0.0;
        for (uint32_t f = lane; f < count; f += 256u) s += (double)x[f] * (double)x[f];
        partial[lane] = s;
    }
    for (uint32_t stride = 128u; stride != 0u; stride >>= 1u) {
        for (uint32_t lane = 0; lane < stride; ++lane) partial[lane] += partial[lane + stride];
    }
    const float inv = (float)(1.0 / sqrt(partial[0] / (double)count + (double)eps));
    for (uint32_t i = 0; i < count; ++i) out[i] = (x[i] * inv) * w[i];
    return AXO_OK;
}

/* axiom_rmsnorm_f32_b1_device_kernel (src/axiom_cuda.cu:14583-14655): float4
 * strided fmaf chains, warp shuffle tree, 8 warp sums reduced by warp 0. */
int axo_rmsnorm_f32_b1(const float *w, const float *x, float *out, uint32_t count, float eps) {
    if (!w || !x || !out || count == 0u) return AXO_INVALID;
    float lane_sum[256];
    const uint32_t vec = count >> 2u, tail = vec << 2u;
    for (uint32_t t = 0; t < 256u; ++t) {
        float s = 0.0f;
        for (uint32_t i = t; i < vec; i += 256u) {
            for (uint32_t j = 0; j < 4u; ++j) s = fmaf(x[4u * i + j], x[4u * i + j], s);
        }
        for (uint32_t i = tail + t; i < count; i += 256u) s = fmaf(x[i], x[i], s);
        lane_sum[t] = s;
    }
    float warp_sum[32] = {0};
    for (uint32_t wp = 0; wp < 8u; ++wp) {
        float v[32];
        memcpy(v, lane_sum + 32u * wp, sizeof(v));
        for (uint32_t off = 16u; off != 0u; off >>= 1u) {
            for (uint32_t l = 0; l + off < 32u; ++l) v[l] = v[l] + v[l + off];
        }
        warp_sum[wp] = v[0];
    }
    for (uint32_t off = 16u; off != 0u; off >>= 1u) {
        for (uint32_t l = 0; l + off < 32u; ++l) warp_sum[l] = warp_sum[l] + warp_sum[l + off];
    }
    const float inv = rsqrt_f32(warp_sum[0] / (float)count + eps);
    for (uint32_t i = 0; i < count; ++i) out[i] = (x[i] * inv) * w[i];
    return AXO_OK;
}

/* axiom_head_rmsnorm_f32_device_kernel (src/axiom_cuda.cu:15119-15141). */
int axo_head_rmsnorm_f32(float *x, uint32_t heads, uint32_t head_dim, float eps) {
    if (!x || heads == 0u || head_dim == 0u) return AXO_INVALID;
    for (uint32_t h = 0; h < heads; ++h) {
        float *row = x + (size_t)h * head_dim;
        const float ss = sum_squares_tree256(row, head_dim);
        const float inv = rsqrt_f32(ss / (float)head_dim + eps);
        for (uint32_t i = 0; i < head_dim; ++i) row[i] *= inv;
    }
    return AXO_OK;
}

/* axiom_qwen_qk_rmsnorm_w_f32_kernel (src/axiom_cuda.cu:15347-15366). */
int axo_qk_rmsnorm_w_f32(float *x, const float *w, uint32_t heads, uint32_t head_dim, float eps) {
    if (!x || !w || heads == 0u || head_dim == 0u) return AXO_INVALID;
    for (uint32_t h = 0; h < heads; ++h) {
        float *row = x + (size_t)h * head_dim;
        double partial[256];
        for (uint32_t lane = 0; lane < 256u; ++lane) {
            double s = 0.0;
            for (uint32_t f = lane; f < head_dim; f += 256u) s += (double)row[f] * (double)row[f];
            partial[lane] = s;
        }
        for (uint32_t stride = 128u; stride != 0u; stride >>= 1u) {
            for (uint32_t lane = 0; lane < stride; ++lane) partial[lane] += partial[lane + stride];
        }
        const float inv = (float)(1.0 / sqrt(partial[0] / (double)head_dim + (double)eps));
        for (uint32_t i = 0; i < head_dim; ++i) row[i] = (row[i] * inv) * w[i];
    }
    return AXO_OK;
}

/* axiom_qwen_rope_neox_precise_kernel / partial twin
 * (src/axiom_cuda_precise.cu:39-52,84-97): freq = powf(theta, -2*ic/n_rot),
 * pairs (ic, ic + n_rot/2), dims >= n_rot untouched, no rounding. */
int axo_rope_neox_f32(float *x, uint32_t heads, uint32_t head_dim, uint32_t n_rot,
                      uint32_t pos, float theta) {
    if (!x || heads == 0u || head_dim == 0u || n_rot == 0u || n_rot > head_dim || (n_rot & 1u)) return AXO_INVALID;
    const uint32_t half = n_rot / 2u;
    for (uint32_t h = 0; h < heads; ++h) {
        float *row = x + (size_t)h * head_dim;
        for (uint32_t ic = 0; ic < half; ++ic) {
            const float freq = powf(theta, -2.0f * (float)ic / (float)n_rot);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), s = sinf(ang);
            const float x0 = row[ic], x1 = row[ic + half];
            row[ic] = fmaf(x0, c, -(x1 * s));
            row[ic + half] = fmaf(x0, s, x1 * c);
        }
    }
    return AXO_OK;
}

/* axiom_qwen_qknorm_rope_precise_kernel (src/axiom_cuda_precise.cu:105-134). */
int axo_qknorm_rope_f32(float *x, const float *w, uint32_t heads, uint32_t head_dim,
                        uint32_t pos, float theta, float eps) {
    if (!x || !w || heads == 0u || head_dim == 0u || head_dim > 1024u ||
        (head_dim & (head_dim - 1u)) != 0u) {
        return AXO_INVALID;
    }
    const uint32_t half = head_dim / 2u;
    for (uint32_t h = 0; h < heads; ++h) {
        float *row = x + (size_t)h * head_dim;
        float n[1024];
        const double ss = sum_squares_tree_f64(row, head_dim);
        const float inv = (float)(1.0 / sqrt(ss / (double)head_dim + (double)eps));
        for (uint32_t i = 0; i < head_dim; ++i) n[i] = (row[i] * inv) * w[i];
        for (uint32_t ic = 0; ic < half; ++ic) {
            const float freq = powf(theta, -2.0f * (float)ic / (float)head_dim);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), s = sinf(ang);
            row[ic] = fmaf(n[ic], c, -(n[ic + half] * s));
            row[ic + half] = fmaf(n[ic], s, n[ic + half] * c);
        }
    }
    return AXO_OK;
}

/* axiom_add_f32_device_kernel (src/axiom_cuda.cu:15803-15810). */
int axo_add_f32(const float *a, const float *b, float *out, uint32_t count) {
    if (!a || !b || !out || count == 0u) return AXO_INVALID;
    for (uint32_t i = 0; i < count; ++i) out[i] = a[i] + b[i];
    return AXO_OK;
}

/* axiom_silu_mul_f32_kernel (src/axiom_cuda.cu:17278-17293): clamp only when
 * clamp_abs > 1e-6; gate clamped from above only, up clamped both sides. */
int axo_silu_mul_f32(const float *gate, const float *up, float *out, uint32_t count,
                     float clamp_abs) {
    if (!gate || !up || !out || count == 0u) return AXO_INVALID;
    for (uint32_t i = 0; i < count; ++i) {
        float g = gate[i], u = up[i];
        if (clamp_abs > 1.0e-6f) {
            g = fminf(g, clamp_abs);
            u = fminf(fmaxf(u, -clamp_abs), clamp_abs);
        }
        out[i] = (g / (1.0f + expf(-g))) * u;
    }
    return AXO_OK;
}

/* axiom_kv_pool_store_paged_f32_kernel (src/axiom_cuda.cu:16954-16969). */
int axo_kv_pool_store_paged_f32(const float *k_stage, const float *v_stage, float *k_pool,
                                float *v_pool, const int32_t *block_tables,
                                const uint32_t *pos, uint32_t active, uint32_t tbl_stride,
                                uint32_t n_layers, uint32_t layer, uint32_t block_tokens,
                                uint32_t pool_stride, uint32_t kv_dim) {
    if (!k_stage || !v_stage || !k_pool || !v_pool || !block_tables || !pos || active == 0u ||
        tbl_stride == 0u || n_layers == 0u || layer >= n_layers || block_tokens == 0u ||
        kv_dim == 0u || pool_stride < kv_dim) {
        return AXO_INVALID;
    }
    for (uint32_t a = 0; a < active; ++a) {
        const uint32_t p = pos[a];
        const uint32_t pb = (uint32_t)block_tables[(size_t)a * tbl_stride + p / block_tokens];
        const uint64_t base = (((uint64_t)pb * n_layers + layer) * block_tokens + p % block_tokens) * pool_stride;
        memcpy(k_pool + base, k_stage + (size_t)a * kv_dim, sizeof(float) * kv_dim);
        memcpy(v_pool + base, v_stage + (size_t)a * kv_dim, sizeof(float) * kv_dim);
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* generic single-token embedding gathers                              */
/* ------------------------------------------------------------------ */

static float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0u) {
        if (man == 0u) {
            bits = sign;
        } else {  /* subnormal: renormalise */
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31u) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

/* axiom_q8_0_embedding_gather_f32_kernel (reference src/axiom_cuda.cu:2213-2240): rows of
 * hidden/32 blocks of 34 bytes, little-endian F16 scale then 32 signed bytes; a token id at
 * or beyond token_count gives zeros. */
int axo_q8_0_embedding_gather_f32(const uint8_t *embedding, uint32_t token_id, uint32_t token_count,
                                  uint32_t hidden, float *out) {
    if (!embedding || !out || hidden == 0u || (hidden % 32u) != 0u) return AXO_INVALID;
    const uint8_t *row = embedding + (size_t)token_id * (hidden / 32u) * 34u;
    for (uint32_t i = 0; i < hidden; ++i) {
        if (token_id >= token_count) {
            out[i] = 0.0f;
            continue;
        }
        const uint8_t *blk = row + (size_t)(i >> 5) * 34u;
        const float d = f16_bits_to_f32((uint16_t)(blk[0] | ((uint16_t)blk[1] << 8)));
        out[i] = d * (float)((const int8_t *)(blk + 2))[i & 31u];
    }
    return AXO_OK;
}

/* axiom_f16_embedding_streams_device_kernel (reference src/axiom_cuda.cu:14458-14469) */
int axo_f16_embedding_streams_f32(const uint16_t *embedding, uint32_t token_id, uint32_t hidden,
                                  uint32_t streams, float *out) {
    if (!embedding || !out || hidden == 0u || streams == 0u) return AXO_INVALID;
    for (uint64_t idx = 0; idx < (uint64_t)hidden * streams; ++idx) {
        out[idx] = f16_bits_to_f32(embedding[(size_t)token_id * hidden + (uint32_t)(idx % hidden)]);
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* greedy selection                                                    */
/* ------------------------------------------------------------------ */

/* qwen38_top1_8_kernel / qwen38_top1_select (reference src/axiom_qwen38_model.cu:408-455,
 * 483-493): the largest finite logit of each row, the smallest id among equal values, and
 * invalid = 1 when any logit of the row is not finite; id 0xffffffff when none is finite.
 * out: rows x {float value, uint32 token_id, uint32 invalid} packed as three uint32 words. */
int axo_top1_f32(const float *logits, uint32_t rows, uint32_t vocab, uint32_t *out) {
    if (!logits || !out || rows == 0u || vocab == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        float best = -INFINITY;
        uint32_t best_id = 0xffffffffu, invalid = 0u;
        for (uint32_t i = 0; i < vocab; ++i) {
            const float v = logits[(size_t)r * vocab + i];
            if (!isfinite(v)) invalid = 1u;
            else if (v > best || (v == best && i < best_id)) { best = v; best_id = i; }
        }
        memcpy(out + 3 * r, &best, sizeof best);
        out[3 * r + 1] = best_id;
        out[3 * r + 2] = invalid;
    }
    return AXO_OK;
}

/* ------------------------------------------------------------------ */
/* FP8 GEMM scale epilogue                                             */
/* ------------------------------------------------------------------ */

/* fp8_group_row_scale_bf16_epilogue_kernel (reference src/axiom_qwen38_fp8.cu:250-262):
 * out[token][feature] = bf16((raw * weight_scale[feature]) * input_scale[token]), weight scales
 * stored as BF16, token-major layout. */
int axo_fp8_row_scale_epilogue_bf16(const float *raw, const uint16_t *weight_scale,
                                    const float *input_scale, uint32_t rows, uint32_t cols,
                                    uint16_t *out_bf16) {
    if (!raw || !weight_scale || !input_scale || !out_bf16 || rows == 0u || cols == 0u) return AXO_INVALID;
    AXO_PARALLEL_FOR
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        for (uint32_t c = 0; c < cols; ++c) {
            const float scaled = raw[(size_t)r * cols + c] * axo_bf16_to_f32(weight_scale[c]);
            out_bf16[(size_t)r * cols + c] = axo_f32_to_bf16(scaled * input_scale[r]);
        }
    }
    return AXO_OK;
}

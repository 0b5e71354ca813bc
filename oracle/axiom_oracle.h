/*
 * CPU oracle for the fused elementwise / reduction / quantize path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the arithmetic of
 * the reference kernels (file:line citations are relative to the reference
 * project root).  It exists so the CUDA library can be checked against an
 * independent implementation; nothing in the shipped library links, loads or
 * calls it.  Only the test-suite, the smoke entry and the CPU-baseline leg of
 * the benchmark may use it.
 *
 * Parity status: the reference ships no golden vector file for these ops
 * (its own tests hold closed-form known-answer cases only).  The oracle is
 * pinned against (a) those closed-form cases, (b) the host paths of the CUDA
 * toolkit FP8/FP4 converters the reference calls, and (c) outputs of the
 * reference's own kernels compiled for sm_100a and run on a B200, committed as
 * fixtures under tests/golden/.
 */
#ifndef AXIOM_ORACLE_H
#define AXIOM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar numeric primitives ---- */
uint16_t axo_f32_to_bf16(float value);           /* RN-even, NaN kept quiet */
float axo_bf16_to_f32(uint16_t bits);
float axo_bf16_round(float value);
float axo_e4m3_decode(uint8_t code);             /* 0x7f / 0xff -> NaN */
uint8_t axo_e4m3_encode_satfinite(float value);  /* RN-even, saturate to +-448, NaN -> 0x7f */
uint8_t axo_e4m3_encode_scale(float value);      /* block-scale flavour: 0 -> 0x20, NaN -> 0x7e */
uint8_t axo_e2m1_encode(float value);            /* RN-even on {0,.5,1,1.5,2,3,4,6}, NaN -> 7 */
float axo_e2m1_decode(uint8_t nibble);

/* ---- NVFP4 activation quantizer ---- */
/* One row-major [rows x cols] F32 matrix -> packed E2M1 codes [rows x cols/2]
 * and canonical E4M3 block scales [rows x cols/16]. */
int axo_nvfp4_quantize_f32(const float *input, uint32_t rows, uint32_t cols,
                           float global_scale, uint8_t *codes, uint8_t *scales);
int axo_nvfp4_quantize_bf16(const uint16_t *input, uint32_t rows, uint32_t cols,
                            float global_scale, uint8_t *codes, uint8_t *scales);
/* Tiled (tensor-core scale plane) layout helpers. */
uint64_t axo_scale_tiled_bytes(uint32_t outer, uint32_t inner);
uint64_t axo_scale_tiled_offset(uint32_t outer, uint32_t inner, uint32_t inner_tiles);
int axo_scales_canonical_to_tiled(const uint8_t *canonical, uint32_t rows, uint32_t groups,
                                  uint8_t *tiled);

/* ---- FP8 E4M3 per-token quantizer ---- */
int axo_fp8_quantize_f32(const float *input, uint32_t rows, uint32_t cols,
                         uint8_t *codes, float *scales);
int axo_fp8_quantize_bf16(const uint16_t *input, uint32_t rows, uint32_t cols,
                          uint8_t *codes, float *scales, uint32_t *status);

/* ---- residual add + RMSNorm ---- */
int axo_add_bf16(const uint16_t *a, const uint16_t *b, uint64_t count, uint16_t *out);
/* residual <- bf16(residual + hidden); norm <- bf16((r * inv) * gamma).  hidden may be
 * NULL (norm only).  norm_f32 (optional) receives the BF16-valued result as F32. */
int axo_add_rmsnorm_bf16(const uint16_t *hidden, const uint16_t *residual_in,
                         const uint16_t *gamma, float eps, uint32_t rows, uint32_t cols,
                         uint16_t *residual_out, uint16_t *norm_out);
int axo_add_rmsnorm_nvfp4_bf16(const uint16_t *hidden, const uint16_t *residual_in,
                               const uint16_t *gamma, float eps, uint32_t rows, uint32_t cols,
                               float global_scale, uint16_t *residual_out, uint16_t *norm_out,
                               uint8_t *codes, uint8_t *scales);

/* ---- SwiGLU ---- */
float axo_silu_mul(float gate, float up);
/* gate_up rows are [gate(width) | up(width)] BF16. */
int axo_swiglu_f32(const uint16_t *gate_up, uint32_t rows, uint32_t width, float *out);
int axo_swiglu_fp8_bf16(const uint16_t *gate_up, uint32_t rows, uint32_t width,
                        uint8_t *codes, float *scales);
int axo_swiglu_nvfp4_bf16(const uint16_t *gate_up, uint32_t rows, uint32_t width,
                          float global_scale, uint8_t *codes, uint8_t *scales);

/* ---- YaRN / RoPE / q-k norm / paged KV ---- */
typedef struct {
    float theta;
    float factor;            /* <= 1 disables YaRN interpolation */
    float original_context;
    float beta_fast;
    float beta_slow;
    uint32_t rope_dim;       /* rotated dims (<= head_dim), even */
} axo_rope_params;

/* Device-formula flavour (all FP32). */
int axo_yarn_inv_freq(const axo_rope_params *p, float *inv_freq /* rope_dim/2 */);
/* Host-table flavour (FP64 correction bounds, clamped). */
int axo_yarn_inv_freq_host_table(const axo_rope_params *p, float *inv_freq);
float axo_yarn_mscale(float factor);

typedef struct {
    uint32_t tokens;
    uint32_t q_heads;
    uint32_t k_heads;
    uint32_t head_dim;
    uint32_t rope_dim;
    float eps;
    float mscale;
    /* paged cache */
    uint32_t block_tokens;
    uint32_t n_layers;
    uint32_t layer;
    uint32_t pool_stride;    /* elements per (block, layer, slot) row, >= k_heads*head_dim */
    uint32_t tbl_stride;     /* int32 entries per block-table row */
    uint32_t n_blocks;       /* physical blocks in the pool (bounds check) */
    uint32_t ring;           /* 1: logical block = (pos / BT) % tbl_stride */
    uint32_t per_token_table;/* 1: token t reads table row t; 0: every token reads row 0 */
} axo_qk_params;

/* q [tokens][q_heads][head_dim] in place; k [tokens][k_heads][head_dim] read-only;
 * rotated K rows scattered into k_pool (BF16); v optional -> v_pool.  k_out optional
 * contiguous copy of rotated K.  status (optional) receives 1 if any token addressed
 * outside the table / pool (that token's cache write is skipped). */
int axo_qk_norm_rope_paged_bf16(const axo_qk_params *p, uint16_t *q, const uint16_t *k,
                                const uint16_t *v, const uint16_t *q_gamma,
                                const uint16_t *k_gamma, const float *inv_freq,
                                const uint32_t *positions, const int32_t *block_tables,
                                uint16_t *k_pool, uint16_t *v_pool, uint16_t *k_out,
                                uint32_t *status);

/* BF16 ("draft") rounding convention of q/k norm + RoPE, x [tokens][heads][head_dim] in place
 * (src/axiom_qwen38_dspark_compute.cu:250-300 + :210-213); rope_table [table_positions][head_dim] = cos | sin */
int axo_qk_norm_rope_round_after_norm_bf16(uint16_t *x, const uint16_t *gamma, const float *rope_table,
                                           uint32_t table_positions, const uint32_t *positions, uint32_t tokens,
                                           uint32_t heads, uint32_t head_dim, float eps, uint32_t *status);
/* host rotary table of that convention (src/axiom_qwen38_dspark_compute.cu:1459-1513) */
int axo_rope_table_host(const float *inv_freq, uint32_t head_dim, float mscale, uint32_t positions, float *out);

/* static-scale E4M3 quantizer (src/axiom_qwen38_fp8.cu:96-107) */
int axo_fp8_quantize_static_f32(const float *input, uint64_t count, float scale, uint8_t *codes);

/* y = bf16(attention * sigmoid(gate)), optional BF16 copy, optional NVFP4 quantize of y */
int axo_sigmoid_gate_nvfp4_bf16(const uint16_t *attention, const uint16_t *gate, uint32_t rows,
                                uint32_t width, float global_scale, uint16_t *out_bf16,
                                uint8_t *codes, uint8_t *scales);

/* E4M3 codes (scale 1, saturating) of BF16 values: the FP8 flavour of the KV cache */
int axo_bf16_to_e4m3_scale1(const uint16_t *in, uint8_t *out, uint64_t count);

/* ---- embedding gather ---- */
int axo_embedding_gather_bf16(const uint16_t *table, uint32_t vocab, uint32_t hidden,
                              const uint32_t *ids, uint32_t tokens, uint16_t *out);

/* ---- FP8 GEMM scale epilogue: bf16((raw * weight_scale[feature]) * input_scale[token]) ---- */
int axo_fp8_row_scale_epilogue_bf16(const float *raw, const uint16_t *weight_scale,
                                    const float *input_scale, uint32_t rows, uint32_t cols,
                                    uint16_t *out_bf16);

/* ---- greedy selection: rows x {float value, uint32 id, uint32 invalid} ---- */
int axo_top1_f32(const float *logits, uint32_t rows, uint32_t vocab, uint32_t *out);

/* ---- generic single-token embedding gathers (Q8_0 blocks / F16 rows) ---- */
int axo_q8_0_embedding_gather_f32(const uint8_t *embedding, uint32_t token_id, uint32_t token_count,
                                  uint32_t hidden, float *out);
int axo_f16_embedding_streams_f32(const uint16_t *embedding, uint32_t token_id, uint32_t hidden,
                                  uint32_t streams, float *out);

/* ---- generic single-row F32 ops (runtime ABI semantics) ---- */
int axo_rmsnorm_f32(const float *w, const float *x, float *out, uint32_t count, float eps);
int axo_rmsnorm_f32_hp(const float *w, const float *x, float *out, uint32_t count, float eps);
int axo_rmsnorm_f32_b1(const float *w, const float *x, float *out, uint32_t count, float eps);
int axo_head_rmsnorm_f32(float *x, uint32_t heads, uint32_t head_dim, float eps);
int axo_qk_rmsnorm_w_f32(float *x, const float *w, uint32_t heads, uint32_t head_dim, float eps);
int axo_rope_neox_f32(float *x, uint32_t heads, uint32_t head_dim, uint32_t n_rot,
                      uint32_t pos, float theta);
int axo_qknorm_rope_f32(float *x, const float *w, uint32_t heads, uint32_t head_dim,
                        uint32_t pos, float theta, float eps);
int axo_add_f32(const float *a, const float *b, float *out, uint32_t count);
int axo_silu_mul_f32(const float *gate, const float *up, float *out, uint32_t count,
                     float clamp_abs);
int axo_kv_pool_store_paged_f32(const float *k_stage, const float *v_stage, float *k_pool,
                                float *v_pool, const int32_t *block_tables,
                                const uint32_t *pos, uint32_t active, uint32_t tbl_stride,
                                uint32_t n_layers, uint32_t layer, uint32_t block_tokens,
                                uint32_t pool_stride, uint32_t kv_dim);

/* threads used by the row-parallel loops (OpenMP); 0 = library default */
void axo_set_threads(int threads);
int axo_get_threads(void);

#ifdef __cplusplus
}
#endif

#endif

/*
 * axiom_b200.h — C ABI of libaxiom_b200.so.
 *
 * A B200 (sm_100a) implementation of ONE path of the Axiom kernel: the fused
 * per-layer elementwise / reduction / quantize chain (residual add + RMSNorm,
 * per-head q/k RMSNorm + NeoX RoPE with YaRN + paged-KV write, SwiGLU, token
 * embedding gather, BF16 -> NVFP4 / FP8-E4M3 activation quantizers).
 *
 * The header has three parts:
 *   1. symbols that exist in the reference with the same name, signature and
 *      behaviour (each cites the reference declaration it replaces);
 *   2. append-only BF16 batched entry points for the fused path, in the three
 *      flavours the reference uses for its own ops:
 *        axiom_qwen38_fused_*_bf16_device(int device, raw pointers, void *stream)
 *            asynchronous on the given stream, cudaGetLastError() only
 *            (family convention, include/axiom/qwen38_nvfp4.h:27-37);
 *        axiom_runtime_*_bf16_device(runtime, axiom_device_buffer + byte offsets)
 *            span-checked, default stream, finish-after-launch
 *            (generic convention, include/axiom/axiom.h:438-486);
 *        axiom_runtime_*_bf16(runtime, host pointers)
 *            host I/O: upload, launch, download (convention of
 *            axiom_runtime_q8_0_matvec_f32, include/axiom/axiom.h:391-397);
 *   3. small helpers (scale-plane layout arithmetic).
 *
 * Citations are relative to the reference project root.  Plain pointers and
 * sizes only; usable from C and C++.  None of the calls is thread-safe on one
 * runtime; callers serialise (include/axiom/axiom_engine.h:39-40).
 */
#ifndef AXIOM_B200_H
#define AXIOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ====================================================================== */
/* Part 1 — reference-compatible symbols                                   */
/* ====================================================================== */

#define AXIOM_ABI_VERSION 1u /* include/axiom/axiom.h:11 */

/* include/axiom/axiom.h:19-28 */
typedef enum {
    AXIOM_OK = 0,
    AXIOM_ERR_INVALID_ARGUMENT = 1,
    AXIOM_ERR_UNSUPPORTED_BACKEND = 2,
    AXIOM_ERR_CUDA = 3,
    AXIOM_ERR_RUNTIME = 4,
    AXIOM_ERR_NOT_IMPLEMENTED = 5,
    AXIOM_ERR_IO = 6,
    AXIOM_ERR_BUDGET = 7,
} axiom_status;

/* include/axiom/axiom.h:30-33 */
typedef enum {
    AXIOM_BACKEND_CUDA = 1,
    AXIOM_BACKEND_CLUSTER = 2,
} axiom_backend;

/* include/axiom/axiom.h:35,42 — opaque */
typedef struct axiom_runtime axiom_runtime;
typedef struct axiom_device_buffer axiom_device_buffer;

/* include/axiom/axiom.h:119-124 */
typedef struct {
    uint32_t abi_version;
    axiom_backend backend;
    uint32_t device;
    uint64_t flags;
} axiom_config;

/* include/axiom/axiom.h:366-375 */
typedef struct {
    uint32_t abi_version;          /* in: AXIOM_ABI_VERSION, else the call is rejected */
    uint32_t header_abi_version;
    uint32_t runtime_abi_version;
    uint32_t struct_size;
    const char *version;
    const char *backend;           /* "cuda" */
    const char *build_target;      /* "sm_100a" */
    uint64_t flags;
} axiom_abi_info;

/* include/axiom/axiom.h:377-381 */
uint32_t axiom_abi_version(void);
const char *axiom_version(void);
int axiom_abi_info_get(axiom_abi_info *out);
int axiom_abi_check(uint32_t header_abi_version);
const char *axiom_status_string(int status);

/* include/axiom/axiom.h:383-384,386,388 */
int axiom_runtime_create(axiom_runtime **out, const axiom_config *config);
void axiom_runtime_destroy(axiom_runtime *runtime);
int axiom_runtime_device_count(uint32_t *out_count);
int axiom_runtime_device_id(const axiom_runtime *runtime, uint32_t *out_device);

/* include/axiom/axiom.h:411-437.  The CUDA pointer is a borrow. */
int axiom_device_buffer_create(axiom_runtime *runtime, axiom_device_buffer **out, uint64_t bytes);
void axiom_device_buffer_destroy(axiom_device_buffer *buffer);
int axiom_device_buffer_upload(axiom_device_buffer *buffer, uint64_t offset, const void *src_host, uint64_t bytes);
int axiom_device_buffer_download(axiom_device_buffer *buffer, uint64_t offset, void *dst_host, uint64_t bytes);
int axiom_device_buffer_copy(axiom_device_buffer *dst, uint64_t dst_offset, const axiom_device_buffer *src, uint64_t src_offset, uint64_t bytes);
int axiom_device_buffer_device_id(const axiom_device_buffer *buffer, uint32_t *out_device);
int axiom_device_buffer_cuda_pointer(const axiom_device_buffer *buffer, void **out_pointer);

/* Generic single-row F32 ops.  Default stream; after the launch the call
 * returns at once when AXIOM_CUDA_LAUNCH_ASYNC is truthy or the stream is being
 * captured, otherwise it synchronises (src/axiom_cuda.cu:162-200). */

/* include/axiom/axiom.h:438-447 — float partial sums, rsqrt; eps <= 0 means 1e-6 */
int axiom_runtime_rmsnorm_f32_device(axiom_runtime *runtime, const axiom_device_buffer *weight_f32, uint64_t weight_offset, const axiom_device_buffer *input, uint64_t input_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count, float eps);
/* include/axiom/axiom.h:451-460 — double sum of squares, (float)(1/sqrt) */
int axiom_runtime_rmsnorm_f32_hp_device(axiom_runtime *runtime, const axiom_device_buffer *weight_f32, uint64_t weight_offset, const axiom_device_buffer *input, uint64_t input_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count, float eps);
/* include/axiom/axiom.h:463-472 — float4 + shuffle reduction */
int axiom_runtime_rmsnorm_f32_b1_device(axiom_runtime *runtime, const axiom_device_buffer *weight_f32, uint64_t weight_offset, const axiom_device_buffer *input, uint64_t input_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count, float eps);
/* include/axiom/axiom.h:473-486 — two rows, one weight */
int axiom_runtime_rmsnorm_f32_dual_device(axiom_runtime *runtime, const axiom_device_buffer *weight_f32, uint64_t weight_offset, const axiom_device_buffer *input0, uint64_t input0_offset, axiom_device_buffer *out0, uint64_t out0_offset, const axiom_device_buffer *input1, uint64_t input1_offset, axiom_device_buffer *out1, uint64_t out1_offset, uint32_t count, float eps);
/* include/axiom/axiom.h:499-505 — weightless per-head norm, in place */
int axiom_runtime_head_rmsnorm_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, uint32_t heads, uint32_t head_dim, float eps);
/* include/axiom/axiom.h:507-514 */
int axiom_runtime_rope_neox_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, uint32_t heads, uint32_t head_dim, uint32_t pos, float theta);
/* include/axiom/axiom.h:518-526 */
int axiom_runtime_rope_neox_partial_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, uint32_t heads, uint32_t head_dim, uint32_t n_rot, uint32_t pos, float theta);
/* include/axiom/axiom.h:528-546 — per-head RMSNorm (double) x weight, then full-head NeoX RoPE */
int axiom_runtime_qknorm_rope_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, const axiom_device_buffer *w, uint64_t w_offset, uint32_t heads, uint32_t head_dim, uint32_t pos, float theta, float eps);
int axiom_runtime_qknorm_rope_pos_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, const axiom_device_buffer *w, uint64_t w_offset, const axiom_device_buffer *pos, uint64_t pos_offset, uint32_t heads, uint32_t head_dim, float theta, float eps);
int axiom_runtime_qknorm_rope_pos_dual_f32_device(axiom_runtime *runtime, axiom_device_buffer *q, uint64_t q_offset, const axiom_device_buffer *qw, uint64_t qw_offset, axiom_device_buffer *k, uint64_t k_offset, const axiom_device_buffer *kw, uint64_t kw_offset, const axiom_device_buffer *pos, uint64_t pos_offset, uint32_t q_heads, uint32_t k_heads, uint32_t head_dim, float theta, float eps);
/* include/axiom/axiom.h:548-556 */
int axiom_runtime_qk_rmsnorm_w_f32_device(axiom_runtime *runtime, axiom_device_buffer *x, uint64_t x_offset, const axiom_device_buffer *w, uint64_t w_offset, uint32_t heads, uint32_t head_dim, float eps);
/* include/axiom/axiom.h:674-690 — one K row and one V row per active sequence into the paged pools */
int axiom_runtime_kv_pool_store_paged_f32_device(axiom_runtime *runtime, const axiom_device_buffer *k_stage, uint64_t k_stage_offset, const axiom_device_buffer *v_stage, uint64_t v_stage_offset, axiom_device_buffer *k_pool, uint64_t k_pool_offset, axiom_device_buffer *v_pool, uint64_t v_pool_offset, const axiom_device_buffer *block_tables, uint64_t tbl_offset, const axiom_device_buffer *pos, uint64_t pos_offset, uint32_t active, uint32_t tbl_stride, uint32_t n_layers, uint32_t layer, uint32_t block_tokens, uint32_t pool_stride, uint32_t kv_dim);
/* include/axiom/axiom.h:742-750 */
int axiom_runtime_add_f32_device(axiom_runtime *runtime, const axiom_device_buffer *a, uint64_t a_offset, const axiom_device_buffer *b, uint64_t b_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count);
/* include/axiom/axiom.h:751-759 */
int axiom_runtime_silu_mul_f32_device(axiom_runtime *runtime, const axiom_device_buffer *gate, uint64_t gate_offset, const axiom_device_buffer *up, uint64_t up_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count);
/* include/axiom/axiom.h:787-796 */
int axiom_runtime_silu_mul_clamp_f32_device(axiom_runtime *runtime, const axiom_device_buffer *gate, uint64_t gate_offset, const axiom_device_buffer *up, uint64_t up_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t count, float clamp_abs);

/* Generic single-token embedding gathers (include/axiom/axiom.h:839-866; kernels src/axiom_cuda.cu:2213-2256,
 * 14458-14469).  Q8_0 rows: blocks of 34 bytes (little-endian F16 scale + 32 signed bytes), hidden % 32 == 0;
 * token id >= token_count gives a zero row in the device-token flavour and is rejected in the immediate one. */
int axiom_runtime_f16_embedding_streams_device(axiom_runtime *runtime, const axiom_device_buffer *embedding_f16, uint64_t embedding_offset, axiom_device_buffer *out_streams, uint64_t out_offset, uint32_t token_id, uint32_t hidden, uint32_t streams);
int axiom_runtime_q8_0_embedding_gather_f32_device(axiom_runtime *runtime, const axiom_device_buffer *embedding_q8, uint64_t embedding_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t token_id, uint32_t token_count, uint32_t hidden);
int axiom_runtime_q8_0_embedding_gather_token_f32_device(axiom_runtime *runtime, const axiom_device_buffer *embedding_q8, uint64_t embedding_offset, const axiom_device_buffer *token_id, uint64_t token_id_offset, axiom_device_buffer *out, uint64_t out_offset, uint32_t token_count, uint32_t hidden);

/* include/axiom/qwen38_nvfp4.h:30-37 — the exported NVFP4 quantizer oracle:
 * one F32 row -> cols/2 packed E2M1 bytes + cols/16 E4M3 scales (canonical
 * order); synchronises its stream before returning
 * (src/axiom_qwen38_nvfp4.cu:121-152). */
int axiom_qwen38_nvfp4_quantize_reference_f32(int device, const float *input, float input_global_scale, uint8_t *out_packed, uint8_t *out_scale, uint32_t cols, void *stream);

/* ====================================================================== */
/* Part 2 — BF16 batched entry points for the fused path (append-only)     */
/* ====================================================================== */

/* Activations are row-major [tokens x features] BF16 (uint16_t bit patterns);
 * a "row" is one token (the reference calls it a column of a column-major
 * [features, batch] matrix, include/axiom/qwen38_nvfp4_mlp.h:18-23).
 * `global_scale` is the NVFP4 multiplier G: block scale = e4m3((max/6)*G),
 * dequantisation divides by G (include/axiom/qwen38_nvfp4.h:12-13). */

/* Layout of the E4M3 block-scale plane. */
#define AXIOM_SCALE_LAYOUT_CANONICAL 0u /* scales[row * groups + group] (src/axiom_qwen38_nvfp4.cu:76) */
#define AXIOM_SCALE_LAYOUT_TILED 1u     /* 128x4 tiles of 512 B, cuBLASLt VEC16_UE4M3 (src/axiom_qwen38_nvfp4_mlp.cu:95-108) */

/* Device status word values written by kernels that meet bad DATA (never a trap). */
#define AXIOM_STATUS_WORD_OK 0u
#define AXIOM_STATUS_WORD_BAD_ADDRESS 1u   /* token id / block id / logical block out of range */
#define AXIOM_STATUS_WORD_NONFINITE 4u     /* non-finite activation met by the BF16 FP8 quantizer */

/* ---- raw-pointer, stream-explicit flavour ---- */

/* Replaces quantize_batch_to_tc[_warp]_kernel (src/axiom_qwen38_nvfp4_mlp.cu:144-223)
 * and, per row, axiom_qwen38_nvfp4_quantize_reference_f32. cols % 16 == 0. */
int axiom_qwen38_fused_nvfp4_quantize_bf16_device(int device, const void *input_bf16, uint32_t rows, uint32_t cols, float global_scale, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);

/* Replaces qwen38_add_bf16_inplace_kernel (src/axiom_qwen38_model.cu:175-184). */
int axiom_qwen38_fused_add_bf16_device(int device, const void *a_bf16, const void *b_bf16, void *out_bf16, uint64_t count, void *stream);

/* Replaces qwen38_add_bf16_rmsnorm8_kernel / qwen38_rmsnorm_bf16_8_kernel
 * (src/axiom_qwen38_model.cu:190-292) followed by the activation quantizer
 * (src/axiom_qwen38_nvfp4_mlp.cu:1347-1381) in one pass.
 *   hidden_bf16    optional addend; NULL = norm of `residual` alone
 *   residual_bf16  read; rewritten with bf16(residual + hidden) when hidden != NULL
 *   norm_out_bf16  optional BF16 copy of the normalised row
 *   out_codes/out_scales optional NVFP4 of the normalised row (both or neither)
 * cols % 16 == 0, cols <= 16384. */
int axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device(int device, const void *hidden_bf16, void *residual_bf16, const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);

/* The same with the addend taken straight from an FP8 GEMM: gemm_out_f32 [rows x cols] holds raw accumulators and the
 * addend is bf16((raw * weight_scale[feature]) * input_scale[token]) — fp8_group_row_scale_bf16_epilogue_kernel
 * (src/axiom_qwen38_fp8.cu:250-262) evaluated in this kernel's prologue, so the scaled tensor never exists in HBM.
 * weight_scale_bf16 [cols], input_scale [rows] (the per-token scales the activation quantizer produced). */
int axiom_qwen38_fused_fp8_epilogue_add_rmsnorm_nvfp4_device(int device, const float *gemm_out_f32, const void *weight_scale_bf16, const float *input_scale, void *residual_bf16, const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);

/* The same with a layer tap: tap_out_bf16 [rows x cols] receives a second copy of the updated residual rows
 * (qwen38_capture_tap8_kernel, src/axiom_qwen38_model.cu:343-351, folded into the write of the residual). */
int axiom_qwen38_fused_add_rmsnorm_nvfp4_tap_bf16_device(int device, const void *hidden_bf16, void *residual_bf16, const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *tap_out_bf16, void *stream);

/* The same with the addend gathered from an embedding table: residual[r] = bf16(residual[r] + table[token_ids[r]]),
 * then norm and quantize as above — qwen38_embedding_gather_columns_kernel (src/axiom_qwen38_model.cu:321-341) fused
 * into the first norm of the chain, so the gathered rows never make a round trip through HBM.  id >= vocab adds a
 * zero row and raises AXIOM_STATUS_WORD_BAD_ADDRESS. */
int axiom_qwen38_fused_gather_add_rmsnorm_nvfp4_bf16_device(int device, const void *table_bf16, uint32_t vocab, const uint32_t *token_ids, void *residual_bf16, const void *gamma_bf16, float eps, uint32_t rows, uint32_t cols, float global_scale, void *norm_out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, uint32_t *status_word, void *stream);

/* Replaces silu_mul_batch_kernel + quantize_columns_e4m3_kernel
 * (src/axiom_qwen38_fp8_mlp.cu:16-21,111-128; src/axiom_qwen38_fp8.cu:64-94).
 * gate_up rows are [gate(width) | up(width)]; scales[row] = rowmax/448 (1 if 0). width % 8 == 0. */
int axiom_qwen38_fused_swiglu_fp8_bf16_device(int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, uint8_t *out_codes, float *out_scales, void *stream);

/* Replaces silu_mul_quantize_batch_to_tc[_warp]_kernel
 * (src/axiom_qwen38_nvfp4_mlp.cu:229-317).  width % 16 == 0. */
int axiom_qwen38_fused_swiglu_nvfp4_bf16_device(int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, float global_scale, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);

/* Replaces qwen38_sigmoid_gate_kernel (src/axiom_qwen38_attention.cu:470-479) and the activation quantizer of
 * the output projection that follows it: y = bf16(attention * (1/(1+expf(-gate)))), optionally written to out_bf16,
 * and/or quantized to NVFP4 (both code outputs or neither).  attention, gate, out: [rows x width] BF16. width % 16 == 0. */
int axiom_qwen38_fused_sigmoid_gate_nvfp4_bf16_device(int device, const void *attention_bf16, const void *gate_bf16, uint32_t rows, uint32_t width, float global_scale, void *out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);
/* The same op with the gate read where the q projection left it, which makes the gate half of
 * qwen38_split_q_gate_round_k8_kernel (src/axiom_qwen38_attention.cu:431-453) unnecessary: q_gate_bf16 is
 * [rows][heads][2*head_dim], each head's head_dim query values followed by its head_dim gate values; attention, out and
 * the codes are [rows][heads*head_dim].  head_dim is 64, 128 or 256. */
int axiom_qwen38_fused_sigmoid_gate_heads_nvfp4_bf16_device(int device, const void *attention_bf16, const void *q_gate_bf16, uint32_t rows, uint32_t heads, uint32_t head_dim, float global_scale, void *out_bf16, uint8_t *out_codes, uint8_t *out_scales, uint32_t scale_layout, void *stream);

/* Greedy selection over rows of F32 logits.  Replaces qwen38_top1_8_kernel and the hierarchical pair
 * qwen38_top1_8_stage1/stage2_kernel with its `partials` scratch (src/axiom_qwen38_model.cu:408-600):
 * largest finite value, smallest id among equals, invalid = 1 if any logit of the row is not finite
 * (token_id = 0xffffffff when none is finite).  Layout of axiom_qwen38_model_dspark_device_top1_result
 * (include/axiom/qwen38_model.h:97-101).  logits: [rows x vocab], rows <= 65535. */
typedef struct {
    float value;
    uint32_t token_id;
    uint32_t invalid;
} axiom_top1_result;
int axiom_qwen38_fused_top1_f32_device(int device, const float *logits, uint32_t rows, uint32_t vocab, axiom_top1_result *results, void *stream);

/* The elementwise launches of ONE decoder layer, in the reference's order, as three calls that sit between the
 * layer's contractions (src/axiom_qwen38_model.cu:1357-1401; verify-block twin :1854-2000):
 *   post_mixer: residual += mixer_out; NVFP4(rmsnorm(residual) * post_norm_gamma) -> mlp_in_*      (:1371-1373 +
 *               src/axiom_qwen38_nvfp4_mlp.cu:1347-1381)
 *   mlp_mid:    NVFP4(silu(gate) * up) of gate_up -> mlp_mid_*                    (src/axiom_qwen38_nvfp4_mlp.cu:1531-1561)
 *   post_mlp:   residual += mlp_out; tap_out = residual (optional, qwen38_capture_tap8_kernel :343-351);
 *               next_norm_out = bf16(rmsnorm(residual) * next_norm_gamma): the next layer's input norm
 *               (src/axiom_qwen38_gdn.cu:177-220, src/axiom_qwen38_attention.cu:318-340) or the final norm (:1418)
 * Each call is one kernel, asynchronous on `stream` and capturable.  Members a call does not use may be NULL / 0. */
typedef struct {
    uint32_t abi_version;            /* AXIOM_ABI_VERSION */
    uint32_t struct_size;            /* sizeof(axiom_layer_glue) */
    uint32_t columns;                /* token columns; the reference's fixed batch is 8 */
    uint32_t hidden;                 /* 5120 */
    uint32_t ffn;                    /* 17408 */
    uint32_t scale_layout;           /* layout of both block-scale planes */
    float eps;
    float gate_up_input_scale;       /* NVFP4 global multiplier of the gate_up projection's input */
    float down_input_scale;          /* NVFP4 global multiplier of the down projection's input */
    uint32_t reserved0;              /* 0 */
    void *residual_bf16;             /* [columns][hidden] running hidden state, updated in place */
    const void *mixer_out_bf16;      /* [columns][hidden] attention / DeltaNet mixer output */
    const void *post_norm_gamma_bf16;/* [hidden] */
    uint8_t *mlp_in_codes;           /* [columns][hidden/2] */
    uint8_t *mlp_in_scales;
    const void *gate_up_bf16;        /* [columns][2*ffn], gate first */
    uint8_t *mlp_mid_codes;          /* [columns][ffn/2] */
    uint8_t *mlp_mid_scales;
    const void *mlp_out_bf16;        /* [columns][hidden] down projection output */
    void *tap_out_bf16;              /* optional [columns][hidden] */
    const void *next_norm_gamma_bf16;/* [hidden] */
    void *next_norm_out_bf16;        /* [columns][hidden] */
} axiom_layer_glue;
int axiom_qwen38_fused_layer_post_mixer_device(int device, const axiom_layer_glue *glue, void *stream);
int axiom_qwen38_fused_layer_mlp_mid_device(int device, const axiom_layer_glue *glue, void *stream);
int axiom_qwen38_fused_layer_post_mlp_device(int device, const axiom_layer_glue *glue, void *stream);

/* Replaces quantize_bf16_rows_e4m3_kernel (src/axiom_qwen38_mtp_compute.cu:239-278)
 * and, for BF16-valued input, quantize_columns_e4m3_kernel.  status_word
 * (optional, device) receives AXIOM_STATUS_WORD_NONFINITE via compare-and-swap. cols % 8 == 0. */
int axiom_qwen38_fused_fp8_quantize_bf16_device(int device, const void *input_bf16, uint32_t rows, uint32_t cols, uint8_t *out_codes, float *out_scales, uint32_t *status_word, void *stream);

/* Given-scale flavours of the two E4M3 quantizers: code = e4m3_satfinite(x / scale) with the scale an argument.
 * Replace quantize_columns_static_e4m3_kernel (src/axiom_qwen38_fp8.cu:96-107, the ModelOpt branch of
 * quantize_input, :830-840) for a BF16 tensor and for silu(gate)*up of a fused [gate | up] row.  One pass, no
 * per-token scale output.  scale finite and > 0; cols (width) % 8 == 0. */
int axiom_qwen38_fused_fp8_quantize_static_bf16_device(int device, const void *input_bf16, uint32_t rows, uint32_t cols, float scale, uint8_t *out_codes, void *stream);
int axiom_qwen38_fused_swiglu_fp8_static_bf16_device(int device, const void *gate_up_bf16, uint32_t rows, uint32_t width, float scale, uint8_t *out_codes, void *stream);

/* Replaces qwen38_embedding_gather_columns_kernel (src/axiom_qwen38_model.cu:321-341):
 * id >= vocab gives a zero row and AXIOM_STATUS_WORD_BAD_ADDRESS.  hidden % 8 == 0. */
int axiom_qwen38_fused_embedding_gather_bf16_device(int device, const void *table_bf16, uint32_t vocab, uint32_t hidden, const uint32_t *token_ids, uint32_t tokens, void *out_bf16, uint32_t *status_word, void *stream);

/* RoPE frequency table.  Replaces qwen38_yarn_inv_frequency
 * (src/axiom_qwen38_attention.cu:98-116), evaluated once on the device into
 * inv_freq[rope_dim/2] instead of per thread per call.  factor <= 1 gives
 * plain theta^(-2p/rope_dim). */
typedef struct {
    uint32_t abi_version;     /* AXIOM_ABI_VERSION */
    uint32_t rope_dim;        /* rotated dims, even, <= head_dim */
    float theta;
    float factor;
    float original_context;
    float beta_fast;
    float beta_slow;
} axiom_rope_config;
int axiom_qwen38_fused_yarn_inv_freq_device(int device, const axiom_rope_config *config, float *out_inv_freq, void *stream);
/* 0.1*ln(factor)+1 (include/axiom/qwen38_attention.h:29) */
float axiom_qwen38_fused_yarn_mscale(float factor);

/* Replaces qwen38_qk_norm_partial_rope_cache8_kernel and its temporal twin
 * (src/axiom_qwen38_attention.cu:481-554,1317-1392) + the paged scatter of
 * axiom_kv_pool_store_paged_f32_kernel (src/axiom_cuda.cu:16954-16969), BF16 cache.
 * Per (token, head): inv = (float)(1/sqrt(mean(x^2)+eps)) in FP64; n = (x*inv)*gamma;
 * NeoX pairs (p, p+rope_dim/2) rotated by angle=(float)pos*inv_freq[p] with
 * cos/sin each scaled by mscale; one BF16 rounding at the end.  Q is rewritten
 * in place.  Rotated K goes to k_pool at
 *   (((block*n_layers + layer)*block_tokens + pos%block_tokens)*pool_stride) + head*head_dim
 * with block = block_tables[row*tbl_stride + logical], logical = pos/block_tokens
 * (modulo tbl_stride when AXIOM_QK_FLAG_RING).  V (optional) is copied to v_pool.
 * k_out (optional) also receives rotated K contiguously. */
#define AXIOM_QK_FLAG_RING 1u            /* logical block index wraps modulo tbl_stride */
#define AXIOM_QK_FLAG_PER_TOKEN_TABLE 2u /* token t uses block-table row t (batched decode); else row 0 (one sequence) */
#define AXIOM_QK_FLAG_CACHE_E4M3 4u      /* k_pool / v_pool hold E4M3 codes at scale 1 (one byte per element) instead of
                                          * BF16: qwen38_kv_store_e4m3fn_scale1, src/axiom_qwen38_attention.cu:245-281 */
#define AXIOM_QK_FLAG_Q_GATE_INTERLEAVED 8u /* q_bf16 is the q_proj output [tokens][q_heads][2*head_dim], each head holding
                                          * its head_dim query values and then its head_dim gate values; only the query
                                          * halves are read and the result goes to q_out_bf16 (required).  Replaces the q part of
                                          * qwen38_split_q_gate_round_k8_kernel, src/axiom_qwen38_attention.cu:431-453; the gate
                                          * halves stay where they are for axiom_qwen38_fused_sigmoid_gate_heads_nvfp4_bf16_device */
#define AXIOM_QK_FLAG_ROUND_AFTER_NORM 16u /* the BF16 ("draft" / SGLang) rounding convention of qk_rmsnorm_rope_bf16_kernel +
                                          * round_f32_to_bf16_inplace_kernel (src/axiom_qwen38_dspark_compute.cu:250-300,
                                          * 210-213, layer sequence :1816-1825) instead of the target's: FP32 sum of squares in
                                          * the kernel's tree order, inv = rsqrtf(ss/head_dim + eps), n = bf16((x*inv)*gamma)
                                          * rounded BEFORE the rotation, then bf16(n1*c - n2*s), bf16(n1*s + n2*c).  Requires
                                          * rope_dim == head_dim.  cos/sin come from rope_table when it is set (the reference's
                                          * host-built table, :1459-1513), else from inv_freq and mscale as usual */
typedef struct {
    uint32_t abi_version;     /* AXIOM_ABI_VERSION */
    uint32_t struct_size;     /* sizeof(axiom_qk_rope_args); the sizes up to and excluding q_out_bf16, and up to and
                               * excluding rope_table, are accepted too (the missing members read as NULL / 0) */
    uint32_t tokens;
    uint32_t q_heads;
    uint32_t k_heads;
    uint32_t head_dim;        /* 64, 128 or 256 */
    uint32_t rope_dim;        /* even, <= head_dim, multiple of 16 */
    uint32_t flags;
    float eps;
    float mscale;
    uint32_t block_tokens;
    uint32_t n_layers;
    uint32_t layer;
    uint32_t pool_stride;     /* elements; >= k_heads*head_dim; multiple of 8 */
    uint32_t tbl_stride;
    uint32_t n_blocks;        /* physical blocks in the pool */
    void *q_bf16;             /* [tokens][q_heads][head_dim], in place; may be NULL when q_heads == 0 */
    const void *k_bf16;       /* [tokens][k_heads][head_dim] */
    const void *v_bf16;       /* optional [tokens][k_heads][head_dim] */
    const void *q_gamma_bf16; /* [head_dim] */
    const void *k_gamma_bf16; /* [head_dim] */
    const float *inv_freq;    /* [rope_dim/2] */
    const uint32_t *positions;/* [tokens] */
    const int32_t *block_tables;
    void *k_pool_bf16;        /* optional; NULL = no cache write.  BF16, or E4M3 bytes with AXIOM_QK_FLAG_CACHE_E4M3 */
    void *v_pool_bf16;        /* optional */
    void *k_out_bf16;         /* optional */
    uint32_t *status_word;    /* optional */
    void *q_out_bf16;         /* optional [tokens][q_heads][head_dim]: when set, q_bf16 is only read and the result goes here */
    const float *rope_table;  /* optional, AXIOM_QK_FLAG_ROUND_AFTER_NORM only: FP32 [rope_table_positions][head_dim], row p =
                               * cos(angle_p,0..head_dim/2-1) * mscale | sin(..) * mscale.  A token whose position is outside
                               * the table is left untouched and raises AXIOM_STATUS_WORD_BAD_ADDRESS */
    uint32_t rope_table_positions;
    uint32_t reserved0;       /* 0 */
} axiom_qk_rope_args;
int axiom_qwen38_fused_qk_norm_rope_paged_bf16_device(int device, const axiom_qk_rope_args *args, void *stream);

/* ---- axiom_device_buffer flavour (span-checked, default stream, finish-after-launch) ---- */
int axiom_runtime_nvfp4_quantize_bf16_device(axiom_runtime *runtime, const axiom_device_buffer *input, uint64_t input_offset, uint32_t rows, uint32_t cols, float global_scale, axiom_device_buffer *out_codes, uint64_t codes_offset, axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout);
int axiom_runtime_add_rmsnorm_nvfp4_bf16_device(axiom_runtime *runtime, const axiom_device_buffer *hidden, uint64_t hidden_offset, axiom_device_buffer *residual, uint64_t residual_offset, const axiom_device_buffer *gamma, uint64_t gamma_offset, float eps, uint32_t rows, uint32_t cols, float global_scale, axiom_device_buffer *norm_out, uint64_t norm_offset, axiom_device_buffer *out_codes, uint64_t codes_offset, axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout);
int axiom_runtime_swiglu_fp8_bf16_device(axiom_runtime *runtime, const axiom_device_buffer *gate_up, uint64_t gate_up_offset, uint32_t rows, uint32_t width, axiom_device_buffer *out_codes, uint64_t codes_offset, axiom_device_buffer *out_scales, uint64_t scales_offset);
int axiom_runtime_swiglu_nvfp4_bf16_device(axiom_runtime *runtime, const axiom_device_buffer *gate_up, uint64_t gate_up_offset, uint32_t rows, uint32_t width, float global_scale, axiom_device_buffer *out_codes, uint64_t codes_offset, axiom_device_buffer *out_scales, uint64_t scales_offset, uint32_t scale_layout);
int axiom_runtime_embedding_gather_bf16_device(axiom_runtime *runtime, const axiom_device_buffer *table, uint64_t table_offset, uint32_t vocab, uint32_t hidden, const axiom_device_buffer *token_ids, uint64_t ids_offset, uint32_t tokens, axiom_device_buffer *out, uint64_t out_offset);

/* The q/k call as a step-engine family provider makes it (forward_step / prefill_token hooks,
 * include/axiom/axiom_engine.h:218-245): the paged-KV addressing comes from the engine's device view.  The view
 * mirrors axiom_engine_dev (include/axiom/axiom_engine.h:183-198) plus the pool geometry of the arena
 * (axiom_engine_kv_arena, :164-181; element offset (((pb*n_layers+L)*BT+slot)*kv_dim), :282-283); the pools hold BF16
 * (E4M3 bytes with AXIOM_QK_FLAG_CACHE_E4M3) instead of F32.  Active sequence a (0 <= a < n_active <= cap, at most
 * 65535 like axiom_runtime_kv_pool_store_paged_f32_device, src/axiom_cuda.cu:16982-16987) uses block-table row a and the
 * position at d_meta byte offset cap*4 + a*4; a position beyond its row's tbl_stride blocks or a block id outside
 * [0, kv_nphys) raises the status word and writes nothing.  q, k, v: [n_active][heads][head_dim] BF16 staging rows.
 * flags: 0 or AXIOM_QK_FLAG_CACHE_E4M3.  Every span is checked against its buffer before the launch. */
typedef struct {
    uint32_t abi_version;     /* AXIOM_ABI_VERSION */
    uint32_t struct_size;     /* sizeof(axiom_paged_kv_view) */
    axiom_device_buffer *d_kpool;       /* kv_nphys * n_layers * block_tokens * kv_dim cache elements */
    axiom_device_buffer *d_vpool;       /* same geometry; may be NULL together with v */
    const axiom_device_buffer *d_tbl;   /* [cap][tbl_stride] int32 */
    const axiom_device_buffer *d_meta;  /* [2*cap] u32: cache_tokens at byte 0, positions at byte cap*4 */
    uint32_t cap;
    uint32_t tbl_stride;
    uint32_t block_tokens;    /* kv_bt (AXIOM_KV_BLOCK, default 16) */
    uint32_t n_layers;
    uint32_t kv_nphys;
    uint32_t kv_dim;          /* elements per pool row; >= k_heads*head_dim, multiple of 8 */
} axiom_paged_kv_view;
int axiom_runtime_qknorm_rope_yarn_paged_bf16_device(axiom_runtime *runtime, const axiom_paged_kv_view *view, uint32_t layer, uint32_t n_active, uint32_t flags, axiom_device_buffer *q, uint64_t q_offset, const axiom_device_buffer *k, uint64_t k_offset, const axiom_device_buffer *v, uint64_t v_offset, const axiom_device_buffer *q_gamma, uint64_t q_gamma_offset, const axiom_device_buffer *k_gamma, uint64_t k_gamma_offset, const axiom_device_buffer *inv_freq, uint64_t inv_freq_offset, uint32_t q_heads, uint32_t k_heads, uint32_t head_dim, uint32_t rope_dim, float eps, float mscale, axiom_device_buffer *status_word, uint64_t status_offset);

/* ---- host I/O flavour: pinned or pageable host pointers in, host pointers out.
 * Rows are streamed through runtime-owned staging buffers in chunks so the
 * upload of chunk i+1, the kernel on chunk i and the download of chunk i-1
 * overlap; the call returns after the last download has completed. ---- */
int axiom_runtime_nvfp4_quantize_bf16(axiom_runtime *runtime, const void *input_bf16_host, uint32_t rows, uint32_t cols, float global_scale, uint8_t *out_codes_host, uint8_t *out_scales_host);
int axiom_runtime_add_rmsnorm_nvfp4_bf16(axiom_runtime *runtime, const void *hidden_bf16_host, void *residual_bf16_host, const void *gamma_bf16_host, float eps, uint32_t rows, uint32_t cols, float global_scale, uint8_t *out_codes_host, uint8_t *out_scales_host);
int axiom_runtime_swiglu_fp8_bf16(axiom_runtime *runtime, const void *gate_up_bf16_host, uint32_t rows, uint32_t width, uint8_t *out_codes_host, float *out_scales_host);

/* ====================================================================== */
/* Part 3 — helpers                                                        */
/* ====================================================================== */

/* scale_view_bytes / scale_view_offset (src/axiom_qwen38_nvfp4_mlp.cu:95-108) */
uint64_t axiom_nvfp4_scale_plane_bytes(uint32_t rows, uint32_t groups, uint32_t scale_layout);
uint64_t axiom_nvfp4_scale_plane_offset(uint32_t row, uint32_t group, uint32_t groups, uint32_t scale_layout);

/* Host-I/O NVFP4 quantize that performs no allocation of any kind.  NO COUNTERPART IN THE
 * REFERENCE: it exists for callers that must not allocate while they run.  Same results as
 * axiom_runtime_nvfp4_quantize_bf16 (which stages through buffers the runtime allocates on
 * demand); here the staging of input, codes and scales is a fixed device array inside the
 * library image, of axiom_b200_static_scratch_bytes() bytes (8 MiB) per device.
 *   - A call whose input + codes + scale plane (each rounded up to 256 bytes) exceed that
 *     size returns AXIOM_ERR_BUDGET and touches nothing.
 *   - The first call on a device looks the array's address up.  With CUDA's lazy module
 *     loading that is when the driver loads the module that holds the array and reserves its
 *     8 MiB on that device; it may synchronise the device and it fails (AXIOM_ERR_CUDA) on a
 *     device with no room left.  Make that first call at start-up, before the memory budget
 *     is frozen and before any stream capture begins; later calls reserve nothing.  The call
 *     itself ends with a synchronisation of `stream` and therefore cannot be captured.
 *   - Whenever the call returns, with success or with an error, nothing it enqueued is still
 *     running: the host buffers and the shared array are idle.
 *   - Every call on a device uses the same array: calls that overlap in time (other host
 *     threads, other streams) corrupt each other.  Serialise them.
 *   - out_scales_host receives axiom_nvfp4_scale_plane_bytes(rows, cols/16, scale_layout) bytes. */
uint64_t axiom_b200_static_scratch_bytes(void);
int axiom_b200_nvfp4_quantize_bf16_host_static(int device, const void *input_bf16_host, uint32_t rows, uint32_t cols, float global_scale, uint32_t scale_layout, uint8_t *out_codes_host, uint8_t *out_scales_host, void *stream);

/* Optional one-time set-up of `device`.  The stream-explicit entries set a few things up lazily on their first
 * use: the two gate tables of the SwiGLU / sigmoid-gate kernels (one small fill kernel each AND a synchronisation of
 * the caller's stream, skipped while that stream is capturing), the dynamic shared-memory limits of the pipelined
 * kernels, and the driver's tensor-map encoder.  This call does all of that at once and synchronises the device;
 * after it has returned AXIOM_OK, no stream-explicit entry on that device launches anything but its own kernel or
 * synchronises anything, whichever comes first — so a first call may sit inside a stream capture.  Call it once
 * per device at start-up (the reference's objects do the equivalent in their create functions,
 * include/axiom/qwen38_nvfp4_mlp.h:111-117: "allocation-free and asynchronous" forward calls). */
int axiom_b200_prepare(int device);

/* Number of kernel launches issued by this library in this process (bench bookkeeping). */
uint64_t axiom_b200_kernel_launch_count(void);

/* The pipelined kernels wait on shared-memory barriers with a bounded number of
 * polls; a wait that runs out raises a device word instead of hanging.  This
 * synchronises `device`, returns the OR of those words (0 = no fault) and
 * clears them. */
uint32_t axiom_b200_pipeline_faults(int device);

/* TEST HOOK, not for production use.  Arms the NEXT launch of the streaming add + RMSNorm kernel (296 rows and
 * more) so that the first row of its first team announces `extra_bytes` more than its copies deliver: that team's
 * barrier never completes, its bounded wait gives up after `spin_limit` polls (0 = the default 2^18), the team
 * writes none of its rows and the kernel returns normally with axiom_b200_pipeline_faults() != 0.  Nothing
 * faults, traps or hangs; every other team's rows are complete.  extra_bytes % 16 == 0. */
int axiom_b200_test_arm_wait_timeout(uint32_t extra_bytes, uint32_t spin_limit);

#ifdef __cplusplus
}
#endif

#endif

/* Step-engine family provider for the fused elementwise path.
 *
 * The reference's step engine (include/axiom/axiom_engine.h) drives a model family through a vtable,
 * axiom_engine_family_ops (:207-274).  Its forward_step hook (:218-225) runs ONE lockstep batched decode forward
 * over the active sequences: embed each sequence's next_tok, run the layers with per-sequence cache length pos + 1
 * addressing the paged KV arena through the engine's device view (axiom_engine_dev, :183-198), and write every
 * sequence's logits into seq->seq_logits.
 *
 * This header declares a provider whose forward_step does exactly that with every elementwise stage taken from
 * libaxiom_b200 — embedding gather, input norm, q/k norm + RoPE + paged-KV write at each sequence's own position,
 * residual add + post norm + NVFP4 quantize, SwiGLU + NVFP4 quantize, residual add + next norm — and every
 * contraction (q/k/v and output projections, the attention core, the two MLP projections, the LM head: the
 * reference's cuBLASLt / attention-kernel calls) left to hooks the integrator supplies.  Nothing of the engine's
 * control plane (admission, sampling, block allocation, prefix cache) is here.
 *
 * The two engine structs the hook receives are mirrored below, member for member, so the provider can be handed to
 * the engine as it is; when the reference's own header has been included first, its declarations are used. */
#ifndef AXIOM_B200_ENGINE_H
#define AXIOM_B200_ENGINE_H

#include "axiom_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef AXIOM_ENGINE_H
/* include/axiom/axiom_engine.h:53-54 */
typedef void (*axiom_engine_on_piece)(void *ctx, int seq, const char *piece, int len);

/* include/axiom/axiom_engine.h:114-153.  The provider reads next_tok and pos and writes seq_logits. */
typedef struct axiom_engine_seq {
    uint64_t sid;
    uint32_t *ids;
    int ids_cap;
    int n_in;
    int n_out;
    int pos;             /* current cache length: the token of this step sits at position pos */
    int generated;
    int max_new;
    int out_cap;
    uint64_t rng;
    float *seq_logits;   /* vocab f32, host */
    int *block_table;
    int n_blocks;
    int blocks_cap;
    uint32_t maxseq;
    int done;
    int use_eos;
    uint32_t next_tok;   /* token to embed this step */
    uint32_t device_greedy_tok;
    int device_greedy_tok_valid;
    int device_greedy_tok_resident;
    int device_greedy_tok_pending;
    int (*device_greedy_tok_materialize)(void *ctx, struct axiom_engine_seq *seq);
    void *device_greedy_tok_materialize_ctx;
    int next_tok_device_resident;
    float temp; int top_k; float top_p; unsigned int seed;
    void *piece_ctx;
    axiom_engine_on_piece on_piece;
    int piece_seq;
    int stream_after_reset;
} axiom_engine_seq;

/* include/axiom/axiom_engine.h:183-198 */
typedef struct axiom_engine_dev {
    axiom_runtime *rt;
    axiom_device_buffer *d_kpool, *d_vpool;   /* arena pools (borrowed); BF16 here, F32 in the reference */
    axiom_device_buffer *d_tbl;    /* [cap][tbl_stride] int32 block-table matrix */
    axiom_device_buffer *d_meta;   /* [2*cap] u32: cache_tokens at 0, pos at byte cap*4 */
    int cap;
    uint32_t tbl_stride;
    int32_t *htbl;
    uint32_t *hmeta;
} axiom_engine_dev;
#endif /* AXIOM_ENGINE_H */

/* Where the reference calls a library contraction.  Every hook is asynchronous on `stream`, reads and writes device
 * memory only, handles `n` active rows, and returns 0 on success (anything else aborts the step with that value).
 * All activations are BF16 row-major; the NVFP4 operands are packed E2M1 codes with block scales in the cuBLASLt
 * VEC16_UE4M3 tile layout (what the reference's FP4 GEMM descriptors expect, src/axiom_qwen38_nvfp4_mlp.cu:1153-1167). */
typedef struct {
    void *user;
    /* q [n][q_heads*head_dim], k and v [n][k_heads*head_dim] from the layer's input norm [n][hidden] */
    int (*qkv_projection)(void *user, uint32_t layer, uint32_t n, const void *norm_bf16, void *q_bf16, void *k_bf16, void *v_bf16, void *stream);
    /* attention over the paged cache (K and V of this step are already in the pools) followed by the output
     * projection: mixer_out [n][hidden].  `dev` is the engine's view, exactly as forward_step received it. */
    int (*attention_output)(void *user, uint32_t layer, uint32_t n, const void *q_bf16, const axiom_engine_dev *dev, void *mixer_out_bf16, void *stream);
    /* gate_up [n][2*ffn] from the NVFP4 image of the post norm */
    int (*gate_up_projection)(void *user, uint32_t layer, uint32_t n, const uint8_t *codes, const uint8_t *scales_tiled, void *gate_up_bf16, void *stream);
    /* mlp_out [n][hidden] from the NVFP4 image of silu(gate)*up */
    int (*down_projection)(void *user, uint32_t layer, uint32_t n, const uint8_t *codes, const uint8_t *scales_tiled, void *mlp_out_bf16, void *stream);
    /* logits F32 [n][vocab] from the final norm [n][hidden] */
    int (*lm_head)(void *user, uint32_t n, const void *final_norm_bf16, float *logits_f32, void *stream);
} axiom_b200_contraction_hooks;

typedef struct {
    uint32_t abi_version;      /* AXIOM_ABI_VERSION */
    uint32_t struct_size;      /* sizeof(axiom_b200_step_provider_config) */
    uint32_t n_layers, hidden, ffn, q_heads, k_heads, head_dim, rope_dim, vocab;
    uint32_t max_batch;        /* most active sequences a step may carry */
    uint32_t kv_block_tokens;  /* the arena's block size (AXIOM_KV_BLOCK, default 16) */
    uint32_t kv_nphys;         /* physical blocks in the arena pools */
    uint32_t kv_dim;           /* elements per pool row, >= k_heads*head_dim */
    float eps, mscale;
    float gate_up_input_scale, down_input_scale;   /* NVFP4 global multipliers of the two MLP projections' inputs */
    /* model tensors, device memory that outlives the provider (BF16 unless noted) */
    const void *embedding;          /* [vocab][hidden] */
    const void *input_norm_gamma;   /* [n_layers][hidden] */
    const void *post_norm_gamma;    /* [n_layers][hidden] */
    const void *final_norm_gamma;   /* [hidden] */
    const void *q_norm_gamma;       /* [n_layers][head_dim] */
    const void *k_norm_gamma;       /* [n_layers][head_dim] */
    const float *inv_freq;          /* F32 [rope_dim/2] */
    axiom_b200_contraction_hooks hooks;
} axiom_b200_step_provider_config;

typedef struct axiom_b200_step_provider axiom_b200_step_provider;

/* Allocates the provider's per-step scratch (max_batch rows of every intermediate) on the runtime's device and one
 * stream.  AXIOM_ERR_BUDGET when the device is out of memory. */
int axiom_b200_step_provider_create(axiom_runtime *runtime, const axiom_b200_step_provider_config *config, axiom_b200_step_provider **out_provider);
void axiom_b200_step_provider_destroy(axiom_b200_step_provider *provider);

/* axiom_engine_family_ops::forward_step (include/axiom/axiom_engine.h:218-225) with fam = the provider.  Returns 0,
 * a hook's non-zero value, or an axiom_status; a sequence whose position addresses a block outside its table or
 * the pool gives AXIOM_ERR_RUNTIME after the step has completed for the others (its KV write was skipped). */
int axiom_b200_step_provider_forward_step(void *fam, axiom_engine_seq *const *active, int n_active, const axiom_engine_dev *dev);

/* Device address of one of the provider's scratch tensors after a step (for integration tests of hook code):
 * 0 residual, 1 norm, 2 q, 3 k, 4 v, 5 mixer_out, 6 mlp_in_codes, 7 mlp_in_scales, 8 gate_up, 9 mlp_mid_codes,
 * 10 mlp_mid_scales, 11 mlp_out, 12 logits.  NULL for any other index. */
void *axiom_b200_step_provider_scratch(axiom_b200_step_provider *provider, uint32_t which);

#ifdef __cplusplus
}
#endif

#endif

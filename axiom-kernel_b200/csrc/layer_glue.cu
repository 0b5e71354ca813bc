// The elementwise launches of ONE decoder layer in the reference's order, as three calls that sit between the
// layer's contractions (which stay the caller's: cuBLASLt in the reference).  Replaces, per layer of
// qwen38_model_forward_batch8_internal (src/axiom_qwen38_model.cu:1357-1401) and of the verify-block twin
// (:1854-2000):
//
//   post_mixer : qwen38_add_bf16_rmsnorm8_kernel (:1371-1373)  +  the NVFP4 activation quantizer that opens the MLP
//                (quantize_batch_to_tc_warp_kernel via projection_run, src/axiom_qwen38_nvfp4_mlp.cu:1347-1381)
//   mlp_mid    : silu_mul_quantize_batch_to_tc_warp_kernel (src/axiom_qwen38_nvfp4_mlp.cu:1531-1561)
//   post_mlp   : qwen38_add_bf16_inplace_kernel (:1378-1379)  +  tap capture (qwen38_capture_tap8_kernel, :343-351)
//                +  the RMSNorm that reads the updated residual next: the next layer's input norm
//                (qwen38_rmsnorm8_kernel, src/axiom_qwen38_gdn.cu:177-220; qwen38_attention_rmsnorm8_kernel,
//                src/axiom_qwen38_attention.cu:318-340) or the final norm (qwen38_rmsnorm_bf16_8_kernel, :1418)
//
// Eight reference launches per layer become three; each is one kernel of this library, stream-explicit and
// capturable, so a whole layer (or model) of them replays from one CUDA graph.  Any column count is accepted; the
// reference's fixed batch is 8.
#include "runtime.hpp"

using namespace axb;

namespace {

bool glue_header_ok(const axiom_layer_glue *g) {
    return g && g->abi_version == AXIOM_ABI_VERSION && g->struct_size == sizeof(axiom_layer_glue) && g->columns != 0u &&
           g->hidden != 0u && (g->hidden % kGroup) == 0u && g->hidden <= 16384u && g->eps > 0.0f && std::isfinite(g->eps) &&
           g->scale_layout <= AXIOM_SCALE_LAYOUT_TILED && g->residual_bf16 && aligned16(g->residual_bf16);
}

}  // namespace

extern "C" int axiom_qwen38_fused_layer_post_mixer_device(int device, const axiom_layer_glue *g, void *stream) {
    if (!glue_header_ok(g) || !g->mixer_out_bf16 || !aligned16(g->mixer_out_bf16) || !g->post_norm_gamma_bf16 ||
        !aligned16(g->post_norm_gamma_bf16) || !g->mlp_in_codes || !g->mlp_in_scales || !valid_scale(g->gate_up_input_scale) ||
        (reinterpret_cast<uintptr_t>(g->mlp_in_codes) & 3u)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_rmsnorm_nvfp4_bf16(g->mixer_out_bf16, g->residual_bf16, g->post_norm_gamma_bf16, g->eps, g->columns, g->hidden,
                                  g->gate_up_input_scale, nullptr, g->mlp_in_codes, g->mlp_in_scales, g->scale_layout,
                                  (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_layer_mlp_mid_device(int device, const axiom_layer_glue *g, void *stream) {
    if (!glue_header_ok(g) || g->ffn == 0u || (g->ffn % kGroup) != 0u || !g->gate_up_bf16 || !aligned16(g->gate_up_bf16) ||
        !g->mlp_mid_codes || !g->mlp_mid_scales || !valid_scale(g->down_input_scale) ||
        (reinterpret_cast<uintptr_t>(g->mlp_mid_codes) & 3u) || (uint64_t)g->columns * (g->ffn / 8u) > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_swiglu_nvfp4_bf16(g->gate_up_bf16, g->columns, g->ffn, g->down_input_scale, g->mlp_mid_codes, g->mlp_mid_scales,
                             g->scale_layout, (cudaStream_t)stream);
    return launch_status();
}

extern "C" int axiom_qwen38_fused_layer_post_mlp_device(int device, const axiom_layer_glue *g, void *stream) {
    if (!glue_header_ok(g) || !g->mlp_out_bf16 || !aligned16(g->mlp_out_bf16) || !g->next_norm_gamma_bf16 ||
        !aligned16(g->next_norm_gamma_bf16) || !g->next_norm_out_bf16 || !aligned16(g->next_norm_out_bf16) ||
        (g->tap_out_bf16 && (!aligned16(g->tap_out_bf16) || g->tap_out_bf16 == g->residual_bf16))) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    launch_add_rmsnorm_tap_nvfp4_bf16(g->mlp_out_bf16, g->residual_bf16, g->next_norm_gamma_bf16, g->eps, g->columns, g->hidden, 1.0f,
                                      g->next_norm_out_bf16, nullptr, nullptr, AXIOM_SCALE_LAYOUT_CANONICAL, g->tap_out_bf16,
                                      (cudaStream_t)stream);
    return launch_status();
}

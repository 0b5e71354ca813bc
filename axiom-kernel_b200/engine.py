"""ctypes mirror of include/axiom_b200_engine.h: the step-engine structs the forward_step hook receives
(axiom_engine_seq, axiom_engine_dev: reference include/axiom/axiom_engine.h:114-153,183-198), the contraction hooks
and the provider configuration.  Used by the tests, which play the engine's part."""
from __future__ import annotations

import ctypes as C

vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int


class EngineSeq(C.Structure):
    _fields_ = [
        ("sid", u64), ("ids", C.POINTER(u32)), ("ids_cap", i32), ("n_in", i32), ("n_out", i32), ("pos", i32),
        ("generated", i32), ("max_new", i32), ("out_cap", i32), ("rng", u64), ("seq_logits", C.POINTER(f32)),
        ("block_table", C.POINTER(i32)), ("n_blocks", i32), ("blocks_cap", i32), ("maxseq", u32), ("done", i32),
        ("use_eos", i32), ("next_tok", u32), ("device_greedy_tok", u32), ("device_greedy_tok_valid", i32),
        ("device_greedy_tok_resident", i32), ("device_greedy_tok_pending", i32), ("device_greedy_tok_materialize", vp),
        ("device_greedy_tok_materialize_ctx", vp), ("next_tok_device_resident", i32), ("temp", f32), ("top_k", i32),
        ("top_p", f32), ("seed", C.c_uint), ("piece_ctx", vp), ("on_piece", vp), ("piece_seq", i32),
        ("stream_after_reset", i32),
    ]


class EngineDev(C.Structure):
    _fields_ = [("rt", vp), ("d_kpool", vp), ("d_vpool", vp), ("d_tbl", vp), ("d_meta", vp), ("cap", i32),
                ("tbl_stride", u32), ("htbl", C.POINTER(C.c_int32)), ("hmeta", C.POINTER(u32))]


QKV_HOOK = C.CFUNCTYPE(i32, vp, u32, u32, vp, vp, vp, vp, vp)
ATTENTION_HOOK = C.CFUNCTYPE(i32, vp, u32, u32, vp, C.POINTER(EngineDev), vp, vp)
NVFP4_GEMM_HOOK = C.CFUNCTYPE(i32, vp, u32, u32, vp, vp, vp, vp)
LM_HEAD_HOOK = C.CFUNCTYPE(i32, vp, u32, vp, vp, vp)


class ContractionHooks(C.Structure):
    _fields_ = [("user", vp), ("qkv_projection", QKV_HOOK), ("attention_output", ATTENTION_HOOK),
                ("gate_up_projection", NVFP4_GEMM_HOOK), ("down_projection", NVFP4_GEMM_HOOK), ("lm_head", LM_HEAD_HOOK)]


class StepProviderConfig(C.Structure):
    _fields_ = [
        ("abi_version", u32), ("struct_size", u32), ("n_layers", u32), ("hidden", u32), ("ffn", u32), ("q_heads", u32),
        ("k_heads", u32), ("head_dim", u32), ("rope_dim", u32), ("vocab", u32), ("max_batch", u32), ("kv_block_tokens", u32),
        ("kv_nphys", u32), ("kv_dim", u32), ("eps", f32), ("mscale", f32), ("gate_up_input_scale", f32),
        ("down_input_scale", f32), ("embedding", vp), ("input_norm_gamma", vp), ("post_norm_gamma", vp),
        ("final_norm_gamma", vp), ("q_norm_gamma", vp), ("k_norm_gamma", vp), ("inv_freq", vp), ("hooks", ContractionHooks),
    ]


SCRATCH = {"residual": 0, "norm": 1, "q": 2, "k": 3, "v": 4, "mixer_out": 5, "mlp_in_codes": 6, "mlp_in_scales": 7,
           "gate_up": 8, "mlp_mid_codes": 9, "mlp_mid_scales": 10, "mlp_out": 11, "logits": 12}

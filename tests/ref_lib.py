"""ctypes front-end of oracle/_ref/libaxiom_ref.so: the reference's own kernels compiled for
sm_100a (built by oracle/build_ref.py where the reference tree is present).  Test infrastructure.
All pointers are device addresses (ints); every call synchronises before it returns."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libaxiom_ref.so"
vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int

SIGNATURES = {
    "ref_quantize_batch_to_tc": [vp, f32, vp, vp, u32, u32, i32],
    "ref_silu_mul_quantize_batch_to_tc": [vp, f32, vp, vp, u32, u32, i32],
    "ref_silu_mul_batch": [vp, vp, vp, u32],
    "ref_quantize_columns_e4m3": [vp, vp, vp, u32, u32],
    "ref_quantize_columns_static_e4m3": [vp, vp, f32, u32, u32],
    "ref_quantize_bf16_rows_e4m3": [vp, vp, vp, u32, u32, vp],
    "ref_add_bf16_inplace": [vp, vp, u64],
    "ref_add_bf16_rmsnorm8": [vp, vp, vp, vp, u32],
    "ref_rmsnorm_bf16_8": [vp, vp, vp, u32],
    "ref_embedding_gather_columns": [vp, vp, vp, u32],
    "ref_yarn_inv_frequency": [vp],
    "ref_qk_norm_partial_rope_cache_temporal8": [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, i32],
    "ref_qk_norm_partial_rope_cache8": [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, i32],
    "ref_sigmoid_gate8": [vp, vp, vp],
    "ref_attention_rmsnorm8": [vp, vp, vp],
    "ref_capture_tap8": [vp, vp, u32],
    "ref_dspark_qk_norm_rope_round": [vp, vp, vp, u32, u32, u32, u32],
    "ref_fp8_group_row_scale_bf16_epilogue": [vp, vp, vp, u32],
    "ref_top1_8": [vp, vp, vp, i32],
    "ref_q8_0_embedding_gather_f32": [vp, vp, u32, u32, u32],
    "ref_q8_0_embedding_gather_token_f32": [vp, vp, vp, u32, u32],
    "ref_f16_embedding_streams": [vp, vp, u32, u32, u32],
    "ref_rmsnorm_f32": [vp, vp, vp, u32, f32, i32],
    "ref_rmsnorm_f32_dual": [vp, vp, vp, vp, vp, u32, f32],
    "ref_head_rmsnorm_f32": [vp, u32, u32, f32],
    "ref_qk_rmsnorm_w_f32": [vp, vp, u32, u32, f32],
    "ref_add_f32": [vp, vp, vp, u32],
    "ref_silu_mul_f32": [vp, vp, vp, u32, f32],
    "ref_kv_pool_store_paged_f32": [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32],
    "axiom_qwen38_nvfp4_quantize_reference_f32": [i32, vp, f32, vp, vp, u32, vp],
    "axiom_rope_neox_precise_launch": [i32, vp, u32, u32, u32, f32],
    "axiom_rope_neox_partial_precise_launch": [i32, vp, u32, u32, u32, u32, f32],
    "axiom_qknorm_rope_precise_launch": [i32, vp, vp, u32, u32, u32, f32, f32],
    "axiom_qknorm_rope_pos_precise_launch": [i32, vp, vp, vp, u32, u32, f32, f32],
    "axiom_qknorm_rope_pos_dual_precise_launch": [i32, vp, vp, vp, vp, vp, u32, u32, u32, f32, f32],
}

_lib = None


def available() -> bool:
    return PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        handle = C.CDLL(str(PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = i32
            fn.argtypes = argtypes
        handle.ref_model_hidden.restype = u32
        handle.ref_model_vocab.restype = u32
        _lib = handle
    return _lib

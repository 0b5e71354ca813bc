"""ctypes binding of libaxiom_b200.so (the C ABI declared in include/axiom_b200.h).

The library is the product; this module only loads it and gives the tests and
the benchmark typed access to its entry points.  There is no fallback: if the
shared object has not been built (``python axiom-kernel_b200/build.py``) loading
raises, and every wrapper below goes through the C ABI.

PyTorch is used by callers for device memory and streams only; the wrappers
take raw addresses (``tensor.data_ptr()``) and sizes.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libaxiom_b200.so"

AXIOM_ABI_VERSION = 1
AXIOM_OK = 0
AXIOM_ERR_INVALID_ARGUMENT = 1
AXIOM_ERR_UNSUPPORTED_BACKEND = 2
AXIOM_ERR_CUDA = 3
AXIOM_ERR_RUNTIME = 4
AXIOM_ERR_NOT_IMPLEMENTED = 5
AXIOM_ERR_IO = 6
AXIOM_ERR_BUDGET = 7
AXIOM_BACKEND_CUDA = 1
AXIOM_BACKEND_CLUSTER = 2

SCALE_CANONICAL = 0
SCALE_TILED = 1
QK_FLAG_RING = 1
QK_FLAG_PER_TOKEN_TABLE = 2
QK_FLAG_CACHE_E4M3 = 4
QK_FLAG_Q_GATE_INTERLEAVED = 8
QK_FLAG_ROUND_AFTER_NORM = 16
STATUS_WORD_OK = 0
STATUS_WORD_BAD_ADDRESS = 1
STATUS_WORD_NONFINITE = 4

u8p = C.POINTER(C.c_uint8)
vp = C.c_void_p
u32 = C.c_uint32
u64 = C.c_uint64
f32 = C.c_float
i32 = C.c_int


class AxiomConfig(C.Structure):
    _fields_ = [("abi_version", u32), ("backend", C.c_int), ("device", u32), ("flags", u64)]


class RopeConfig(C.Structure):
    _fields_ = [("abi_version", u32), ("rope_dim", u32), ("theta", f32), ("factor", f32),
                ("original_context", f32), ("beta_fast", f32), ("beta_slow", f32)]


class PagedKvView(C.Structure):
    """axiom_paged_kv_view: the engine's device view of the paged KV arena."""
    _fields_ = [
        ("abi_version", u32), ("struct_size", u32), ("d_kpool", vp), ("d_vpool", vp), ("d_tbl", vp), ("d_meta", vp),
        ("cap", u32), ("tbl_stride", u32), ("block_tokens", u32), ("n_layers", u32), ("kv_nphys", u32), ("kv_dim", u32),
    ]


class QkRopeArgs(C.Structure):
    _fields_ = [
        ("abi_version", u32), ("struct_size", u32), ("tokens", u32), ("q_heads", u32), ("k_heads", u32),
        ("head_dim", u32), ("rope_dim", u32), ("flags", u32), ("eps", f32), ("mscale", f32),
        ("block_tokens", u32), ("n_layers", u32), ("layer", u32), ("pool_stride", u32), ("tbl_stride", u32),
        ("n_blocks", u32),
        ("q_bf16", vp), ("k_bf16", vp), ("v_bf16", vp), ("q_gamma_bf16", vp), ("k_gamma_bf16", vp),
        ("inv_freq", vp), ("positions", vp), ("block_tables", vp), ("k_pool_bf16", vp), ("v_pool_bf16", vp),
        ("k_out_bf16", vp), ("status_word", vp), ("q_out_bf16", vp), ("rope_table", vp), ("rope_table_positions", u32),
        ("reserved0", u32),
    ]


class LayerGlue(C.Structure):
    """axiom_layer_glue: buffers of one decoder layer's elementwise launches."""
    _fields_ = [
        ("abi_version", u32), ("struct_size", u32), ("columns", u32), ("hidden", u32), ("ffn", u32), ("scale_layout", u32),
        ("eps", f32), ("gate_up_input_scale", f32), ("down_input_scale", f32), ("reserved0", u32),
        ("residual_bf16", vp), ("mixer_out_bf16", vp), ("post_norm_gamma_bf16", vp), ("mlp_in_codes", vp), ("mlp_in_scales", vp),
        ("gate_up_bf16", vp), ("mlp_mid_codes", vp), ("mlp_mid_scales", vp), ("mlp_out_bf16", vp), ("tap_out_bf16", vp),
        ("next_norm_gamma_bf16", vp), ("next_norm_out_bf16", vp),
    ]


class AxiomError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status} ({status_string(status)})")


# name -> (restype, argtypes); every symbol include/axiom_b200.h declares
_BUF = [vp, u64]  # (axiom_device_buffer*, byte offset)
SIGNATURES = {
    "axiom_abi_version": (u32, []),
    "axiom_version": (C.c_char_p, []),
    "axiom_abi_info_get": (i32, [vp]),
    "axiom_abi_check": (i32, [u32]),
    "axiom_status_string": (C.c_char_p, [i32]),
    "axiom_runtime_create": (i32, [C.POINTER(vp), C.POINTER(AxiomConfig)]),
    "axiom_runtime_destroy": (None, [vp]),
    "axiom_runtime_device_count": (i32, [C.POINTER(u32)]),
    "axiom_runtime_device_id": (i32, [vp, C.POINTER(u32)]),
    "axiom_device_buffer_create": (i32, [vp, C.POINTER(vp), u64]),
    "axiom_device_buffer_destroy": (None, [vp]),
    "axiom_device_buffer_upload": (i32, [vp, u64, vp, u64]),
    "axiom_device_buffer_download": (i32, [vp, u64, vp, u64]),
    "axiom_device_buffer_copy": (i32, [vp, u64, vp, u64, u64]),
    "axiom_device_buffer_device_id": (i32, [vp, C.POINTER(u32)]),
    "axiom_device_buffer_cuda_pointer": (i32, [vp, C.POINTER(vp)]),
    "axiom_runtime_rmsnorm_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, f32]),
    "axiom_runtime_rmsnorm_f32_hp_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, f32]),
    "axiom_runtime_rmsnorm_f32_b1_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, f32]),
    "axiom_runtime_rmsnorm_f32_dual_device": (i32, [vp, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF, u32, f32]),
    "axiom_runtime_head_rmsnorm_f32_device": (i32, [vp, *_BUF, u32, u32, f32]),
    "axiom_runtime_rope_neox_f32_device": (i32, [vp, *_BUF, u32, u32, u32, f32]),
    "axiom_runtime_rope_neox_partial_f32_device": (i32, [vp, *_BUF, u32, u32, u32, u32, f32]),
    "axiom_runtime_qknorm_rope_f32_device": (i32, [vp, *_BUF, *_BUF, u32, u32, u32, f32, f32]),
    "axiom_runtime_qknorm_rope_pos_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, u32, f32, f32]),
    "axiom_runtime_qknorm_rope_pos_dual_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF, u32, u32, u32, f32, f32]),
    "axiom_runtime_qk_rmsnorm_w_f32_device": (i32, [vp, *_BUF, *_BUF, u32, u32, f32]),
    "axiom_runtime_kv_pool_store_paged_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF, u32, u32, u32, u32, u32, u32, u32]),
    "axiom_runtime_add_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32]),
    "axiom_runtime_silu_mul_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32]),
    "axiom_runtime_silu_mul_clamp_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, f32]),
    "axiom_runtime_f16_embedding_streams_device": (i32, [vp, *_BUF, *_BUF, u32, u32, u32]),
    "axiom_runtime_q8_0_embedding_gather_f32_device": (i32, [vp, *_BUF, *_BUF, u32, u32, u32]),
    "axiom_runtime_q8_0_embedding_gather_token_f32_device": (i32, [vp, *_BUF, *_BUF, *_BUF, u32, u32]),
    "axiom_qwen38_nvfp4_quantize_reference_f32": (i32, [i32, vp, f32, vp, vp, u32, vp]),
    "axiom_qwen38_fused_nvfp4_quantize_bf16_device": (i32, [i32, vp, u32, u32, f32, vp, vp, u32, vp]),
    "axiom_qwen38_fused_add_bf16_device": (i32, [i32, vp, vp, vp, u64, vp]),
    "axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device": (i32, [i32, vp, vp, vp, f32, u32, u32, f32, vp, vp, vp, u32, vp]),
    "axiom_qwen38_fused_fp8_epilogue_add_rmsnorm_nvfp4_device": (i32, [i32, vp, vp, vp, vp, vp, f32, u32, u32, f32, vp, vp, vp, u32, vp]),
    "axiom_qwen38_fused_add_rmsnorm_nvfp4_tap_bf16_device": (i32, [i32, vp, vp, vp, f32, u32, u32, f32, vp, vp, vp, u32, vp, vp]),
    "axiom_qwen38_fused_gather_add_rmsnorm_nvfp4_bf16_device": (i32, [i32, vp, u32, vp, vp, vp, f32, u32, u32, f32, vp, vp, vp, u32, vp, vp]),
    "axiom_qwen38_fused_swiglu_fp8_bf16_device": (i32, [i32, vp, u32, u32, vp, vp, vp]),
    "axiom_qwen38_fused_swiglu_nvfp4_bf16_device": (i32, [i32, vp, u32, u32, f32, vp, vp, u32, vp]),
    "axiom_qwen38_fused_sigmoid_gate_nvfp4_bf16_device": (i32, [i32, vp, vp, u32, u32, f32, vp, vp, vp, u32, vp]),
    "axiom_qwen38_fused_sigmoid_gate_heads_nvfp4_bf16_device": (i32, [i32, vp, vp, u32, u32, u32, f32, vp, vp, vp, u32, vp]),
    "axiom_qwen38_fused_top1_f32_device": (i32, [i32, vp, u32, u32, vp, vp]),
    "axiom_qwen38_fused_fp8_quantize_bf16_device": (i32, [i32, vp, u32, u32, vp, vp, vp, vp]),
    "axiom_qwen38_fused_embedding_gather_bf16_device": (i32, [i32, vp, u32, u32, vp, u32, vp, vp, vp]),
    "axiom_qwen38_fused_yarn_inv_freq_device": (i32, [i32, C.POINTER(RopeConfig), vp, vp]),
    "axiom_qwen38_fused_yarn_mscale": (f32, [f32]),
    "axiom_qwen38_fused_qk_norm_rope_paged_bf16_device": (i32, [i32, C.POINTER(QkRopeArgs), vp]),
    "axiom_runtime_nvfp4_quantize_bf16_device": (i32, [vp, *_BUF, u32, u32, f32, *_BUF, *_BUF, u32]),
    "axiom_runtime_add_rmsnorm_nvfp4_bf16_device": (i32, [vp, *_BUF, *_BUF, *_BUF, f32, u32, u32, f32, *_BUF, *_BUF, *_BUF, u32]),
    "axiom_runtime_swiglu_fp8_bf16_device": (i32, [vp, *_BUF, u32, u32, *_BUF, *_BUF]),
    "axiom_runtime_swiglu_nvfp4_bf16_device": (i32, [vp, *_BUF, u32, u32, f32, *_BUF, *_BUF, u32]),
    "axiom_runtime_embedding_gather_bf16_device": (i32, [vp, *_BUF, u32, u32, *_BUF, u32, *_BUF]),
    "axiom_runtime_qknorm_rope_yarn_paged_bf16_device": (i32, [vp, vp, u32, u32, u32, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF, *_BUF,
                                                                 u32, u32, u32, u32, f32, f32, *_BUF]),
    "axiom_runtime_nvfp4_quantize_bf16": (i32, [vp, vp, u32, u32, f32, vp, vp]),
    "axiom_runtime_add_rmsnorm_nvfp4_bf16": (i32, [vp, vp, vp, vp, f32, u32, u32, f32, vp, vp]),
    "axiom_runtime_swiglu_fp8_bf16": (i32, [vp, vp, u32, u32, vp, vp]),
    "axiom_nvfp4_scale_plane_bytes": (u64, [u32, u32, u32]),
    "axiom_nvfp4_scale_plane_offset": (u64, [u32, u32, u32, u32]),
    "axiom_b200_kernel_launch_count": (u64, []),
    "axiom_b200_static_scratch_bytes": (u64, []),
    "axiom_b200_nvfp4_quantize_bf16_host_static": (i32, [C.c_int, vp, u32, u32, f32, u32, vp, vp, vp]),
    "axiom_b200_pipeline_faults": (u32, [i32]),
    "axiom_b200_prepare": (i32, [i32]),
    # include/axiom_b200_engine.h (typed structures: axiom-kernel_b200/engine.py)
    "axiom_b200_step_provider_create": (i32, [vp, vp, C.POINTER(vp)]),
    "axiom_b200_step_provider_destroy": (None, [vp]),
    "axiom_b200_step_provider_forward_step": (i32, [vp, vp, i32, vp]),
    "axiom_b200_step_provider_scratch": (vp, [vp, u32]),
    "axiom_qwen38_fused_layer_post_mixer_device": (i32, [i32, C.POINTER(LayerGlue), vp]),
    "axiom_qwen38_fused_layer_mlp_mid_device": (i32, [i32, C.POINTER(LayerGlue), vp]),
    "axiom_qwen38_fused_layer_post_mlp_device": (i32, [i32, C.POINTER(LayerGlue), vp]),
    "axiom_b200_test_arm_wait_timeout": (i32, [u32, u32]),
    "axiom_qwen38_fused_fp8_quantize_static_bf16_device": (i32, [i32, vp, u32, u32, f32, vp, vp]),
    "axiom_qwen38_fused_swiglu_fp8_static_bf16_device": (i32, [i32, vp, u32, u32, f32, vp, vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libaxiom_b200.so (once) and type every exported symbol."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {HERE.name}/build.py`; "
                "there is no CPU or PyTorch fallback for this library")
        handle = C.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = header/library mismatch
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().axiom_status_string(status).decode()


def check(status: int, where: str) -> None:
    if status != AXIOM_OK:
        raise AxiomError(status, where)


def _ptr(t) -> int | None:
    """Address of a torch tensor / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream_handle(stream) -> int | None:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


# ---------------------------------------------------------------------------
# raw-pointer, stream-explicit wrappers (tensors are torch CUDA tensors)
# ---------------------------------------------------------------------------

def nvfp4_quantize(device, x_bf16, rows, cols, global_scale, codes, scales, layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_nvfp4_quantize_bf16_device(
        device, _ptr(x_bf16), rows, cols, global_scale, _ptr(codes), _ptr(scales), layout, _stream_handle(stream))


def add_bf16(device, a, b, out, count, stream=None):
    return lib().axiom_qwen38_fused_add_bf16_device(device, _ptr(a), _ptr(b), _ptr(out), count, _stream_handle(stream))


def add_rmsnorm_nvfp4(device, hidden, residual, gamma, eps, rows, cols, global_scale, norm_out, codes, scales,
                      layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device(
        device, _ptr(hidden), _ptr(residual), _ptr(gamma), eps, rows, cols, global_scale, _ptr(norm_out),
        _ptr(codes), _ptr(scales), layout, _stream_handle(stream))


def swiglu_fp8(device, gate_up, rows, width, codes, scales, stream=None):
    return lib().axiom_qwen38_fused_swiglu_fp8_bf16_device(
        device, _ptr(gate_up), rows, width, _ptr(codes), _ptr(scales), _stream_handle(stream))


def swiglu_nvfp4(device, gate_up, rows, width, global_scale, codes, scales, layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_swiglu_nvfp4_bf16_device(
        device, _ptr(gate_up), rows, width, global_scale, _ptr(codes), _ptr(scales), layout, _stream_handle(stream))


def fp8_epilogue_add_rmsnorm_nvfp4(device, gemm_out, weight_scale, input_scale, residual, gamma, eps, rows, cols, global_scale,
                                   norm_out, codes, scales, layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_fp8_epilogue_add_rmsnorm_nvfp4_device(
        device, _ptr(gemm_out), _ptr(weight_scale), _ptr(input_scale), _ptr(residual), _ptr(gamma), eps, rows, cols,
        global_scale, _ptr(norm_out), _ptr(codes), _ptr(scales), layout, _stream_handle(stream))


def add_rmsnorm_nvfp4_tap(device, hidden, residual, gamma, eps, rows, cols, global_scale, norm_out, codes, scales, layout, tap,
                          stream=None):
    return lib().axiom_qwen38_fused_add_rmsnorm_nvfp4_tap_bf16_device(
        device, _ptr(hidden), _ptr(residual), _ptr(gamma), eps, rows, cols, global_scale, _ptr(norm_out), _ptr(codes),
        _ptr(scales), layout, _ptr(tap), _stream_handle(stream))


def gather_add_rmsnorm_nvfp4(device, table, vocab, token_ids, residual, gamma, eps, rows, cols, G, norm_out, codes, scales,
                             layout=SCALE_CANONICAL, status_word=None, stream=None):
    return lib().axiom_qwen38_fused_gather_add_rmsnorm_nvfp4_bf16_device(
        device, _ptr(table), vocab, _ptr(token_ids), _ptr(residual), _ptr(gamma), eps, rows, cols, G, _ptr(norm_out),
        _ptr(codes), _ptr(scales), layout, _ptr(status_word), _stream_handle(stream))


def sigmoid_gate_heads_nvfp4(device, attention, q_gate, rows, heads, head_dim, G, out_bf16, codes, scales,
                             layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_sigmoid_gate_heads_nvfp4_bf16_device(
        device, _ptr(attention), _ptr(q_gate), rows, heads, head_dim, G, _ptr(out_bf16), _ptr(codes), _ptr(scales), layout,
        _stream_handle(stream))


def sigmoid_gate_nvfp4(device, attention, gate, rows, width, G, out_bf16, codes, scales, layout=SCALE_CANONICAL, stream=None):
    return lib().axiom_qwen38_fused_sigmoid_gate_nvfp4_bf16_device(device, _ptr(attention), _ptr(gate), rows, width, G,
                                                                   _ptr(out_bf16), _ptr(codes), _ptr(scales), layout,
                                                                   _stream_handle(stream))


def top1(device, logits, rows, vocab, results, stream=None):
    """results: device buffer of rows x (float value, uint32 token_id, uint32 invalid)."""
    return lib().axiom_qwen38_fused_top1_f32_device(device, _ptr(logits), rows, vocab, _ptr(results), _stream_handle(stream))


def fp8_quantize_static(device, x_bf16, rows, cols, scale, codes, stream=None):
    return lib().axiom_qwen38_fused_fp8_quantize_static_bf16_device(device, _ptr(x_bf16), rows, cols, scale, _ptr(codes),
                                                                   _stream_handle(stream))


def swiglu_fp8_static(device, gate_up, rows, width, scale, codes, stream=None):
    return lib().axiom_qwen38_fused_swiglu_fp8_static_bf16_device(device, _ptr(gate_up), rows, width, scale, _ptr(codes),
                                                                 _stream_handle(stream))


def fp8_quantize(device, x_bf16, rows, cols, codes, scales, status_word=None, stream=None):
    return lib().axiom_qwen38_fused_fp8_quantize_bf16_device(
        device, _ptr(x_bf16), rows, cols, _ptr(codes), _ptr(scales), _ptr(status_word), _stream_handle(stream))


def embedding_gather(device, table, vocab, hidden, ids, tokens, out, status_word=None, stream=None):
    return lib().axiom_qwen38_fused_embedding_gather_bf16_device(
        device, _ptr(table), vocab, hidden, _ptr(ids), tokens, _ptr(out), _ptr(status_word), _stream_handle(stream))


def yarn_inv_freq(device, rope_dim, theta, factor, original_context, beta_fast, beta_slow, out, stream=None):
    cfg = RopeConfig(AXIOM_ABI_VERSION, rope_dim, theta, factor, original_context, beta_fast, beta_slow)
    return lib().axiom_qwen38_fused_yarn_inv_freq_device(device, C.byref(cfg), _ptr(out), _stream_handle(stream))


def yarn_mscale(factor: float) -> float:
    return float(lib().axiom_qwen38_fused_yarn_mscale(factor))


def make_qk_args(*, tokens, q_heads, k_heads, head_dim, rope_dim, flags=0, eps=1e-6, mscale=1.0, block_tokens=16,
                 n_layers=1, layer=0, pool_stride=0, tbl_stride=0, n_blocks=0, q=None, k=None, v=None,
                 q_gamma=None, k_gamma=None, inv_freq=None, positions=None, block_tables=None, k_pool=None,
                 v_pool=None, k_out=None, status_word=None, q_out=None, rope_table=None,
                 rope_table_positions=0) -> QkRopeArgs:
    return QkRopeArgs(AXIOM_ABI_VERSION, C.sizeof(QkRopeArgs), tokens, q_heads, k_heads, head_dim, rope_dim, flags,
                      eps, mscale, block_tokens, n_layers, layer, pool_stride, tbl_stride, n_blocks, _ptr(q),
                      _ptr(k), _ptr(v), _ptr(q_gamma), _ptr(k_gamma), _ptr(inv_freq), _ptr(positions),
                      _ptr(block_tables), _ptr(k_pool), _ptr(v_pool), _ptr(k_out), _ptr(status_word), _ptr(q_out),
                      _ptr(rope_table), rope_table_positions, 0)


def make_layer_glue(*, columns, hidden, ffn, scale_layout=SCALE_TILED, eps=1e-6, gate_up_input_scale=1.0, down_input_scale=1.0,
                    residual=None, mixer_out=None, post_norm_gamma=None, mlp_in_codes=None, mlp_in_scales=None, gate_up=None,
                    mlp_mid_codes=None, mlp_mid_scales=None, mlp_out=None, tap_out=None, next_norm_gamma=None,
                    next_norm_out=None) -> LayerGlue:
    return LayerGlue(AXIOM_ABI_VERSION, C.sizeof(LayerGlue), columns, hidden, ffn, scale_layout, eps, gate_up_input_scale,
                     down_input_scale, 0, _ptr(residual), _ptr(mixer_out), _ptr(post_norm_gamma), _ptr(mlp_in_codes),
                     _ptr(mlp_in_scales), _ptr(gate_up), _ptr(mlp_mid_codes), _ptr(mlp_mid_scales), _ptr(mlp_out), _ptr(tap_out),
                     _ptr(next_norm_gamma), _ptr(next_norm_out))


def layer_post_mixer(device, glue: LayerGlue, stream=None):
    return lib().axiom_qwen38_fused_layer_post_mixer_device(device, C.byref(glue), _stream_handle(stream))


def layer_mlp_mid(device, glue: LayerGlue, stream=None):
    return lib().axiom_qwen38_fused_layer_mlp_mid_device(device, C.byref(glue), _stream_handle(stream))


def layer_post_mlp(device, glue: LayerGlue, stream=None):
    return lib().axiom_qwen38_fused_layer_post_mlp_device(device, C.byref(glue), _stream_handle(stream))


def qk_norm_rope_paged(device, args: QkRopeArgs, stream=None):
    return lib().axiom_qwen38_fused_qk_norm_rope_paged_bf16_device(device, C.byref(args), _stream_handle(stream))


# ---------------------------------------------------------------------------
# runtime / device-buffer handles
# ---------------------------------------------------------------------------

class Runtime:
    """Owns an axiom_runtime handle."""

    def __init__(self, device: int = 0, backend: int = AXIOM_BACKEND_CUDA, abi_version: int = AXIOM_ABI_VERSION):
        self.handle = vp()
        cfg = AxiomConfig(abi_version, backend, device, 0)
        check(lib().axiom_runtime_create(C.byref(self.handle), C.byref(cfg)), "axiom_runtime_create")
        self.device = device

    def close(self):
        if self.handle:
            lib().axiom_runtime_destroy(self.handle)
            self.handle = vp()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class DeviceBuffer:
    """Owns an axiom_device_buffer handle."""

    def __init__(self, runtime: Runtime, nbytes: int):
        self.handle = vp()
        check(lib().axiom_device_buffer_create(runtime.handle, C.byref(self.handle), nbytes), "axiom_device_buffer_create")
        self.nbytes = nbytes

    def upload(self, array, offset: int = 0):
        """array: contiguous numpy array."""
        return lib().axiom_device_buffer_upload(self.handle, offset, array.ctypes.data, array.nbytes)

    def download(self, array, offset: int = 0):
        return lib().axiom_device_buffer_download(self.handle, offset, array.ctypes.data, array.nbytes)

    def cuda_pointer(self) -> int:
        out = vp()
        check(lib().axiom_device_buffer_cuda_pointer(self.handle, C.byref(out)), "axiom_device_buffer_cuda_pointer")
        return out.value

    def close(self):
        if self.handle:
            lib().axiom_device_buffer_destroy(self.handle)
            self.handle = vp()

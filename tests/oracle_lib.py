"""numpy front-end of the CPU oracle (oracle/liboracle.so) for the tests.

Test infrastructure only.  The shared objects are built on demand with
`make -C oracle`; nothing here is imported by the library or its binding.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"

u8p, u16p, u32p, i32p, f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_uint32, C.c_int32, C.c_float))


def _build():
    subprocess.run(["make", "-C", str(ORACLE_DIR), "-s"], check=True, capture_output=True)


def _load(name: str) -> C.CDLL:
    path = ORACLE_DIR / name
    if not path.exists():
        _build()
    return C.CDLL(str(path))


class RopeParams(C.Structure):
    _fields_ = [("theta", C.c_float), ("factor", C.c_float), ("original_context", C.c_float),
                ("beta_fast", C.c_float), ("beta_slow", C.c_float), ("rope_dim", C.c_uint32)]


class QkParams(C.Structure):
    _fields_ = [("tokens", C.c_uint32), ("q_heads", C.c_uint32), ("k_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("rope_dim", C.c_uint32), ("eps", C.c_float), ("mscale", C.c_float), ("block_tokens", C.c_uint32),
                ("n_layers", C.c_uint32), ("layer", C.c_uint32), ("pool_stride", C.c_uint32),
                ("tbl_stride", C.c_uint32), ("n_blocks", C.c_uint32), ("ring", C.c_uint32),
                ("per_token_table", C.c_uint32)]


_o = None
_pin = None


def o() -> C.CDLL:
    global _o
    if _o is None:
        _o = _load("liboracle.so")
        _o.axo_bf16_round.restype = C.c_float
        _o.axo_bf16_round.argtypes = [C.c_float]
        _o.axo_bf16_to_f32.restype = C.c_float
        _o.axo_bf16_to_f32.argtypes = [C.c_uint16]
        _o.axo_f32_to_bf16.restype = C.c_uint16
        _o.axo_f32_to_bf16.argtypes = [C.c_float]
        _o.axo_e4m3_decode.restype = C.c_float
        _o.axo_e4m3_decode.argtypes = [C.c_uint8]
        for n in ("axo_e4m3_encode_satfinite", "axo_e4m3_encode_scale", "axo_e2m1_encode"):
            getattr(_o, n).restype = C.c_uint8
            getattr(_o, n).argtypes = [C.c_float]
        _o.axo_e2m1_decode.restype = C.c_float
        _o.axo_e2m1_decode.argtypes = [C.c_uint8]
        _o.axo_silu_mul.restype = C.c_float
        _o.axo_silu_mul.argtypes = [C.c_float, C.c_float]
        _o.axo_yarn_mscale.restype = C.c_float
        _o.axo_yarn_mscale.argtypes = [C.c_float]
        _o.axo_scale_tiled_bytes.restype = C.c_uint64
        _o.axo_scale_tiled_bytes.argtypes = [C.c_uint32, C.c_uint32]
        _o.axo_scale_tiled_offset.restype = C.c_uint64
        _o.axo_scale_tiled_offset.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        _o.axo_set_threads.argtypes = [C.c_int]
        _o.axo_get_threads.restype = C.c_int
    return _o


def pin() -> C.CDLL:
    """Host paths of the CUDA toolkit FP8/FP4 converters."""
    global _pin
    if _pin is None:
        _pin = _load("libtoolkit_pin.so")
    return _pin


def _p(a, typ=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _ok(rc, what):
    if rc != 0:
        raise ValueError(f"oracle {what} rejected its arguments (rc={rc})")


# ---- bf16 helpers in numpy (bit-identical to axo_f32_to_bf16 for non-NaN) ----

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (b & 0x7fffffff) > 0x7f800000
    r = ((b + 0x7fff + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7fff
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of BF16 at the magnitude of x (F32 array); smallest normal spacing near 0."""
    a = np.abs(np.asarray(x, dtype=np.float32))
    e = np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -126))))
    return np.exp2(e - 7).astype(np.float32)


# ---- quantizers ----

def nvfp4_quantize_bf16(x_bits: np.ndarray, G: float):
    rows, cols = x_bits.shape
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    _ok(o().axo_nvfp4_quantize_bf16(_p(x_bits), rows, cols, C.c_float(G), _p(codes), _p(scales)), "nvfp4_quantize_bf16")
    return codes, scales


def nvfp4_quantize_f32(x: np.ndarray, G: float):
    rows, cols = x.shape
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    _ok(o().axo_nvfp4_quantize_f32(_p(x), rows, cols, C.c_float(G), _p(codes), _p(scales)), "nvfp4_quantize_f32")
    return codes, scales


def scales_to_tiled(canonical: np.ndarray) -> np.ndarray:
    rows, groups = canonical.shape
    out = np.empty(int(o().axo_scale_tiled_bytes(rows, groups)), np.uint8)
    _ok(o().axo_scales_canonical_to_tiled(_p(canonical), rows, groups, _p(out)), "scales_to_tiled")
    return out


def fp8_quantize_f32(x: np.ndarray):
    rows, cols = x.shape
    codes = np.empty((rows, cols), np.uint8)
    scales = np.empty(rows, np.float32)
    _ok(o().axo_fp8_quantize_f32(_p(x), rows, cols, _p(codes), _p(scales)), "fp8_quantize_f32")
    return codes, scales


def fp8_quantize_static_f32(x: np.ndarray, scale: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    codes = np.empty(x.shape, np.uint8)
    _ok(o().axo_fp8_quantize_static_f32(_p(x), x.size, C.c_float(scale), _p(codes)), "fp8_quantize_static_f32")
    return codes


def fp8_quantize_bf16(x_bits: np.ndarray):
    rows, cols = x_bits.shape
    codes = np.empty((rows, cols), np.uint8)
    scales = np.empty(rows, np.float32)
    status = np.zeros(1, np.uint32)
    _ok(o().axo_fp8_quantize_bf16(_p(x_bits), rows, cols, _p(codes), _p(scales), _p(status)), "fp8_quantize_bf16")
    return codes, scales, int(status[0])


# ---- add / rmsnorm ----

def add_bf16(a_bits, b_bits):
    out = np.empty_like(a_bits)
    _ok(o().axo_add_bf16(_p(a_bits), _p(b_bits), C.c_uint64(a_bits.size), _p(out)), "add_bf16")
    return out


def add_rmsnorm_bf16(hidden_bits, residual_bits, gamma_bits, eps):
    rows, cols = residual_bits.shape
    res_out = np.empty_like(residual_bits)
    norm = np.empty_like(residual_bits)
    _ok(o().axo_add_rmsnorm_bf16(_p(hidden_bits), _p(residual_bits), _p(gamma_bits), C.c_float(eps), rows, cols,
                                 _p(res_out), _p(norm)), "add_rmsnorm_bf16")
    return res_out, norm


def add_rmsnorm_nvfp4_bf16(hidden_bits, residual_bits, gamma_bits, eps, G):
    rows, cols = residual_bits.shape
    res_out = np.empty_like(residual_bits)
    norm = np.empty_like(residual_bits)
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    _ok(o().axo_add_rmsnorm_nvfp4_bf16(_p(hidden_bits), _p(residual_bits), _p(gamma_bits), C.c_float(eps), rows, cols,
                                       C.c_float(G), _p(res_out), _p(norm), _p(codes), _p(scales)),
        "add_rmsnorm_nvfp4_bf16")
    return res_out, norm, codes, scales


# ---- swiglu ----

def swiglu_f32(gate_up_bits):
    rows, two_w = gate_up_bits.shape
    out = np.empty((rows, two_w // 2), np.float32)
    _ok(o().axo_swiglu_f32(_p(gate_up_bits), rows, two_w // 2, _p(out)), "swiglu_f32")
    return out


def swiglu_fp8_bf16(gate_up_bits):
    rows, two_w = gate_up_bits.shape
    codes = np.empty((rows, two_w // 2), np.uint8)
    scales = np.empty(rows, np.float32)
    _ok(o().axo_swiglu_fp8_bf16(_p(gate_up_bits), rows, two_w // 2, _p(codes), _p(scales)), "swiglu_fp8_bf16")
    return codes, scales


def swiglu_nvfp4_bf16(gate_up_bits, G):
    rows, two_w = gate_up_bits.shape
    w = two_w // 2
    codes = np.empty((rows, w // 2), np.uint8)
    scales = np.empty((rows, w // 16), np.uint8)
    _ok(o().axo_swiglu_nvfp4_bf16(_p(gate_up_bits), rows, w, C.c_float(G), _p(codes), _p(scales)), "swiglu_nvfp4_bf16")
    return codes, scales


# ---- rope / qk ----

def yarn_inv_freq(theta, factor, original_context, beta_fast, beta_slow, rope_dim, host_table=False):
    p = RopeParams(theta, factor, original_context, beta_fast, beta_slow, rope_dim)
    out = np.empty(rope_dim // 2, np.float32)
    fn = o().axo_yarn_inv_freq_host_table if host_table else o().axo_yarn_inv_freq
    _ok(fn(C.byref(p), _p(out)), "yarn_inv_freq")
    return out


def qk_norm_rope_paged(q_bits, k_bits, v_bits, q_gamma, k_gamma, inv_freq, positions, block_tables, *,
                       rope_dim, eps, mscale, block_tokens=16, n_layers=1, layer=0, pool_stride=None, n_blocks=0,
                       ring=False, per_token_table=False, k_pool=None, v_pool=None, want_k_out=False):
    """q_bits [T,Hq,D] (returns a rotated copy), k_bits [T,Hk,D]; pools are modified in place."""
    tokens = positions.shape[0]
    q_heads = q_bits.shape[1] if q_bits is not None else 0
    k_heads = k_bits.shape[1] if k_bits is not None else 0
    head_dim = (q_bits if q_bits is not None else k_bits).shape[2]
    tbl_stride = block_tables.shape[-1] if block_tables is not None else 0
    p = QkParams(tokens, q_heads, k_heads, head_dim, rope_dim, eps, mscale, block_tokens, n_layers, layer,
                 pool_stride if pool_stride is not None else k_heads * head_dim, tbl_stride, n_blocks,
                 1 if ring else 0, 1 if per_token_table else 0)
    q_out = q_bits.copy() if q_bits is not None else None
    k_out = np.empty_like(k_bits) if (want_k_out and k_bits is not None) else None
    status = np.zeros(1, np.uint32)
    _ok(o().axo_qk_norm_rope_paged_bf16(C.byref(p), _p(q_out), _p(k_bits), _p(v_bits), _p(q_gamma), _p(k_gamma),
                                        _p(inv_freq), _p(positions), _p(block_tables), _p(k_pool), _p(v_pool),
                                        _p(k_out), _p(status)), "qk_norm_rope_paged_bf16")
    return q_out, k_out, int(status[0])


def qk_norm_rope_round_after_norm(x_bits, gamma, rope_table, positions, eps=1e-6):
    """The BF16 ("draft") rounding convention; x_bits [T, H, D] (returns a copy), rope_table [P, D] = cos | sin."""
    tokens, heads, head_dim = x_bits.shape
    out = x_bits.copy()
    status = np.zeros(1, np.uint32)
    table = np.ascontiguousarray(rope_table, np.float32)
    _ok(o().axo_qk_norm_rope_round_after_norm_bf16(_p(out), _p(gamma), _p(table), table.shape[0], _p(positions), tokens, heads,
                                                   head_dim, C.c_float(eps), _p(status)), "qk_norm_rope_round_after_norm")
    return out, int(status[0])


def rope_table_host(inv_freq, head_dim, mscale, positions):
    out = np.empty((positions, head_dim), np.float32)
    _ok(o().axo_rope_table_host(_p(inv_freq), head_dim, C.c_float(mscale), positions, _p(out)), "rope_table_host")
    return out


def sigmoid_gate_nvfp4_bf16(attention_bits, gate_bits, G):
    rows, width = attention_bits.shape
    out = np.empty_like(attention_bits)
    codes = np.empty((rows, width // 2), np.uint8)
    scales = np.empty((rows, width // 16), np.uint8)
    _ok(o().axo_sigmoid_gate_nvfp4_bf16(_p(attention_bits), _p(gate_bits), rows, width, C.c_float(G), _p(out), _p(codes),
                                        _p(scales)), "sigmoid_gate_nvfp4_bf16")
    return out, codes, scales


def bf16_to_e4m3_scale1(bits):
    flat = np.ascontiguousarray(bits).reshape(-1)
    out = np.empty(flat.size, np.uint8)
    _ok(o().axo_bf16_to_e4m3_scale1(_p(flat), _p(out), C.c_uint64(flat.size)), "bf16_to_e4m3_scale1")
    return out.reshape(bits.shape)


def embedding_gather_bf16(table_bits, ids):
    vocab, hidden = table_bits.shape
    out = np.empty((ids.shape[0], hidden), np.uint16)
    _ok(o().axo_embedding_gather_bf16(_p(table_bits), vocab, hidden, _p(ids), ids.shape[0], _p(out)), "embedding_gather")
    return out


def fp8_row_scale_epilogue_bf16(raw, weight_scale_bits, input_scale):
    rows, cols = raw.shape
    out = np.empty((rows, cols), np.uint16)
    _ok(o().axo_fp8_row_scale_epilogue_bf16(_p(np.ascontiguousarray(raw)), _p(weight_scale_bits), _p(input_scale), rows, cols,
                                            _p(out)), "fp8 epilogue")
    return out


def top1_f32(logits):
    rows, vocab = logits.shape
    out = np.empty((rows, 3), np.uint32)
    _ok(o().axo_top1_f32(_p(np.ascontiguousarray(logits)), rows, vocab, _p(out)), "top1")
    return out


def q8_0_embedding_gather_f32(embedding_bytes, token_id, token_count, hidden):
    out = np.empty(hidden, np.float32)
    _ok(o().axo_q8_0_embedding_gather_f32(_p(embedding_bytes), token_id, token_count, hidden, _p(out)), "q8_0 gather")
    return out


def f16_embedding_streams_f32(embedding_bits, token_id, hidden, streams):
    out = np.empty(hidden * streams, np.float32)
    _ok(o().axo_f16_embedding_streams_f32(_p(embedding_bits), token_id, hidden, streams, _p(out)), "f16 streams")
    return out


# ---- generic f32 ops ----

def rmsnorm_f32(w, x, eps, variant="plain"):
    out = np.empty_like(x)
    fn = {"plain": o().axo_rmsnorm_f32, "hp": o().axo_rmsnorm_f32_hp, "b1": o().axo_rmsnorm_f32_b1}[variant]
    _ok(fn(_p(w), _p(x), _p(out), x.size, C.c_float(eps)), "rmsnorm_f32")
    return out


def head_rmsnorm_f32(x, heads, head_dim, eps):
    out = x.copy()
    _ok(o().axo_head_rmsnorm_f32(_p(out), heads, head_dim, C.c_float(eps)), "head_rmsnorm_f32")
    return out


def qk_rmsnorm_w_f32(x, w, heads, head_dim, eps):
    out = x.copy()
    _ok(o().axo_qk_rmsnorm_w_f32(_p(out), _p(w), heads, head_dim, C.c_float(eps)), "qk_rmsnorm_w_f32")
    return out


def rope_neox_f32(x, heads, head_dim, n_rot, pos, theta):
    out = x.copy()
    _ok(o().axo_rope_neox_f32(_p(out), heads, head_dim, n_rot, pos, C.c_float(theta)), "rope_neox_f32")
    return out


def qknorm_rope_f32(x, w, heads, head_dim, pos, theta, eps):
    out = x.copy()
    _ok(o().axo_qknorm_rope_f32(_p(out), _p(w), heads, head_dim, pos, C.c_float(theta), C.c_float(eps)), "qknorm_rope_f32")
    return out


def add_f32(a, b):
    out = np.empty_like(a)
    _ok(o().axo_add_f32(_p(a), _p(b), _p(out), a.size), "add_f32")
    return out


def silu_mul_f32(gate, up, clamp_abs=0.0):
    out = np.empty_like(gate)
    _ok(o().axo_silu_mul_f32(_p(gate), _p(up), _p(out), gate.size, C.c_float(clamp_abs)), "silu_mul_f32")
    return out


def kv_pool_store_paged_f32(k_stage, v_stage, k_pool, v_pool, tables, pos, *, n_layers, layer, block_tokens,
                            pool_stride):
    active, kv_dim = k_stage.shape
    _ok(o().axo_kv_pool_store_paged_f32(_p(k_stage), _p(v_stage), _p(k_pool), _p(v_pool), _p(tables), _p(pos), active,
                                        tables.shape[1], n_layers, layer, block_tokens, pool_stride, kv_dim),
        "kv_pool_store_paged_f32")

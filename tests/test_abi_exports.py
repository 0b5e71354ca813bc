"""CPU-side checks of the C-ABI boundary: the library loads, exports every
symbol the public header declares, and the binding's signature table covers
exactly that set.  No compute call is made (no GPU needed)."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADERS = [ROOT / "include" / "axiom_b200.h", ROOT / "include" / "axiom_b200_engine.h"]


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", "\n".join(h.read_text() for h in HEADERS), flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    names = re.findall(r"\b(axiom_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_hot_path_entry_points():
    names = declared_functions()
    for must in ["axiom_qwen38_nvfp4_quantize_reference_f32", "axiom_runtime_create",
                 "axiom_device_buffer_cuda_pointer", "axiom_runtime_kv_pool_store_paged_f32_device",
                 "axiom_qwen38_fused_add_rmsnorm_nvfp4_bf16_device",
                 "axiom_qwen38_fused_qk_norm_rope_paged_bf16_device", "axiom_qwen38_fused_swiglu_fp8_bf16_device",
                 "axiom_qwen38_fused_embedding_gather_bf16_device", "axiom_qwen38_fused_nvfp4_quantize_bf16_device"]:
        assert must in names


def test_library_exports_every_declared_symbol(axk):
    lib = C.CDLL(str(axk.LIB_PATH))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_signature_table_matches_header(axk):
    assert sorted(axk.SIGNATURES) == declared_functions()
    axk.lib()  # types every symbol; raises on a missing one


def test_identity_calls_need_no_device(axk):
    lib = axk.lib()
    assert lib.axiom_abi_version() == 1
    assert lib.axiom_abi_check(1) == axk.AXIOM_OK
    assert lib.axiom_abi_check(2) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert b"sm_100a" in lib.axiom_version()

    class AbiInfo(C.Structure):
        _fields_ = [("abi_version", C.c_uint32), ("header_abi_version", C.c_uint32), ("runtime_abi_version", C.c_uint32),
                    ("struct_size", C.c_uint32), ("version", C.c_char_p), ("backend", C.c_char_p), ("build_target", C.c_char_p),
                    ("flags", C.c_uint64)]

    info = AbiInfo(abi_version=1)
    assert lib.axiom_abi_info_get(C.byref(info)) == axk.AXIOM_OK
    assert (info.header_abi_version, info.runtime_abi_version, info.struct_size) == (1, 1, C.sizeof(AbiInfo))
    assert info.backend == b"cuda" and info.build_target == b"sm_100a" and info.version == lib.axiom_version()
    stale = AbiInfo(abi_version=2)
    assert lib.axiom_abi_info_get(C.byref(stale)) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_abi_info_get(None) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert axk.status_string(0) == "ok" and axk.status_string(1) == "invalid argument"
    assert axk.status_string(7) == "budget exceeded" and axk.status_string(99) == "unknown error"
    assert lib.axiom_nvfp4_scale_plane_bytes(4096, 320, axk.SCALE_TILED) == 32 * 80 * 512
    assert lib.axiom_nvfp4_scale_plane_bytes(4096, 320, axk.SCALE_CANONICAL) == 4096 * 320
    assert lib.axiom_nvfp4_scale_plane_offset(33, 5, 320, axk.SCALE_TILED) == 512 + 16 + 4 + 1
    assert abs(axk.yarn_mscale(4.0) - 1.138629436111989) < 1e-7


def test_argument_checks_come_before_any_device_work(axk):
    """Bad arguments are rejected on the host: these calls return without touching CUDA."""
    lib = axk.lib()
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, None, 1.0, None, None, 16, None) == inv
    assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, 16, 1.0, 16, 16, 24, None) == inv       # cols % 16
    assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, 16, 0.0, 16, 16, 32, None) == inv       # scale <= 0
    assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, 16, float("inf"), 16, 16, 32, None) == inv
    assert axk.nvfp4_quantize(0, 16, 4, 24, 1.0, 16, 16) == inv
    assert axk.nvfp4_quantize(0, 16, 4, 32, float("nan"), 16, 16) == inv
    assert axk.nvfp4_quantize(0, 16, 4, 32, 1.0, 16, 16, layout=7) == inv
    assert axk.nvfp4_quantize(0, 8, 4, 32, 1.0, 16, 16) == inv                                       # misaligned input
    assert axk.swiglu_fp8(0, 16, 0, 64, 16, 16) == inv
    assert axk.swiglu_fp8(0, 16, 4, 60, 16, 16) == inv
    assert axk.add_rmsnorm_nvfp4(0, None, 16, 16, 1e-6, 4, 40, 1.0, None, 16, 16) == inv              # cols % 16
    assert axk.add_rmsnorm_nvfp4(0, None, 16, 16, 1e-6, 4, 64, 1.0, None, 16, None) == inv            # codes without scales
    assert axk.add_rmsnorm_nvfp4(0, None, 16, 16, 0.0, 4, 64, 1.0, 16, None, None) == inv             # eps
    assert axk.embedding_gather(0, 16, 0, 64, 16, 4, 16) == inv
    args = axk.make_qk_args(tokens=4, q_heads=2, k_heads=1, head_dim=96, rope_dim=32)
    assert axk.qk_norm_rope_paged(0, args) == inv                                                     # head_dim
    out = C.c_void_p(123)
    assert lib.axiom_runtime_create(C.byref(out), None) == inv
    cfg = axk.AxiomConfig(2, axk.AXIOM_BACKEND_CUDA, 0, 0)
    assert lib.axiom_runtime_create(C.byref(out), C.byref(cfg)) == inv                                # abi mismatch
    cfg = axk.AxiomConfig(1, axk.AXIOM_BACKEND_CLUSTER, 0, 0)
    assert lib.axiom_runtime_create(C.byref(out), C.byref(cfg)) == axk.AXIOM_ERR_UNSUPPORTED_BACKEND
    assert out.value is None                                                                          # out-param nulled first
    assert lib.axiom_device_buffer_create(None, C.byref(out), 16) == inv
    assert lib.axiom_runtime_add_f32_device(None, None, 0, None, 0, None, 0, 4) == inv

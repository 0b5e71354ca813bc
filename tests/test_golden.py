"""CPU oracle vs the committed fixture of the REFERENCE'S OWN KERNELS' outputs
(tests/golden/reference_b200.npz, written by tests/golden/make_golden.py on a B200).

Integer outputs of ops without a transcendental are bit-exact.  Where the device math library
enters (rsqrtf, expf, cosf/sinf, powf) the oracle uses the C library and is held to the stated
tolerance instead."""
import importlib
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as ol

wl = importlib.import_module("axiom-kernel_b200.workloads")
FIXTURE = Path(__file__).resolve().parent / "golden" / "reference_b200.npz"


@pytest.fixture(scope="module")
def fx():
    return np.load(FIXTURE)


def test_nvfp4_quantizer_bit_exact(fx):
    codes, scales = ol.nvfp4_quantize_bf16(fx["q_in"], float(fx["q_G"]))
    assert np.array_equal(codes, fx["q_codes"]) and np.array_equal(scales, fx["q_scales"])
    assert np.array_equal(ol.scales_to_tiled(scales), fx["q_plane_warp"])          # tiled scale plane layout
    for tag in "abc":                                                               # zeros, NaN, inf, denormals, ties
        codes, scales = ol.nvfp4_quantize_bf16(fx["qs_in"], float(fx[f"qs_G_{tag}"]))
        assert np.array_equal(codes, fx[f"qs_codes_{tag}"]) and np.array_equal(scales, fx[f"qs_scales_{tag}"])


def test_add_rmsnorm(fx):
    res, norm = ol.add_rmsnorm_bf16(fx["n_hidden"], fx["n_residual"], fx["n_gamma"], 1e-6)
    assert np.array_equal(res, fx["n_res_out"])                                    # bit-exact
    a, b = wl.from_bf16_bits(norm), wl.from_bf16_bits(fx["n_norm"])
    assert np.all(np.abs(a - b) <= ol.bf16_ulp(b))                                 # rsqrtf: within 1 BF16 ulp
    assert np.mean(norm != fx["n_norm"]) < 0.01
    _, norm_only = ol.add_rmsnorm_bf16(None, fx["n_residual"], fx["n_gamma"], 1e-6)
    b = wl.from_bf16_bits(fx["n_norm_only"])
    assert np.all(np.abs(wl.from_bf16_bits(norm_only) - b) <= ol.bf16_ulp(b))
    codes, scales = ol.nvfp4_quantize_bf16(fx["n_norm"], float(fx["n_G"]))         # quantizer on the reference's norm
    assert np.array_equal(codes, fx["n_codes"]) and np.array_equal(scales, fx["n_scales"])


def test_add_bf16_bit_exact(fx):
    assert np.array_equal(ol.add_bf16(fx["a_a"], fx["a_b"]), fx["a_out"])


def test_fp8_quantizers_bit_exact(fx):
    codes, scales = ol.fp8_quantize_f32(wl.from_bf16_bits(fx["f_in"]))
    assert np.array_equal(codes, fx["f_codes"]) and np.array_equal(scales, fx["f_scales"])
    codes, scales, status = ol.fp8_quantize_bf16(fx["f2_in"])
    assert np.array_equal(codes, fx["f2_codes"]) and np.array_equal(scales, fx["f2_scales"])
    assert status == int(fx["f2_status"]) == 4


def test_swiglu(fx):
    y = ol.swiglu_f32(fx["s_in"])
    ref = fx["s_y"]
    assert np.all(np.abs(y - ref) <= 4 * np.spacing(np.abs(ref)) + 1e-45)           # device expf: <= 4 FP32 ulp on y
    assert np.array_equal(y[0, :2].view(np.uint32), ref[0, :2].view(np.uint32))    # silu(+-0) * u keeps its sign
    codes, scales = ol.swiglu_fp8_bf16(fx["s_in"])
    assert np.all(np.abs(scales - fx["s_fp8_scales"]) <= 4 * np.spacing(fx["s_fp8_scales"]))
    assert np.mean(codes != fx["s_fp8_codes"]) < 2e-3
    codes, scales = ol.fp8_quantize_f32(ref)                                        # quantizer on the reference's y
    assert np.array_equal(codes, fx["s_fp8_codes"]) and np.array_equal(scales, fx["s_fp8_scales"])
    codes, scales = ol.nvfp4_quantize_f32(ref, float(fx["s_G"]))
    assert np.array_equal(codes, fx["s_nv_codes"]) and np.array_equal(ol.scales_to_tiled(scales), fx["s_nv_plane"])


def test_yarn_table_and_qk_norm_rope(fx):
    inv = ol.yarn_inv_freq(1e7, 4.0, 262144.0, 32.0, 1.0, 64)
    assert np.allclose(inv, fx["y_inv_freq"], rtol=4e-7, atol=0)                    # powf: a couple of FP32 ulp
    mscale = float(np.float32(1.138629436111989))
    for tag in ("lo", "hi"):
        base = int(fx[f"k_{tag}_base"])
        pos = (base + np.arange(8)).astype(np.uint32)
        q_out, k_out, _ = ol.qk_norm_rope_paged(fx[f"k_{tag}_q"], fx[f"k_{tag}_k"], None, fx[f"k_{tag}_qg"], fx[f"k_{tag}_kg"],
                                                fx["y_inv_freq"], pos, None, rope_dim=64, eps=1e-6, mscale=mscale, want_k_out=True)
        for got, want in ((q_out, fx[f"k_{tag}_q_out"]), (k_out, fx[f"k_{tag}_k_out"])):
            assert np.array_equal(got[..., 64:], want[..., 64:])                    # pass-through dims: bit-exact
            a, b = wl.from_bf16_bits(got), wl.from_bf16_bits(want)
            assert np.all(np.abs(a - b) <= 2 * ol.bf16_ulp(np.maximum(np.abs(b), 0.25)))
            assert np.mean(got != want) < 0.01


def test_e4m3_cache_rows_bit_exact(fx):
    """The reference's E4M3 (scale 1) cache rows are the saturating codes of its own rotated BF16 K rows."""
    for tag in ("lo", "hi"):
        want = fx[f"k_{tag}_k_e4m3"].reshape(-1)
        assert np.array_equal(ol.bf16_to_e4m3_scale1(fx[f"k_{tag}_k_out"]).reshape(-1), want)


def test_sigmoid_gate(fx):
    got, _, _ = ol.sigmoid_gate_nvfp4_bf16(fx["sg_attention"], fx["sg_gate"], 1.0)
    a, b = wl.from_bf16_bits(got), wl.from_bf16_bits(fx["sg_out"])
    assert np.array_equal(np.isnan(a), np.isnan(b))
    ok = ~np.isnan(b)
    assert np.all(np.abs(a[ok] - b[ok]) <= ol.bf16_ulp(np.abs(b[ok])) * np.float32(1.01))  # libm vs device expf
    assert np.mean(got != fx["sg_out"]) < 2e-3


def test_generic_f32_ops(fx):
    x, w = fx["g_x"], fx["g_w"]
    for tag, tol in (("plain", 1e-3), ("hp", 2e-6), ("b1", 1e-3)):                  # fast-math unit: reference tolerance 1e-3
        assert np.allclose(ol.rmsnorm_f32(w, x, 1e-6, tag), fx[f"g_rmsnorm_{tag}"], rtol=tol, atol=tol * 1e-2)
    assert np.allclose(ol.head_rmsnorm_f32(fx["g_hx"], 7, 128, 1e-6), fx["g_head_rmsnorm"], rtol=1e-3, atol=1e-5)
    assert np.allclose(ol.qk_rmsnorm_w_f32(fx["g_hx"], fx["g_hw"], 7, 128, 1e-6), fx["g_qk_rmsnorm_w"], rtol=2e-6, atol=0)
    for pos in (5, 4097):
        assert np.allclose(ol.qknorm_rope_f32(fx["g_hx"], fx["g_hw"], 7, 128, pos, 1e6, 1e-6), fx[f"g_qknorm_rope_{pos}"],
                           rtol=0, atol=3e-5 + 2e-6 * pos)
        assert np.allclose(ol.rope_neox_f32(fx["g_hx"], 7, 128, 64, pos, 1e4), fx[f"g_rope_partial_{pos}"],
                           rtol=0, atol=3e-5 + 2e-6 * pos)
    assert np.array_equal(ol.add_f32(fx["g_a"], fx["g_b"]), fx["g_add"])
    assert np.allclose(ol.silu_mul_f32(fx["g_a"], fx["g_b"]), fx["g_silu_mul"], rtol=1e-3, atol=1e-5)
    assert np.allclose(ol.silu_mul_f32(fx["g_a"], fx["g_b"], 3.0), fx["g_silu_mul_clamp3"], rtol=1e-3, atol=1e-5)


def test_round_after_norm_convention(fx):
    """The draft's q/k convention against the reference kernel's output: the rotary table rows are inputs of both
    sides; the oracle's inverse square root is the C library's, so three BF16 ulps at the operands' magnitude."""
    first = int(fx["d_first"])
    table = np.zeros((first + 8, 128), np.float32)
    table[first:] = fx["d_table_rows"]
    positions = (first + np.arange(8)).astype(np.uint32)
    got, status = ol.qk_norm_rope_round_after_norm(fx["d_q"], fx["d_gamma"], table, positions)
    assert status == 0
    a, b = wl.from_bf16_bits(got), wl.from_bf16_bits(fx["d_out"])
    x = wl.from_bf16_bits(fx["d_q"]).astype(np.float64)
    n = np.abs(x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6)) * 1.2     # |normalised operand| * gamma * mscale, roughly
    mag = np.maximum(n[..., :64], n[..., 64:])
    bound = 3 * ol.bf16_ulp(np.concatenate([mag, mag], axis=-1).astype(np.float32) * np.float32(1.2))
    assert np.all(np.abs(a - b) <= bound)
    assert np.mean(got != fx["d_out"]) < 0.05


def test_static_scale_fp8_bit_exact(fx):
    codes = ol.fp8_quantize_static_f32(wl.from_bf16_bits(fx["fs_in"]), float(fx["fs_scale"]))
    assert np.array_equal(codes, fx["fs_codes"])

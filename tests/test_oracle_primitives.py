"""Pins the oracle's scalar encoders against the CUDA toolkit's host converters
and against the closed-form cases the reference's own tests hold."""
import ctypes as C
import math

import numpy as np

import oracle_lib as ol


def _sweep_values():
    rng = np.random.default_rng(1234)
    parts = [
        rng.standard_normal(200_000).astype(np.float32) * np.float32(3.0),
        (rng.standard_normal(100_000) * 200).astype(np.float32),
        np.exp(rng.uniform(-30, 10, 100_000)).astype(np.float32) * rng.choice([-1, 1], 100_000).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 448.0, 464.0, 480.0, -448.0, 2.0 ** -9, 2.0 ** -10,
                  1.5 * 2.0 ** -10, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25, -5.0], np.float32),
    ]
    # every E4M3 value, every midpoint between neighbours, and their float neighbours
    grid = np.array([ol.o().axo_e4m3_decode(c) for c in range(0x7f)], np.float32)
    mids = (grid[:-1] + grid[1:]) / np.float32(2)
    edge = np.concatenate([grid, mids])
    parts += [edge, np.nextafter(edge, np.float32(np.inf)), np.nextafter(edge, np.float32(-np.inf))]
    v = np.concatenate(parts).astype(np.float32)
    return np.concatenate([v, -v])


def test_e4m3_encoder_matches_toolkit_host_path():
    v = _sweep_values()
    want = np.empty(v.size, np.uint8)
    ol.pin().pin_e4m3_satfinite_many(v.ctypes.data_as(C.c_void_p), want.ctypes.data_as(C.c_void_p), C.c_uint64(v.size))
    got = np.array([ol.o().axo_e4m3_encode_satfinite(float(x)) for x in v], np.uint8)
    assert np.array_equal(got, want)


def test_e2m1_encoder_matches_toolkit_host_path():
    v = _sweep_values()
    want = np.empty(v.size, np.uint8)
    ol.pin().pin_e2m1_rn_many(v.ctypes.data_as(C.c_void_p), want.ctypes.data_as(C.c_void_p), C.c_uint64(v.size))
    got = np.array([ol.o().axo_e2m1_encode(float(x)) for x in v], np.uint8)
    assert np.array_equal(got & 0xF, want & 0xF)


def test_e2m1_ties_and_table():
    # tests/axiom_nvfp4_smoke.cpp:34-39 (value table) and the tie cases of cuda_fp4.hpp
    assert [ol.o().axo_e2m1_decode(c) for c in range(8)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    ties = {0.25: 0.0, 0.75: 1.0, 1.25: 1.0, 1.75: 2.0, 2.5: 2.0, 3.5: 4.0, 5.0: 4.0, 7.0: 6.0}
    for x, want in ties.items():
        assert ol.o().axo_e2m1_decode(ol.o().axo_e2m1_encode(x)) == want
        assert ol.o().axo_e2m1_decode(ol.o().axo_e2m1_encode(-x)) == -want


def test_e4m3_known_codes():
    # tests/axiom_nvfp4_smoke.cpp:202 — 0x38=1.0, 0x30=0.5, 0x40=2.0, 0x3c=1.5
    for code, value in {0x38: 1.0, 0x30: 0.5, 0x40: 2.0, 0x3c: 1.5, 0x7e: 448.0, 0x01: 2.0 ** -9, 0x20: 0.125}.items():
        assert ol.o().axo_e4m3_decode(code) == value
        assert ol.o().axo_e4m3_encode_satfinite(value) == code
    assert math.isnan(ol.o().axo_e4m3_decode(0x7f)) and math.isnan(ol.o().axo_e4m3_decode(0xff))
    assert ol.o().axo_e4m3_encode_scale(0.0) == 0x20  # zero-scale guard
    assert ol.o().axo_e4m3_encode_scale(float("nan")) == 0x7e
    assert ol.o().axo_e4m3_encode_scale(1e9) == 0x7e


def test_bf16_round_matches_numpy_and_ties():
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.standard_normal(50_000).astype(np.float32),
                        np.array([1.0 + 2 ** -8, 1.0 + 3 * 2 ** -8, 3.3895314e38, -0.0, 1e-40], np.float32)])
    got = np.array([ol.o().axo_f32_to_bf16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, ol.f32_to_bf16_bits(x))
    assert ol.o().axo_bf16_round(1.0 + 2 ** -8) == 1.0            # tie to even (down)
    assert ol.o().axo_bf16_round(1.0 + 3 * 2 ** -8) == 1.0 + 2 ** -6  # tie to even (up)
    assert ol.o().axo_f32_to_bf16(float("nan")) == 0x7fff


def test_rmsnorm_known_answer():
    # tests/axiom_quant_smoke.cpp:108-123 — {1,2,3,4}, w=1, eps=1e-6 -> x/sqrt(7.5+1e-6), tol 1e-3
    x = np.array([1, 2, 3, 4], np.float32)
    w = np.ones(4, np.float32)
    want = x / math.sqrt(7.5 + 1e-6)
    for variant in ("plain", "hp", "b1"):
        assert np.allclose(ol.rmsnorm_f32(w, x, 1e-6, variant), want, atol=1e-3)
    # tests/axiom_safetensors_smoke.cpp:166-191 — {1,2,3} scaled by w={1,.5,2}? only the first vector is closed form
    x3 = np.array([1, 2, 3], np.float32)
    got = ol.rmsnorm_f32(np.ones(3, np.float32), x3, 1e-6, "hp")
    assert np.allclose(got, x3 / math.sqrt(14.0 / 3.0 + 1e-6), atol=1e-6)


def test_silu_mul_known_answer():
    # tests/axiom_safetensors_smoke.cpp:234-244 — gate {0,1,-1}, up 2 -> {0, 1.4621.., -0.5378..}
    got = ol.silu_mul_f32(np.array([0, 1, -1], np.float32), np.full(3, 2, np.float32))
    assert np.allclose(got, [0.0, 1.4621172, -0.5378828], atol=1e-6)


def test_qknorm_rope_analytic_case():
    # tests/qwen4exp/qsa_test.cpp style: with cos=0, sin=1 the pair (a, b) maps to (-b, a).
    # theta chosen so pair 0 has angle pi/2 at pos 1 is not expressible; use pos=0 (identity rotation) and
    # check the norm, then a hand-rolled rotation.
    head_dim = 8
    x = np.arange(1, head_dim + 1, dtype=np.float32)
    w = np.full(head_dim, 0.5, np.float32)
    got = ol.qknorm_rope_f32(x, w, 1, head_dim, 0, 10000.0, 1e-6)
    inv = 1.0 / math.sqrt(float(np.mean(x.astype(np.float64) ** 2)) + 1e-6)
    assert np.allclose(got, x * inv * 0.5, rtol=1e-6)
    pos = 3
    got = ol.qknorm_rope_f32(x, w, 1, head_dim, pos, 10000.0, 1e-6)
    n = x.astype(np.float64) * inv * 0.5
    half = head_dim // 2
    want = np.empty(head_dim)
    for i in range(half):
        ang = pos * 10000.0 ** (-2.0 * i / head_dim)
        want[i] = n[i] * math.cos(ang) - n[i + half] * math.sin(ang)
        want[i + half] = n[i] * math.sin(ang) + n[i + half] * math.cos(ang)
    assert np.allclose(got, want, rtol=2e-5, atol=2e-6)


def test_scale_plane_tiled_layout_formula():
    # src/axiom_qwen38_nvfp4_mlp.cu:101-108 evaluated by hand for a few cells
    assert ol.o().axo_scale_tiled_bytes(4096, 320) == 32 * 80 * 512
    assert ol.o().axo_scale_tiled_bytes(1, 1) == 512
    inner_tiles = 80
    assert ol.o().axo_scale_tiled_offset(0, 0, inner_tiles) == 0
    assert ol.o().axo_scale_tiled_offset(1, 0, inner_tiles) == 16
    assert ol.o().axo_scale_tiled_offset(32, 0, inner_tiles) == 4
    assert ol.o().axo_scale_tiled_offset(0, 5, inner_tiles) == 512 + 1
    assert ol.o().axo_scale_tiled_offset(128, 0, inner_tiles) == 80 * 512
    canonical = np.arange(130 * 6, dtype=np.uint32).astype(np.uint8).reshape(130, 6)
    tiled = ol.scales_to_tiled(canonical)
    assert tiled.size == 2 * 2 * 512
    for r, g in [(0, 0), (5, 3), (33, 4), (129, 5)]:
        assert tiled[ol.o().axo_scale_tiled_offset(r, g, 2)] == canonical[r, g]
    assert int(tiled.astype(np.int64).sum()) == int(canonical.astype(np.int64).sum())  # padding is zero


def test_nvfp4_group_semantics():
    # zero block -> scale 0x20, codes 0; saturating block scale; (max/6)*G then e4m3
    x = np.zeros((1, 32), np.float32)
    x[0, 16:] = np.array([6, -6, 3, 1.5, 0.5, 0.25, 0.75, -0.75, 0, 0, 0, 0, 0, 0, 0, 4], np.float32)
    codes, scales = ol.nvfp4_quantize_f32(x, 1.0)
    assert scales[0, 0] == 0x20 and not codes[0, :8].any()
    assert scales[0, 1] == 0x38  # max 6 -> (6/6)*1 = 1.0
    want = [6, -6, 3, 1.5, 0.5, 0.0, 1.0, -1.0, 0, 0, 0, 0, 0, 0, 0, 4]  # 0.25 -> 0 and 0.75 -> 1.0 (ties to even)
    got = []
    for b in codes[0, 8:]:
        got += [ol.o().axo_e2m1_decode(int(b) & 0xF), ol.o().axo_e2m1_decode(int(b) >> 4)]
    assert got == want
    big = np.full((1, 16), 1e6, np.float32)
    _, s = ol.nvfp4_quantize_f32(big, 1.0)
    assert s[0, 0] == 0x7e


def test_fp8_row_semantics():
    x = np.array([[0.0, 0.0, 0.0, 0.0], [448.0, -224.0, 1.0, 0.0]], np.float32)
    codes, scales = ol.fp8_quantize_f32(x)
    assert scales[0] == 1.0 and not codes[0].any()  # zero row -> scale 1
    assert scales[1] == 1.0
    assert list(codes[1]) == [0x7e, 0xf6, 0x38, 0x00]


def test_yarn_frequencies_flavours_agree_and_ramp():
    for theta, ctx, dim in [(1e6, 32768.0, 128), (1e7, 262144.0, 64)]:
        dev = ol.yarn_inv_freq(theta, 4.0, ctx, 32.0, 1.0, dim)
        host = ol.yarn_inv_freq(theta, 4.0, ctx, 32.0, 1.0, dim, host_table=True)
        plain = ol.yarn_inv_freq(theta, 1.0, ctx, 32.0, 1.0, dim)
        assert np.allclose(dev, host, rtol=3e-6)
        assert dev[0] == 1.0                       # high frequencies untouched
        assert np.isclose(dev[-1], plain[-1] / 4)  # low frequencies interpolated by the factor
        assert np.all(dev <= plain * (1 + 1e-6)) and np.all(dev >= plain / 4 * (1 - 1e-6))
    assert abs(ol.o().axo_yarn_mscale(4.0) - 1.138629436111989) < 1e-7  # include/axiom/qwen38_attention.h:29


def test_top1_rule():
    """Largest finite value, smallest id among equals, invalid flag (reference src/axiom_qwen38_model.cu:483-493)."""
    x = np.array([[1.0, 5.0, 5.0, -2.0], [np.nan, -1.0, np.inf, -3.0], [np.nan, np.nan, np.nan, np.nan]], np.float32)
    out = ol.top1_f32(x)
    assert out[0, 1] == 1 and out[0, 2] == 0 and out[0, 0] == np.float32(5.0).view(np.uint32)
    assert out[1, 1] == 1 and out[1, 2] == 1 and out[1, 0] == np.float32(-1.0).view(np.uint32)
    assert out[2, 1] == 0xFFFFFFFF and out[2, 2] == 1 and out[2, 0] == np.float32(-np.inf).view(np.uint32)


def test_q8_0_and_f16_gathers():
    import struct

    blk = bytearray(34 * 2)
    blk[0:2] = struct.pack("<e", 0.5)
    blk[2:34] = bytes((i - 16) & 0xFF for i in range(32))
    blk[34:36] = struct.pack("<e", -2.0)
    blk[36:68] = bytes([3] * 32)
    table = np.frombuffer(bytes(blk), np.uint8)
    got = ol.q8_0_embedding_gather_f32(table, 0, 1, 64)
    assert np.array_equal(got[:32], 0.5 * (np.arange(32) - 16)) and np.array_equal(got[32:], np.full(32, -6.0, np.float32))
    assert not ol.q8_0_embedding_gather_f32(table, 1, 1, 64).any()  # id beyond the table: zeros
    h = np.array([0.0, 1.5, -65504.0, 6e-8], np.float16)
    out = ol.f16_embedding_streams_f32(h.view(np.uint16), 0, 4, 3)
    assert np.array_equal(out.reshape(3, 4), np.tile(h.astype(np.float32), (3, 1)))

"""Runtime / device-buffer handles, the axiom_device_buffer and host-I/O flavours of the fused ops,
and the generic single-row F32 ops of the runtime ABI."""
import ctypes as C
import importlib
import math
import os

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


@pytest.fixture()
def rt(axk, cuda_device):
    r = axk.Runtime(0)
    yield r
    r.close()


def buf_from(axk, rt, array):
    b = axk.DeviceBuffer(rt, max(array.nbytes, 1))
    assert b.upload(np.ascontiguousarray(array)) == axk.AXIOM_OK
    return b


def test_runtime_and_buffer_lifecycle(axk, rt):
    lib = axk.lib()
    n = C.c_uint32(0)
    assert lib.axiom_runtime_device_count(C.byref(n)) == axk.AXIOM_OK and n.value >= 1
    d = C.c_uint32(99)
    assert lib.axiom_runtime_device_id(rt.handle, C.byref(d)) == axk.AXIOM_OK and d.value == 0
    data = np.arange(1024, dtype=np.uint8)
    a = buf_from(axk, rt, data)
    b = axk.DeviceBuffer(rt, 2048)
    assert lib.axiom_device_buffer_copy(b.handle, 512, a.handle, 0, 1024) == axk.AXIOM_OK
    back = np.zeros(1024, np.uint8)
    assert b.download(back, 512) == axk.AXIOM_OK and np.array_equal(back, data)
    # span checks (src/axiom_runtime.cpp:3224-3247 in the reference): offset + bytes must stay inside
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert b.download(back, 1025) == inv
    assert a.upload(data, 1) == inv
    assert lib.axiom_device_buffer_copy(b.handle, 1025, a.handle, 0, 1024) == inv
    assert lib.axiom_device_buffer_copy(b.handle, 0, a.handle, 0, 0) == inv
    assert lib.axiom_device_buffer_upload(a.handle, 0, None, 4) == inv
    assert a.cuda_pointer() != 0
    d.value = 99
    assert lib.axiom_device_buffer_device_id(a.handle, C.byref(d)) == axk.AXIOM_OK and d.value == 0
    out = C.c_void_p(1)
    assert lib.axiom_device_buffer_create(rt.handle, C.byref(out), 0) == inv
    with pytest.raises(axk.AxiomError):
        axk.Runtime(device=77)
    a.close(); b.close()
    lib.axiom_device_buffer_destroy(None)
    lib.axiom_runtime_destroy(None)


def test_buffer_flavour_nvfp4_quantize(axk, rt):
    x = wl.quantize_input_np(96, 5120, seed=2)
    G = 200.0
    xin = buf_from(axk, rt, x)
    codes = axk.DeviceBuffer(rt, 96 * 2560 + 64)
    scales = axk.DeviceBuffer(rt, 96 * 320)
    lib = axk.lib()
    rc = lib.axiom_runtime_nvfp4_quantize_bf16_device(rt.handle, xin.handle, 0, 96, 5120, G, codes.handle, 64,
                                                      scales.handle, 0, 0)
    assert rc == axk.AXIOM_OK  # synchronous by default (finish-after-launch)
    got_codes = np.empty((96, 2560), np.uint8); got_scales = np.empty((96, 320), np.uint8)
    codes.download(got_codes, 64); scales.download(got_scales)
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    assert np.array_equal(got_codes, want_codes) and np.array_equal(got_scales, want_scales)
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    # span / alias / ownership failures
    assert lib.axiom_runtime_nvfp4_quantize_bf16_device(rt.handle, xin.handle, 0, 97, 5120, G, codes.handle, 64, scales.handle, 0, 0) == inv
    assert lib.axiom_runtime_nvfp4_quantize_bf16_device(rt.handle, xin.handle, 0, 96, 5120, G, codes.handle, 128, scales.handle, 0, 0) == inv
    assert lib.axiom_runtime_nvfp4_quantize_bf16_device(rt.handle, xin.handle, 0, 8, 64, G, xin.handle, 0, scales.handle, 0, 0) == inv
    other = axk.Runtime(0)
    foreign = axk.DeviceBuffer(other, 96 * 320)
    assert lib.axiom_runtime_nvfp4_quantize_bf16_device(rt.handle, xin.handle, 0, 96, 5120, G, codes.handle, 64, foreign.handle, 0, 0) == inv
    foreign.close(); other.close()
    for b in (xin, codes, scales):
        b.close()


def test_buffer_flavour_fused_ops(axk, rt):
    lib = axk.lib()
    rows, cols = 40, 5120
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    h, r, g = buf_from(axk, rt, hidden), buf_from(axk, rt, residual), buf_from(axk, rt, gamma)
    norm = axk.DeviceBuffer(rt, rows * cols * 2)
    codes = axk.DeviceBuffer(rt, rows * cols // 2)
    scales = axk.DeviceBuffer(rt, rows * cols // 16)
    G = 120.0
    rc = lib.axiom_runtime_add_rmsnorm_nvfp4_bf16_device(rt.handle, h.handle, 0, r.handle, 0, g.handle, 0, 1e-6, rows, cols,
                                                         G, norm.handle, 0, codes.handle, 0, scales.handle, 0, 0)
    assert rc == axk.AXIOM_OK
    got_res = np.empty((rows, cols), np.uint16); got_norm = np.empty((rows, cols), np.uint16)
    got_codes = np.empty((rows, cols // 2), np.uint8)
    r.download(got_res); norm.download(got_norm); codes.download(got_codes)
    want_res, want_norm = ol.add_rmsnorm_bf16(hidden, residual, gamma, 1e-6)
    assert np.array_equal(got_res, want_res)
    assert np.all(np.abs(wl.from_bf16_bits(got_norm) - wl.from_bf16_bits(want_norm)) <= ol.bf16_ulp(wl.from_bf16_bits(want_norm)))
    assert np.array_equal(got_codes, ol.nvfp4_quantize_bf16(got_norm, G)[0])
    # hidden aliasing residual is rejected
    assert lib.axiom_runtime_add_rmsnorm_nvfp4_bf16_device(rt.handle, r.handle, 0, r.handle, 0, g.handle, 0, 1e-6, rows, cols, G,
                                                           norm.handle, 0, codes.handle, 0, scales.handle, 0, 0) == axk.AXIOM_ERR_INVALID_ARGUMENT

    gu = wl.swiglu_input_np(12, 1024)
    gub = buf_from(axk, rt, gu)
    c8 = axk.DeviceBuffer(rt, 12 * 1024); s8 = axk.DeviceBuffer(rt, 12 * 4)
    assert lib.axiom_runtime_swiglu_fp8_bf16_device(rt.handle, gub.handle, 0, 12, 1024, c8.handle, 0, s8.handle, 0) == axk.AXIOM_OK
    got = np.empty((12, 1024), np.uint8); c8.download(got)
    assert np.mean(got != ol.swiglu_fp8_bf16(gu)[0]) < 5e-3
    c4 = axk.DeviceBuffer(rt, 12 * 512); s4 = axk.DeviceBuffer(rt, 12 * 64)
    assert lib.axiom_runtime_swiglu_nvfp4_bf16_device(rt.handle, gub.handle, 0, 12, 1024, 50.0, c4.handle, 0, s4.handle, 0, 0) == axk.AXIOM_OK
    got4 = np.empty((12, 512), np.uint8); c4.download(got4)
    assert np.mean(got4 != ol.swiglu_nvfp4_bf16(gu, 50.0)[0]) < 5e-3

    table, ids = wl.embedding_inputs_np(17, vocab=300, hidden=256)
    tb, ib = buf_from(axk, rt, table), buf_from(axk, rt, ids)
    ob = axk.DeviceBuffer(rt, 17 * 256 * 2)
    assert lib.axiom_runtime_embedding_gather_bf16_device(rt.handle, tb.handle, 0, 300, 256, ib.handle, 0, 17, ob.handle, 0) == axk.AXIOM_OK
    got = np.empty((17, 256), np.uint16); ob.download(got)
    assert np.array_equal(got, ol.embedding_gather_bf16(table, ids))


def test_host_io_flavour(axk, rt):
    """Host pointers in, host pointers out; rows stream through the runtime's staging slots in chunks."""
    lib = axk.lib()
    rows, cols = 3000, 5120  # several 16 MiB chunks
    x = wl.quantize_input_np(rows, cols, seed=8)
    G = 300.0
    codes = np.zeros((rows, cols // 2), np.uint8); scales = np.zeros((rows, cols // 16), np.uint8)
    rc = lib.axiom_runtime_nvfp4_quantize_bf16(rt.handle, x.ctypes.data, rows, cols, G, codes.ctypes.data, scales.ctypes.data)
    assert rc == axk.AXIOM_OK
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    assert np.array_equal(codes, want_codes) and np.array_equal(scales, want_scales)

    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(1500, cols)
    res_io = residual.copy()
    codes = np.zeros((1500, cols // 2), np.uint8); scales = np.zeros((1500, cols // 16), np.uint8)
    rc = lib.axiom_runtime_add_rmsnorm_nvfp4_bf16(rt.handle, hidden.ctypes.data, res_io.ctypes.data, gamma.ctypes.data,
                                                  1e-6, 1500, cols, G, codes.ctypes.data, scales.ctypes.data)
    assert rc == axk.AXIOM_OK
    want_res, _, want_codes, _ = ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
    assert np.array_equal(res_io, want_res)
    assert np.mean(codes != want_codes) < 0.02

    gu = wl.swiglu_input_np(700, 17408)
    c8 = np.zeros((700, 17408), np.uint8); s8 = np.zeros(700, np.float32)
    assert lib.axiom_runtime_swiglu_fp8_bf16(rt.handle, gu.ctypes.data, 700, 17408, c8.ctypes.data, s8.ctypes.data) == axk.AXIOM_OK
    want_c8, want_s8 = ol.swiglu_fp8_bf16(gu)
    assert np.allclose(s8, want_s8, rtol=1e-6) and np.mean(c8 != want_c8) < 2e-3


@pytest.mark.parametrize("rows", [40, 1500])
def test_host_io_with_page_locked_buffers_matches_staged_path(axk, rt, rows):
    """Page-locked (mapped) host buffers are read and written by the kernel itself, pageable ones go through the
    staging slots: both give the same bytes, and a mix of the two kinds takes the staged path."""
    import torch

    lib = axk.lib()
    cols, G = 5120, 300.0
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)

    def run(pin_in, pin_out):
        def place(a, pin):
            t = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).clone()
            return t.pin_memory() if pin else t
        h, r = place(hidden, pin_in), place(residual, pin_in)
        c = place(np.zeros((rows, cols // 2), np.uint8), pin_out)
        sc = place(np.zeros((rows, cols // 16), np.uint8), pin_out)
        rc = lib.axiom_runtime_add_rmsnorm_nvfp4_bf16(rt.handle, h.data_ptr(), r.data_ptr(), gamma.ctypes.data, 1e-6, rows,
                                                      cols, G, c.data_ptr(), sc.data_ptr())
        assert rc == axk.AXIOM_OK
        return r.numpy().view(np.uint16).copy(), c.numpy().copy(), sc.numpy().copy()

    staged, direct, mixed = run(False, False), run(True, True), run(True, False)
    os.environ["AXIOM_B200_HOST_IO"] = "staged"  # the knob that keeps page-locked buffers on the staged path
    try:
        forced = run(True, True)
    finally:
        del os.environ["AXIOM_B200_HOST_IO"]
    for a, b, c, f in zip(staged, direct, mixed, forced):
        assert np.array_equal(a, b) and np.array_equal(a, c) and np.array_equal(a, f)
    want_res, _, want_codes, want_scales = ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
    assert np.array_equal(direct[0], want_res)
    assert np.mean(direct[1] != want_codes) < 0.02
    assert lib.axiom_b200_pipeline_faults(0) == 0


def test_host_io_quantize_and_swiglu_with_page_locked_buffers(axk, rt):
    import torch

    lib = axk.lib()
    rows, cols, G = 700, 5120, 300.0
    x = torch.from_numpy(wl.quantize_input_np(rows, cols, seed=4).view(np.int16)).pin_memory()
    codes = torch.zeros((rows, cols // 2), dtype=torch.uint8).pin_memory()
    scales = torch.zeros((rows, cols // 16), dtype=torch.uint8).pin_memory()
    assert lib.axiom_runtime_nvfp4_quantize_bf16(rt.handle, x.data_ptr(), rows, cols, G, codes.data_ptr(), scales.data_ptr()) == axk.AXIOM_OK
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x.numpy().view(np.uint16), G)
    assert np.array_equal(codes.numpy(), want_codes) and np.array_equal(scales.numpy(), want_scales)

    gu_np = wl.swiglu_input_np(300, 17408)
    gu = torch.from_numpy(gu_np.view(np.int16)).pin_memory()
    c8 = torch.zeros((300, 17408), dtype=torch.uint8).pin_memory()
    s8 = torch.zeros(300, dtype=torch.float32).pin_memory()
    assert lib.axiom_runtime_swiglu_fp8_bf16(rt.handle, gu.data_ptr(), 300, 17408, c8.data_ptr(), s8.data_ptr()) == axk.AXIOM_OK
    c8_staged = np.zeros((300, 17408), np.uint8); s8_staged = np.zeros(300, np.float32)
    assert lib.axiom_runtime_swiglu_fp8_bf16(rt.handle, gu_np.ctypes.data, 300, 17408, c8_staged.ctypes.data, s8_staged.ctypes.data) == axk.AXIOM_OK
    assert np.array_equal(c8.numpy(), c8_staged) and np.array_equal(s8.numpy(), s8_staged)


def f32buf(axk, rt, a):
    return buf_from(axk, rt, np.ascontiguousarray(a, np.float32))


def test_generic_f32_norms(axk, rt):
    lib = axk.lib()
    rng = np.random.default_rng(0)
    for count in (4, 5120, 4096 + 3):
        x = rng.standard_normal(count).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(count)).astype(np.float32)
        if count == 4:
            x = np.array([1, 2, 3, 4], np.float32); w = np.ones(4, np.float32)  # tests/axiom_quant_smoke.cpp:108-123
        xb, wb = f32buf(axk, rt, x), f32buf(axk, rt, w)
        for name, variant, tol in (("axiom_runtime_rmsnorm_f32_device", "plain", 1e-3),
                                   ("axiom_runtime_rmsnorm_f32_hp_device", "hp", 2e-6),
                                   ("axiom_runtime_rmsnorm_f32_b1_device", "b1", 1e-3)):
            ob = axk.DeviceBuffer(rt, count * 4)
            assert getattr(lib, name)(rt.handle, wb.handle, 0, xb.handle, 0, ob.handle, 0, count, 0.0) == axk.AXIOM_OK
            got = np.empty(count, np.float32); ob.download(got)
            assert np.allclose(got, ol.rmsnorm_f32(w, x, 1e-6, variant), rtol=tol, atol=tol * 1e-2)  # eps<=0 -> 1e-6
        x1 = rng.standard_normal(count).astype(np.float32)
        x1b = f32buf(axk, rt, x1)
        o0, o1 = axk.DeviceBuffer(rt, count * 4), axk.DeviceBuffer(rt, count * 4)
        assert lib.axiom_runtime_rmsnorm_f32_dual_device(rt.handle, wb.handle, 0, xb.handle, 0, o0.handle, 0, x1b.handle, 0,
                                                         o1.handle, 0, count, 1e-6) == axk.AXIOM_OK
        g0 = np.empty(count, np.float32); g1 = np.empty(count, np.float32); o0.download(g0); o1.download(g1)
        assert np.allclose(g0, ol.rmsnorm_f32(w, x, 1e-6), rtol=1e-3) and np.allclose(g1, ol.rmsnorm_f32(w, x1, 1e-6), rtol=1e-3)
    heads, hd = 6, 128
    x = rng.standard_normal(heads * hd).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    xb = f32buf(axk, rt, x)
    assert lib.axiom_runtime_head_rmsnorm_f32_device(rt.handle, xb.handle, 0, heads, hd, 1e-6) == axk.AXIOM_OK
    got = np.empty_like(x); xb.download(got)
    assert np.allclose(got, ol.head_rmsnorm_f32(x, heads, hd, 1e-6), rtol=1e-3)
    xb, wb = f32buf(axk, rt, x), f32buf(axk, rt, w)
    assert lib.axiom_runtime_qk_rmsnorm_w_f32_device(rt.handle, xb.handle, 0, wb.handle, 0, heads, hd, 1e-6) == axk.AXIOM_OK
    xb.download(got)
    assert np.allclose(got, ol.qk_rmsnorm_w_f32(x, w, heads, hd, 1e-6), rtol=2e-6)
    assert lib.axiom_runtime_head_rmsnorm_f32_device(rt.handle, xb.handle, 0, heads, hd, 0.0) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_runtime_head_rmsnorm_f32_device(rt.handle, xb.handle, 4, heads, hd, 1e-6) == axk.AXIOM_ERR_INVALID_ARGUMENT


def test_generic_f32_rope_and_qknorm(axk, rt):
    lib = axk.lib()
    rng = np.random.default_rng(1)
    heads, hd = 5, 128
    x = rng.standard_normal(heads * hd).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    for pos in (0, 1, 1024, 70000):
        xb = f32buf(axk, rt, x)
        assert lib.axiom_runtime_rope_neox_f32_device(rt.handle, xb.handle, 0, heads, hd, pos, 1e6) == axk.AXIOM_OK
        got = np.empty_like(x); xb.download(got)
        assert np.allclose(got, ol.rope_neox_f32(x, heads, hd, hd, pos, 1e6), rtol=0, atol=2e-5 + 2e-6 * pos)
        xb = f32buf(axk, rt, x)
        assert lib.axiom_runtime_rope_neox_partial_f32_device(rt.handle, xb.handle, 0, heads, hd, 64, pos, 1e4) == axk.AXIOM_OK
        xb.download(got)
        want = ol.rope_neox_f32(x, heads, hd, 64, pos, 1e4)
        assert np.allclose(got, want, rtol=0, atol=2e-5 + 2e-6 * pos)
        assert np.array_equal(got.reshape(heads, hd)[:, 64:], x.reshape(heads, hd)[:, 64:])  # pass-through untouched
        xb, wb = f32buf(axk, rt, x), f32buf(axk, rt, w)
        assert lib.axiom_runtime_qknorm_rope_f32_device(rt.handle, xb.handle, 0, wb.handle, 0, heads, hd, pos, 1e6, 1e-6) == axk.AXIOM_OK
        xb.download(got)
        want = ol.qknorm_rope_f32(x, w, heads, hd, pos, 1e6, 1e-6)
        assert np.allclose(got, want, rtol=0, atol=3e-5 + 2e-6 * pos)
        # device-position and dual flavours give the same bits as the scalar-position one
        pb = buf_from(axk, rt, np.array([pos], np.uint32))
        xb2 = f32buf(axk, rt, x)
        assert lib.axiom_runtime_qknorm_rope_pos_f32_device(rt.handle, xb2.handle, 0, wb.handle, 0, pb.handle, 0, heads, hd, 1e6, 1e-6) == axk.AXIOM_OK
        got2 = np.empty_like(x); xb2.download(got2)
        assert np.array_equal(got, got2)
        qb, kb = f32buf(axk, rt, x), f32buf(axk, rt, x[:2 * hd])
        assert lib.axiom_runtime_qknorm_rope_pos_dual_f32_device(rt.handle, qb.handle, 0, wb.handle, 0, kb.handle, 0, wb.handle, 0,
                                                                 pb.handle, 0, heads, 2, hd, 1e6, 1e-6) == axk.AXIOM_OK
        gq = np.empty_like(x); gk = np.empty(2 * hd, np.float32); qb.download(gq); kb.download(gk)
        assert np.array_equal(gq, got) and np.array_equal(gk, got[:2 * hd])
    xb, wb = f32buf(axk, rt, x), f32buf(axk, rt, w)
    assert lib.axiom_runtime_qknorm_rope_f32_device(rt.handle, xb.handle, 0, wb.handle, 0, 5, 96, 0, 1e6, 1e-6) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_runtime_rope_neox_f32_device(rt.handle, xb.handle, 0, heads, 127, 0, 1e6) == axk.AXIOM_ERR_INVALID_ARGUMENT


def test_generic_f32_elementwise_and_paged_store(axk, rt):
    lib = axk.lib()
    rng = np.random.default_rng(2)
    n = 10007
    a = rng.standard_normal(n).astype(np.float32); b = rng.standard_normal(n).astype(np.float32)
    ab, bb, ob = f32buf(axk, rt, a), f32buf(axk, rt, b), axk.DeviceBuffer(rt, n * 4)
    assert lib.axiom_runtime_add_f32_device(rt.handle, ab.handle, 0, bb.handle, 0, ob.handle, 0, n) == axk.AXIOM_OK
    got = np.empty(n, np.float32); ob.download(got)
    assert np.array_equal(got, ol.add_f32(a, b))
    g3 = np.array([0, 1, -1], np.float32)  # tests/axiom_safetensors_smoke.cpp:234-244
    gb, ub, o3 = f32buf(axk, rt, g3), f32buf(axk, rt, np.full(3, 2, np.float32)), axk.DeviceBuffer(rt, 12)
    assert lib.axiom_runtime_silu_mul_f32_device(rt.handle, gb.handle, 0, ub.handle, 0, o3.handle, 0, 3) == axk.AXIOM_OK
    got3 = np.empty(3, np.float32); o3.download(got3)
    assert np.allclose(got3, [0.0, 1.4621172, -0.5378828], atol=1e-3)
    assert lib.axiom_runtime_silu_mul_f32_device(rt.handle, ab.handle, 0, bb.handle, 0, ob.handle, 0, n) == axk.AXIOM_OK
    ob.download(got)
    assert np.allclose(got, ol.silu_mul_f32(a, b), rtol=1e-3, atol=1e-5)
    a5 = a * 5
    ab = f32buf(axk, rt, a5)
    assert lib.axiom_runtime_silu_mul_clamp_f32_device(rt.handle, ab.handle, 0, bb.handle, 0, ob.handle, 0, n, 2.0) == axk.AXIOM_OK
    ob.download(got)
    assert np.allclose(got, ol.silu_mul_f32(a5, b, 2.0), rtol=1e-3, atol=1e-5)

    # paged store: 0xFF-poisoned pools, host-recomputed addresses, bit-verify (tools/axiom_paged_attn_parity_smoke.cpp:207-241)
    active, kv_dim, stride, BT, NL, L, nblk, tbl = 7, 1024, 1088, 16, 3, 1, 40, 9
    ks = rng.standard_normal((active, kv_dim)).astype(np.float32); vs = rng.standard_normal((active, kv_dim)).astype(np.float32)
    tables = np.stack([rng.permutation(nblk)[:tbl] for _ in range(active)]).astype(np.int32)
    pos = rng.integers(0, tbl * BT, active).astype(np.uint32)
    elems = nblk * NL * BT * stride
    poison = np.full(elems, np.frombuffer(b"\xff\xff\xff\xff", np.float32)[0], np.float32)
    kp, vp = f32buf(axk, rt, poison), f32buf(axk, rt, poison)
    rc = lib.axiom_runtime_kv_pool_store_paged_f32_device(
        rt.handle, f32buf(axk, rt, ks).handle, 0, f32buf(axk, rt, vs).handle, 0, kp.handle, 0, vp.handle, 0,
        buf_from(axk, rt, tables).handle, 0, buf_from(axk, rt, pos).handle, 0, active, tbl, NL, L, BT, stride, kv_dim)
    assert rc == axk.AXIOM_OK
    want_k, want_v = poison.copy(), poison.copy()
    ol.kv_pool_store_paged_f32(ks, vs, want_k, want_v, tables, pos, n_layers=NL, layer=L, block_tokens=BT, pool_stride=stride)
    gk = np.empty(elems, np.float32); gv = np.empty(elems, np.float32); kp.download(gk); vp.download(gv)
    assert np.array_equal(gk.view(np.uint32), want_k.view(np.uint32)) and np.array_equal(gv.view(np.uint32), want_v.view(np.uint32))
    assert lib.axiom_runtime_kv_pool_store_paged_f32_device(
        rt.handle, kp.handle, 0, vp.handle, 0, kp.handle, 0, vp.handle, 0, kp.handle, 0, vp.handle, 0,
        active, tbl, NL, NL, BT, stride, kv_dim) == axk.AXIOM_ERR_INVALID_ARGUMENT  # layer >= n_layers


def make_q8_0_table(rng, tokens, hidden):
    """Rows of hidden/32 blocks: little-endian F16 scale, then 32 signed bytes."""
    blocks = tokens * hidden // 32
    table = np.zeros((blocks, 34), np.uint8)
    scales = (rng.standard_normal(blocks) * 0.01).astype(np.float16)
    scales[::7] = np.float16(6e-8)  # F16 subnormals
    table[:, :2] = scales.view(np.uint8).reshape(blocks, 2)
    table[:, 2:] = rng.integers(-128, 128, (blocks, 32)).astype(np.int8).view(np.uint8)
    return table.reshape(-1)


def test_generic_embedding_gathers(axk, rt):
    """axiom_runtime_{q8_0_embedding_gather[_token],f16_embedding_streams}_f32_device vs the oracle, bit for bit,
    and vs the reference's kernels when its harness library is present."""
    import ref_lib

    lib = axk.lib()
    rng = np.random.default_rng(7)
    tokens, hidden = 50, 5120
    table = make_q8_0_table(rng, tokens, hidden)
    tb = buf_from(axk, rt, table)
    ob = axk.DeviceBuffer(rt, hidden * 4 + 64)
    got = np.empty(hidden, np.float32)
    for tok in (0, 17, 49):
        assert lib.axiom_runtime_q8_0_embedding_gather_f32_device(rt.handle, tb.handle, 0, ob.handle, 64, tok, tokens, hidden) == 0
        full = np.empty(hidden + 16, np.float32); ob.download(full); got = full[16:]
        want = ol.q8_0_embedding_gather_f32(table, tok, tokens, hidden)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        idb = buf_from(axk, rt, np.array([tok], np.uint32))
        assert lib.axiom_runtime_q8_0_embedding_gather_token_f32_device(rt.handle, tb.handle, 0, idb.handle, 0, ob.handle, 64,
                                                                        tokens, hidden) == 0
        ob.download(full)
        assert np.array_equal(full[16:].view(np.uint32), want.view(np.uint32))
    # device-side id beyond the table: zero row; immediate id beyond the table: rejected
    idb = buf_from(axk, rt, np.array([tokens], np.uint32))
    assert lib.axiom_runtime_q8_0_embedding_gather_token_f32_device(rt.handle, tb.handle, 0, idb.handle, 0, ob.handle, 64, tokens, hidden) == 0
    ob.download(full)
    assert not full[16:].any()
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_runtime_q8_0_embedding_gather_f32_device(rt.handle, tb.handle, 0, ob.handle, 64, tokens, tokens, hidden) == inv
    assert lib.axiom_runtime_q8_0_embedding_gather_f32_device(rt.handle, tb.handle, 0, ob.handle, 64, 0, tokens, hidden + 8) == inv
    assert lib.axiom_runtime_q8_0_embedding_gather_f32_device(rt.handle, tb.handle, 34, ob.handle, 64, 0, tokens, hidden) == inv  # span
    # F16 rows replicated into streams
    emb = rng.standard_normal((tokens, hidden)).astype(np.float16)
    emb[3, :4] = np.array([0.0, -0.0, 6e-8, 65504.0], np.float16)
    eb = buf_from(axk, rt, emb.view(np.uint16))
    streams = 4
    sb = axk.DeviceBuffer(rt, hidden * streams * 4)
    out = np.empty(hidden * streams, np.float32)
    for tok in (3, 49):
        assert lib.axiom_runtime_f16_embedding_streams_device(rt.handle, eb.handle, 0, sb.handle, 0, tok, hidden, streams) == 0
        sb.download(out)
        want = ol.f16_embedding_streams_f32(emb.view(np.uint16).reshape(-1), tok, hidden, streams)
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
        assert np.array_equal(out.reshape(streams, hidden)[2], emb[tok].astype(np.float32))
    assert lib.axiom_runtime_f16_embedding_streams_device(rt.handle, eb.handle, 0, sb.handle, 0, tokens, hidden, streams) == inv
    assert lib.axiom_runtime_f16_embedding_streams_device(rt.handle, eb.handle, 0, sb.handle, 0, 0, hidden, streams + 1) == inv
    if ref_lib.available():
        import torch

        r = ref_lib.lib()
        t_dev = torch.from_numpy(table).cuda()
        o_dev = torch.zeros(hidden, dtype=torch.float32, device="cuda")
        assert r.ref_q8_0_embedding_gather_f32(t_dev.data_ptr(), o_dev.data_ptr(), 17, tokens, hidden) == 0
        assert np.array_equal(o_dev.cpu().numpy().view(np.uint32), ol.q8_0_embedding_gather_f32(table, 17, tokens, hidden).view(np.uint32))
        e_dev = torch.from_numpy(emb.view(np.int16)).cuda()
        s_dev = torch.zeros(hidden * streams, dtype=torch.float32, device="cuda")
        assert r.ref_f16_embedding_streams(e_dev.data_ptr(), s_dev.data_ptr(), 3, hidden, streams) == 0
        assert np.array_equal(s_dev.cpu().numpy().view(np.uint32),
                              ol.f16_embedding_streams_f32(emb.view(np.uint16).reshape(-1), 3, hidden, streams).view(np.uint32))


def test_launch_async_env_is_honoured(axk, rt):
    """With AXIOM_CUDA_LAUNCH_ASYNC=1 the generic ops return right after the launch; results are
    complete after an explicit synchronisation (src/axiom_cuda.cu:162-200 in the reference)."""
    import torch

    lib = axk.lib()
    a = np.arange(4096, dtype=np.float32)
    ab, ob = f32buf(axk, rt, a), axk.DeviceBuffer(rt, a.nbytes)
    os.environ["AXIOM_CUDA_LAUNCH_ASYNC"] = "1"
    try:
        assert lib.axiom_runtime_add_f32_device(rt.handle, ab.handle, 0, ab.handle, 0, ob.handle, 0, 4096) == axk.AXIOM_OK
    finally:
        del os.environ["AXIOM_CUDA_LAUNCH_ASYNC"]
    torch.cuda.synchronize()
    got = np.empty_like(a); ob.download(got)
    assert np.array_equal(got, a + a)


def test_engine_view_qk_step_ragged_batch(axk, rt):
    """One decode step of a ragged continuous batch as a step-engine family provider issues it: block tables and
    positions come from the engine's device bookkeeping (d_tbl [cap][tbl_stride], positions at byte cap*4 of
    d_meta), the pools are poisoned with 0xFF first and every written cell is recomputed on the host — the scheme
    of the reference's paged-store parity tool (tools/axiom_paged_attn_parity_smoke.cpp:207-241), on BF16 pools."""
    lib = axk.lib()
    cap, n_active, tbl_stride, bt, n_layers, layer, nphys = 12, 7, 6, 16, 3, 1, 40
    q_heads, k_heads, D, rope_dim = 16, 2, 128, 128
    kv_dim = k_heads * D + 64  # a pool row wider than the K row: the tail lanes must stay untouched
    rng = np.random.default_rng(77)
    q, k, v, qg, kg, _, _ = wl.qk_inputs_np(n_active, q_heads, k_heads, D, nphys, seed=9)
    lengths = np.array([0, 15, 16, 17, 63, 95, 40], np.uint32)  # cache length of each active sequence = write position
    tbl = np.full((cap, tbl_stride), -1, np.int32)
    free = list(rng.permutation(nphys))
    for a in range(n_active):
        for lb in range(int(lengths[a]) // bt + 1):
            tbl[a, lb] = free.pop()
    meta = np.zeros(2 * cap, np.uint32)
    meta[:n_active] = lengths + 1
    meta[cap:cap + n_active] = lengths
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, rope_dim)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    pool_elems = nphys * n_layers * bt * kv_dim
    poison = np.full(pool_elems, 0xFFFF, np.uint16)
    bufs = {name: buf_from(axk, rt, a) for name, a in dict(q=q, k=k, v=v, qg=qg, kg=kg, f=inv_freq, tbl=tbl, meta=meta,
                                                           kpool=poison, vpool=poison, status=np.zeros(1, np.uint32)).items()}
    view = axk.PagedKvView(axk.AXIOM_ABI_VERSION, C.sizeof(axk.PagedKvView), bufs["kpool"].handle, bufs["vpool"].handle,
                           bufs["tbl"].handle, bufs["meta"].handle, cap, tbl_stride, bt, n_layers, nphys, kv_dim)

    def call(n=n_active, lyr=layer, flags=0, view_=view):
        return lib.axiom_runtime_qknorm_rope_yarn_paged_bf16_device(
            rt.handle, C.byref(view_), lyr, n, flags, bufs["q"].handle, 0, bufs["k"].handle, 0, bufs["v"].handle, 0,
            bufs["qg"].handle, 0, bufs["kg"].handle, 0, bufs["f"].handle, 0, q_heads, k_heads, D, rope_dim, 1e-6, mscale,
            bufs["status"].handle, 0)

    assert call() == axk.AXIOM_OK
    got_q, got_kpool, got_vpool = np.empty_like(q), np.empty_like(poison), np.empty_like(poison)
    status = np.ones(1, np.uint32)
    for name, out in (("q", got_q), ("kpool", got_kpool), ("vpool", got_vpool), ("status", status)):
        assert bufs[name].download(out) == axk.AXIOM_OK
    assert int(status[0]) == 0
    o_kpool, o_vpool = poison.copy(), poison.copy()
    want_q, _, want_status = ol.qk_norm_rope_paged(
        q, k, v, qg, kg, inv_freq, lengths[:n_active], tbl[:n_active], rope_dim=rope_dim, eps=1e-6, mscale=mscale,
        block_tokens=bt, n_layers=n_layers, layer=layer, pool_stride=kv_dim, n_blocks=nphys, ring=False,
        per_token_table=True, k_pool=o_kpool, v_pool=o_vpool, want_k_out=True)
    assert want_status == 0
    assert np.mean(got_q != want_q) < 0.02
    assert np.all(np.abs(wl.from_bf16_bits(got_q) - wl.from_bf16_bits(want_q)) <=
                  ol.bf16_ulp(np.abs(wl.from_bf16_bits(want_q))) * np.float32(4.0) + np.float32(1e-3))
    # cells: exactly the oracle's, V bit for bit, K within the rotation tolerance and at the same addresses
    assert np.array_equal(got_vpool, o_vpool)
    assert np.array_equal(got_kpool != 0xFFFF, o_kpool != 0xFFFF)
    for a in range(n_active):
        pos = int(lengths[a])
        base = ((int(tbl[a, pos // bt]) * n_layers + layer) * bt + pos % bt) * kv_dim
        assert np.all(got_kpool[base:base + k_heads * D] != 0xFFFF) and np.all(got_kpool[base + k_heads * D:base + kv_dim] == 0xFFFF)
    assert int((got_kpool != 0xFFFF).sum()) == n_active * k_heads * D

    # a sequence whose position has no block yet (-1 in its row) raises the status word and writes nothing for it
    meta2 = meta.copy()
    meta2[cap + 2] = 5 * bt
    assert bufs["meta"].upload(meta2) == axk.AXIOM_OK and bufs["kpool"].upload(poison) == axk.AXIOM_OK
    assert call() == axk.AXIOM_OK
    assert bufs["status"].download(status) == axk.AXIOM_OK and int(status[0]) == axk.STATUS_WORD_BAD_ADDRESS
    assert bufs["kpool"].download(got_kpool) == axk.AXIOM_OK
    assert int((got_kpool != 0xFFFF).sum()) == (n_active - 1) * k_heads * D

    # validation: more sequences than slots, layer out of range, unknown flag, pool smaller than its geometry
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert call(n=cap + 1) == inv and call(lyr=n_layers) == inv and call(flags=axk.QK_FLAG_RING) == inv and call(n=0) == inv
    big = axk.PagedKvView(axk.AXIOM_ABI_VERSION, C.sizeof(axk.PagedKvView), bufs["kpool"].handle, bufs["vpool"].handle,
                          bufs["tbl"].handle, bufs["meta"].handle, cap, tbl_stride, bt, n_layers, nphys + 1, kv_dim)
    assert call(view_=big) == inv
    wide = axk.PagedKvView(axk.AXIOM_ABI_VERSION, C.sizeof(axk.PagedKvView), bufs["kpool"].handle, bufs["vpool"].handle,
                           bufs["tbl"].handle, bufs["meta"].handle, cap + 1, tbl_stride, bt, n_layers, nphys, kv_dim)
    assert call(view_=wide) == inv
    for b in bufs.values():
        b.close()

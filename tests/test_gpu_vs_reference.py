"""The CUDA path against the REFERENCE'S OWN KERNELS (oracle/_ref, built from the reference tree for
sm_100a) on identical seeded inputs, on the same GPU: every comparison here is bit-exact, including
the ops whose transcendental functions make the CPU oracle differ in the last bits."""
import ctypes as C
import importlib

import numpy as np
import pytest

import oracle_lib as ol
import ref_lib

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref is built only where the reference tree is present")]
wl = importlib.import_module("axiom-kernel_b200.workloads")


def mine_nvfp4(axk, bits, G, layout):
    import torch
    from gpu_util import dev, sync

    rows, cols = bits.shape
    codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, layout)), dtype=torch.uint8, device="cuda")
    assert axk.nvfp4_quantize(0, dev(bits), rows, cols, G, codes, scales, layout) == 0
    sync()
    return codes.cpu().numpy(), scales.cpu().numpy()


@pytest.mark.parametrize("rows,cols", [(8, 5120), (200, 5120), (12, 64), (130, 17408)])
def test_nvfp4_quantizer_three_reference_kernels(axk, cuda_device, rows, cols):
    import ref_cases as rc

    bits = rc.special_rows(cols) if rows == 12 else wl.quantize_input_np(rows, cols, seed=rows)
    amax = np.nanmax(np.abs(np.where(np.isfinite(wl.from_bf16_bits(bits)), wl.from_bf16_bits(bits), 0)))
    for G in (wl.nvfp4_global_scale(float(amax)), 1.0, 3.3e4):
        row_codes, row_scales = rc.nvfp4_quantize(bits, G, "row")
        got_codes, got_scales = mine_nvfp4(axk, bits, G, 0)
        assert np.array_equal(got_codes, row_codes) and np.array_equal(got_scales.reshape(rows, -1), row_scales)
        got_codes_t, got_scales_t = mine_nvfp4(axk, bits, G, 1)
        for variant in ("thread", "warp"):
            ref_codes, ref_plane = rc.nvfp4_quantize(bits, G, variant)
            assert np.array_equal(got_codes_t, ref_codes), variant
            if rows == 12 and variant == "warp":
                # An all-NaN block (row 3, block 0): the reference's warp kernel starts its maximum from
                # |x| instead of 0 and so encodes a NaN scale (0x7e after the fix-up), while its thread kernel
                # and its exported oracle entry give the zero-block guard 0x20.  The oracle entry is followed.
                cell = int(axk.lib().axiom_nvfp4_scale_plane_offset(3, 0, cols // 16, 1))
                assert ref_plane[cell] == 0x7e and got_scales_t[cell] == 0x20
                ref_plane = ref_plane.copy()
                ref_plane[cell] = 0x20
            assert np.array_equal(got_scales_t, ref_plane), variant


def test_reference_named_entry_is_a_drop_in(axk, cuda_device):
    """Same symbol, same arguments, same bytes out: libaxiom_b200 vs the reference's axiom_qwen38_nvfp4.cu."""
    import torch

    rng = np.random.default_rng(0)
    for cols in (16, 5120, 17408):
        x = torch.from_numpy((rng.standard_normal(cols) * 3).astype(np.float32)).cuda()
        outs = []
        for lib in (axk.lib(), ref_lib.lib()):
            codes = torch.zeros(cols // 2, dtype=torch.uint8, device="cuda")
            scales = torch.zeros(cols // 16, dtype=torch.uint8, device="cuda")
            assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, x.data_ptr(), 55.5, codes.data_ptr(), scales.data_ptr(), cols, None) == 0
            outs.append((codes.cpu().numpy(), scales.cpu().numpy()))
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
        for lib in (axk.lib(), ref_lib.lib()):  # identical argument checks
            assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, x.data_ptr(), 0.0, 16, 16, cols, None) == 1
            assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, x.data_ptr(), 1.0, 16, 16, 24, None) == 1
            assert lib.axiom_qwen38_nvfp4_quantize_reference_f32(0, None, 1.0, 16, 16, cols, None) == 1


@pytest.mark.parametrize("rows", [8, 64, 1024])
@pytest.mark.parametrize("with_add", [True, False])
def test_add_rmsnorm_nvfp4_bit_exact(axk, cuda_device, rows, with_add):
    import torch
    import ref_cases as rc
    from gpu_util import dev, host, sync

    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, 5120)
    ref_res, ref_norm = rc.add_rmsnorm(hidden if with_add else None, residual, gamma)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(ref_norm)).max()))
    ref_codes, ref_plane = rc.nvfp4_quantize(ref_norm, G, "warp")
    r = dev(residual)
    norm = torch.zeros((rows, 5120), dtype=torch.int16, device="cuda")
    codes = torch.zeros((rows, 2560), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(ref_plane.size, dtype=torch.uint8, device="cuda")
    assert axk.add_rmsnorm_nvfp4(0, dev(hidden) if with_add else None, r, dev(gamma), 1e-6, rows, 5120, G, norm, codes, plane, 1) == 0
    sync()
    assert np.array_equal(host(r, np.uint16).reshape(rows, 5120), ref_res)
    assert np.array_equal(host(norm, np.uint16).reshape(rows, 5120), ref_norm)      # same FP32 summation order, same rsqrtf
    assert np.array_equal(codes.cpu().numpy(), ref_codes) and np.array_equal(plane.cpu().numpy(), ref_plane)


def test_add_bf16_bit_exact(axk, cuda_device):
    import torch
    import ref_cases as rc
    from gpu_util import dev, host, sync

    rng = np.random.default_rng(1)
    a = wl.to_bf16_bits(rng.standard_normal(40960).astype(np.float32) * 4)
    b = wl.to_bf16_bits(rng.standard_normal(40960).astype(np.float32))
    out = torch.zeros(40960, dtype=torch.int16, device="cuda")
    assert axk.add_bf16(0, dev(a), dev(b), out, 40960) == 0
    sync()
    assert np.array_equal(host(out, np.uint16), rc.add_bf16(a, b))


def test_fp8_quantizers_bit_exact(axk, cuda_device):
    import torch
    import ref_cases as rc
    from gpu_util import dev, sync

    for rows, cols in [(8, 5120), (24, 17408), (3, 64), (640, 8192), (600, 5120)]:
        bits = wl.quantize_input_np(rows, cols, seed=cols)
        bits[0, :] = 0
        codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
        scales = torch.zeros(rows, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert axk.fp8_quantize(0, dev(bits), rows, cols, codes, scales, status) == 0
        sync()
        ref_codes, ref_scales = rc.fp8_quantize_f32(rc.f32_dev(bits))           # F32-input target kernel
        assert np.array_equal(codes.cpu().numpy(), ref_codes) and np.array_equal(scales.cpu().numpy(), ref_scales)
        bits[1, 7] = 0x7F80                                                     # BF16-input twin with a non-finite value
        status.zero_()
        assert axk.fp8_quantize(0, dev(bits), rows, cols, codes, scales, status) == 0
        sync()
        twin_codes, twin_scales, twin_status = rc.fp8_quantize_bf16(bits)
        assert np.array_equal(codes.cpu().numpy(), twin_codes) and np.array_equal(scales.cpu().numpy(), twin_scales)
        assert int(status.item()) == twin_status == 4


def test_static_scale_fp8_bit_exact(axk, cuda_device):
    """Given-scale flavours against quantize_columns_static_e4m3_kernel: a BF16 tensor, and silu(gate)*up through the
    reference's silu_mul_batch_kernel followed by that quantizer."""
    import torch
    import ref_cases as rc
    from gpu_util import dev, sync

    for rows, cols, scale in [(8, 5120, 0.011), (24, 17408, 0.5), (3, 64, 1.0e-3), (320, 1024, 0.02)]:
        bits = wl.quantize_input_np(rows, cols, seed=cols)
        bits[0, :4] = [0x7F80, 0xFF80, 0x7FC0, 0x8000]
        codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
        assert axk.fp8_quantize_static(0, dev(bits), rows, cols, scale, codes) == 0
        sync()
        assert np.array_equal(codes.cpu().numpy(), rc.fp8_quantize_static_f32(rc.f32_dev(bits), scale))
        gu = wl.swiglu_input_np(rows, cols, seed=rows)
        assert axk.swiglu_fp8_static(0, dev(gu), rows, cols, scale, codes) == 0
        sync()
        assert np.array_equal(codes.cpu().numpy(), rc.fp8_quantize_static_f32(rc.swiglu_f32(gu), scale))


@pytest.mark.parametrize("rows,width", [(8, 17408), (40, 4096), (3, 64), (16, 11008), (320, 1024), (304, 17408)])
def test_swiglu_fp8_and_nvfp4_bit_exact(axk, cuda_device, rows, width):
    import torch
    import ref_cases as rc
    from gpu_util import dev, sync

    gu = wl.swiglu_input_np(rows, width, seed=rows)
    gu[0, :8] = [0x0000, 0x8000, 0xC2C8, 0x42C8, 0x4300, 0xC300, 0x3F80, 0xBF80]  # 0, -0, -100, 100, 128, -128, 1, -1
    ref_codes, ref_scales = rc.swiglu_fp8(gu)
    codes = torch.zeros((rows, width), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, dtype=torch.float32, device="cuda")
    assert axk.swiglu_fp8(0, dev(gu), rows, width, codes, scales) == 0
    sync()
    assert np.array_equal(scales.cpu().numpy(), ref_scales)
    assert np.array_equal(codes.cpu().numpy(), ref_codes)
    G = wl.nvfp4_global_scale(float(rc.swiglu_f32(gu).abs().max().item()))
    c4 = torch.zeros((rows, width // 2), dtype=torch.uint8, device="cuda")
    for variant in ("thread", "warp"):
        ref_c4, ref_plane = rc.swiglu_nvfp4(gu, G, variant)
        plane = torch.zeros(ref_plane.size, dtype=torch.uint8, device="cuda")
        assert axk.swiglu_nvfp4(0, dev(gu), rows, width, G, c4, plane, 1) == 0
        sync()
        assert np.array_equal(c4.cpu().numpy(), ref_c4) and np.array_equal(plane.cpu().numpy(), ref_plane)


def test_yarn_table_and_qk_norm_rope_bit_exact(axk, cuda_device):
    """Reference geometry (24 q / 4 kv heads x 256, rope_dim 64, theta 1e7, YaRN x4 / 262144), 8 tokens."""
    import torch
    import ref_cases as rc
    from gpu_util import dev, host, sync

    inv = torch.zeros(32, dtype=torch.float32, device="cuda")
    assert axk.yarn_inv_freq(0, 64, rc.REF_THETA, rc.REF_YARN_FACTOR, rc.REF_YARN_CTX, 32.0, 1.0, inv) == 0
    sync()
    assert np.array_equal(inv.cpu().numpy().view(np.uint32), rc.yarn_inv_freq().view(np.uint32))
    assert np.float32(axk.yarn_mscale(4.0)) == np.float32(rc.REF_MSCALE)
    for base in (0, 1, 1000, 99992, 262000, 1000000):
        q, k, v, qg, kg = rc.qk_inputs(seed=base)
        ref_q, ref_k, ref_v, _ = rc.qk_temporal8(q, k, v, qg, kg, base)
        qd, kd, qgd, kgd = dev(q), dev(k), dev(qg), dev(kg)
        k_out = torch.zeros((8, 4, 256), dtype=torch.int16, device="cuda")
        positions = dev((base + np.arange(8)).astype(np.uint32))
        args = axk.make_qk_args(tokens=8, q_heads=24, k_heads=4, head_dim=256, rope_dim=64, eps=1e-6, mscale=rc.REF_MSCALE,
                                q=qd, k=kd, q_gamma=qgd, k_gamma=kgd, inv_freq=inv, positions=positions, k_out=k_out)
        assert axk.qk_norm_rope_paged(0, args) == 0
        sync()
        assert np.array_equal(host(qd, np.uint16).reshape(q.shape), ref_q), base
        assert np.array_equal(host(k_out, np.uint16).reshape(k.shape), ref_k), base
        assert np.array_equal(ref_v, v)
    # FP8 cache flavour against the reference's own E4M3 cache rows (positions 0..7 of one 8-token block)
    q, k, v, qg, kg = rc.qk_inputs(seed=0)
    ref_q, ref_k, ref_v, ref_kcache = rc.qk_temporal8(q, k, v, qg, kg, 0)
    qd, kd, vd, qgd, kgd = dev(q), dev(k), dev(v), dev(qg), dev(kg)
    k_cache = torch.zeros((8, 1024), dtype=torch.uint8, device="cuda")
    v_cache = torch.zeros((8, 1024), dtype=torch.uint8, device="cuda")
    table = dev(np.zeros((1, 1), np.int32))
    positions = dev(np.arange(8, dtype=np.uint32))
    args = axk.make_qk_args(tokens=8, q_heads=24, k_heads=4, head_dim=256, rope_dim=64, eps=1e-6, mscale=rc.REF_MSCALE,
                            flags=axk.QK_FLAG_CACHE_E4M3, block_tokens=8, n_layers=1, layer=0, pool_stride=1024,
                            tbl_stride=1, n_blocks=1, q=qd, k=kd, v=vd, q_gamma=qgd, k_gamma=kgd, inv_freq=inv,
                            positions=positions, block_tables=table, k_pool=k_cache, v_pool=v_cache)
    assert axk.qk_norm_rope_paged(0, args) == 0
    sync()
    assert np.array_equal(host(qd, np.uint16).reshape(q.shape), ref_q)
    assert np.array_equal(k_cache.cpu().numpy(), ref_kcache)
    assert np.array_equal(v_cache.cpu().numpy().reshape(-1), ol.bf16_to_e4m3_scale1(v).reshape(-1))


@pytest.mark.parametrize("q_heads,k_heads,tokens,first", [(40, 8, 8, 0), (40, 8, 16, 1000), (64, 8, 8, 99990), (40, 8, 300, 5)])
def test_round_after_norm_convention_bit_exact(axk, cuda_device, q_heads, k_heads, tokens, first):
    """AXIOM_QK_FLAG_ROUND_AFTER_NORM against the reference's qk_rmsnorm_rope_bf16_kernel + round_f32_to_bf16 pass
    (the draft's geometry, 40 q / 8 kv heads x 128 with full-head rotation, and the benchmark's 64 / 8 x 128), cos/sin
    from a host-built [position][cos | sin] table as the reference builds it: Q, K and the cached K rows bit for bit."""
    import torch
    import ref_cases as rc
    from gpu_util import dev, host, sync

    rng = np.random.default_rng(q_heads + tokens)
    q = wl.to_bf16_bits(rng.standard_normal((tokens, q_heads, 128), dtype=np.float32))
    k = wl.to_bf16_bits(rng.standard_normal((tokens, k_heads, 128), dtype=np.float32) * np.float32(3.0))
    qg = wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(128, dtype=np.float32))
    kg = wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(128, dtype=np.float32))
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128, host_table=True)
    table = ol.rope_table_host(inv_freq, 128, float(ol.o().axo_yarn_mscale(4.0)), first + tokens)
    positions = (first + np.arange(tokens)).astype(np.uint32)
    want_q = rc.draft_qk_norm_rope(q, qg, table, first)
    want_k = rc.draft_qk_norm_rope(k, kg, table, first)

    n_blocks = (first + tokens) // 16 + 1
    btab = np.random.default_rng(3).permutation(n_blocks).astype(np.int32).reshape(1, n_blocks)
    qd, kd, qgd, kgd, td, pd, bd = dev(q), dev(k), dev(qg), dev(kg), dev(table), dev(positions), dev(btab)
    pool = torch.full((n_blocks * 16 * k_heads * 128,), -1, dtype=torch.int16, device="cuda")
    k_out = torch.zeros((tokens, k_heads, 128), dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = axk.make_qk_args(tokens=tokens, q_heads=q_heads, k_heads=k_heads, head_dim=128, rope_dim=128,
                            flags=axk.QK_FLAG_ROUND_AFTER_NORM, eps=1e-6, mscale=1.0, block_tokens=16, n_layers=1, layer=0,
                            pool_stride=k_heads * 128, tbl_stride=n_blocks, n_blocks=n_blocks, q=qd, k=kd, q_gamma=qgd,
                            k_gamma=kgd, positions=pd, block_tables=bd, k_pool=pool, k_out=k_out, status_word=status,
                            rope_table=td, rope_table_positions=table.shape[0])
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
    sync()
    assert int(status.item()) == 0
    assert np.array_equal(host(qd, np.uint16).reshape(q.shape), want_q)
    assert np.array_equal(host(k_out, np.uint16).reshape(k.shape), want_k)
    cells = host(pool, np.uint16).reshape(n_blocks, 16, k_heads * 128)
    assert np.array_equal(cells[btab[0, positions // 16], positions % 16], want_k.reshape(tokens, -1))
    # and the CPU restatement stays within one BF16 ulp of the kernels (its inverse square root is not the device's)
    cpu_q, st = ol.qk_norm_rope_round_after_norm(q, qg, table, positions)
    assert st == 0
    # (a one-ulp difference of the factor can flip the BF16 rounding of both rotation operands, so the bound is three
    # BF16 ulps at the magnitude of the rotation terms: one per operand and one for the final rounding)
    from test_gpu_qk_rope import tolerance

    a, b = wl.from_bf16_bits(cpu_q), wl.from_bf16_bits(want_q)
    assert np.all(np.abs(a - b) <= 3 * tolerance(q, qg, inv_freq, positions, 128, float(ol.o().axo_yarn_mscale(4.0))))
    assert np.mean(cpu_q != want_q) < 0.05


def test_sigmoid_gate_bit_exact(axk, cuda_device):
    """qwen38_sigmoid_gate_kernel on its fixed [8 x 6144] batch: the BF16 output must match bit for bit, also when the
    same rows go through the tabulated flavour (a call of 8 x 50 rows takes the table path)."""
    import torch
    from gpu_util import dev, sync

    r = ref_lib.lib()
    rng = np.random.default_rng(12)
    rows, width = 8, 6144
    attn = wl.to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32))
    gate = wl.to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32) * np.float32(3.0))
    gate.reshape(-1)[:8] = wl.to_bf16_bits(np.array([0.0, -0.0, 90.0, -90.0, 200.0, -200.0, 1e-30, np.inf], np.float32))
    a32 = torch.from_numpy(wl.from_bf16_bits(attn)).cuda()
    g32 = torch.from_numpy(wl.from_bf16_bits(gate)).cuda()
    out32 = torch.zeros_like(a32)
    assert r.ref_sigmoid_gate8(a32.data_ptr(), g32.data_ptr(), out32.data_ptr()) == 0
    want = wl.to_bf16_bits(out32.cpu().numpy())
    assert np.array_equal(wl.from_bf16_bits(want), out32.cpu().numpy())  # the reference output is BF16-valued
    for reps in (1, 50):
        a, g = dev(np.tile(attn, (reps, 1))), dev(np.tile(gate, (reps, 1)))
        y = torch.zeros((rows * reps, width), dtype=torch.int16, device="cuda")
        assert axk.sigmoid_gate_nvfp4(0, a, g, rows * reps, width, 1.0, y, None, None, 0) == axk.AXIOM_OK
        sync()
        got = y.cpu().numpy().view(np.uint16)
        assert np.array_equal(got[:rows], want) and np.array_equal(got[-rows:], want)


def test_generic_f32_ops_bit_exact(axk, cuda_device):
    import torch

    r = ref_lib.lib()
    lib = axk.lib()
    rt = axk.Runtime(0)
    rng = np.random.default_rng(4)

    def buf(a):
        b = axk.DeviceBuffer(rt, a.nbytes)
        assert b.upload(np.ascontiguousarray(a)) == 0
        return b

    def down(b, like):
        out = np.empty_like(like)
        b.download(out)
        return out

    for count in (5120, 4099, 64):
        x = rng.standard_normal(count).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(count)).astype(np.float32)
        xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        for variant, name in enumerate(["axiom_runtime_rmsnorm_f32_device", "axiom_runtime_rmsnorm_f32_hp_device", "axiom_runtime_rmsnorm_f32_b1_device"]):
            want = torch.zeros(count, device="cuda")
            assert r.ref_rmsnorm_f32(wt.data_ptr(), xt.data_ptr(), want.data_ptr(), count, 1e-6, variant) == 0
            ob = axk.DeviceBuffer(rt, count * 4)
            assert getattr(lib, name)(rt.handle, buf(w).handle, 0, buf(x).handle, 0, ob.handle, 0, count, 1e-6) == 0
            assert np.array_equal(down(ob, x).view(np.uint32), want.cpu().numpy().view(np.uint32)), (name, count)
    heads, hd = 7, 128
    x = rng.standard_normal(heads * hd).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    xb = buf(x)
    assert r.ref_head_rmsnorm_f32(xt.data_ptr(), heads, hd, 1e-6) == 0
    assert lib.axiom_runtime_head_rmsnorm_f32_device(rt.handle, xb.handle, 0, heads, hd, 1e-6) == 0
    assert np.array_equal(down(xb, x).view(np.uint32), xt.cpu().numpy().view(np.uint32))
    xt, xb = torch.from_numpy(x).cuda(), buf(x)
    assert r.ref_qk_rmsnorm_w_f32(xt.data_ptr(), wt.data_ptr(), heads, hd, 1e-6) == 0
    assert lib.axiom_runtime_qk_rmsnorm_w_f32_device(rt.handle, xb.handle, 0, buf(w).handle, 0, heads, hd, 1e-6) == 0
    assert np.array_equal(down(xb, x).view(np.uint32), xt.cpu().numpy().view(np.uint32))
    for pos in (0, 5, 4097, 123456):
        xt, xb = torch.from_numpy(x).cuda(), buf(x)
        assert r.axiom_qknorm_rope_precise_launch(0, xt.data_ptr(), wt.data_ptr(), heads, hd, pos, 1e6, 1e-6) == 0
        assert lib.axiom_runtime_qknorm_rope_f32_device(rt.handle, xb.handle, 0, buf(w).handle, 0, heads, hd, pos, 1e6, 1e-6) == 0
        assert np.array_equal(down(xb, x).view(np.uint32), xt.cpu().numpy().view(np.uint32)), pos
        xt, xb = torch.from_numpy(x).cuda(), buf(x)
        assert r.axiom_rope_neox_precise_launch(0, xt.data_ptr(), heads, hd, pos, 1e4) == 0
        assert lib.axiom_runtime_rope_neox_f32_device(rt.handle, xb.handle, 0, heads, hd, pos, 1e4) == 0
        assert np.array_equal(down(xb, x).view(np.uint32), xt.cpu().numpy().view(np.uint32)), pos
        xt, xb = torch.from_numpy(x).cuda(), buf(x)
        assert r.axiom_rope_neox_partial_precise_launch(0, xt.data_ptr(), heads, hd, 64, pos, 1e4) == 0
        assert lib.axiom_runtime_rope_neox_partial_f32_device(rt.handle, xb.handle, 0, heads, hd, 64, pos, 1e4) == 0
        assert np.array_equal(down(xb, x).view(np.uint32), xt.cpu().numpy().view(np.uint32)), pos
    n = 10001
    a = rng.standard_normal(n).astype(np.float32) * 4
    b = rng.standard_normal(n).astype(np.float32)
    at, bt, ot = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.zeros(n, device="cuda")
    ob = axk.DeviceBuffer(rt, n * 4)
    assert r.ref_add_f32(at.data_ptr(), bt.data_ptr(), ot.data_ptr(), n) == 0
    assert lib.axiom_runtime_add_f32_device(rt.handle, buf(a).handle, 0, buf(b).handle, 0, ob.handle, 0, n) == 0
    assert np.array_equal(down(ob, a).view(np.uint32), ot.cpu().numpy().view(np.uint32))
    for clamp in (0.0, 3.0):
        assert r.ref_silu_mul_f32(at.data_ptr(), bt.data_ptr(), ot.data_ptr(), n, clamp) == 0
        assert lib.axiom_runtime_silu_mul_clamp_f32_device(rt.handle, buf(a).handle, 0, buf(b).handle, 0, ob.handle, 0, n, clamp) == 0
        assert np.array_equal(down(ob, a).view(np.uint32), ot.cpu().numpy().view(np.uint32)), clamp
    rt.close()


def test_embedding_gather_bit_exact(axk, cuda_device):
    import torch
    from gpu_util import sync

    r = ref_lib.lib()
    vocab, hidden = int(r.ref_model_vocab()), int(r.ref_model_hidden())
    table = torch.zeros((vocab, hidden), dtype=torch.int16, device="cuda")
    ids = np.array([0, 1, 777, vocab - 1, 123456, vocab, 0xFFFFFFFF, 5], np.uint32)
    g = torch.Generator(device="cuda"); g.manual_seed(0)
    for i in ids[ids < vocab]:
        table[int(i)] = torch.randint(-30000, 30000, (hidden,), generator=g, device="cuda", dtype=torch.int32).to(torch.int16)
    idt = torch.from_numpy(ids.view(np.int32)).cuda()
    want = torch.zeros((8, hidden), dtype=torch.float32, device="cuda")
    assert r.ref_embedding_gather_columns(table.data_ptr(), idt.data_ptr(), want.data_ptr(), 8) == 0
    out = torch.zeros((8, hidden), dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert axk.embedding_gather(0, table, vocab, hidden, idt, 8, out, status) == 0
    sync()
    got = (out.cpu().numpy().view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(got.view(np.uint32), want.cpu().numpy().view(np.uint32))
    assert int(status.item()) == axk.STATUS_WORD_BAD_ADDRESS

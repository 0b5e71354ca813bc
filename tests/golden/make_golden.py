"""Writes tests/golden/reference_b200.npz: outputs of the REFERENCE'S OWN KERNELS (oracle/_ref,
compiled from the reference tree for sm_100a) on seeded inputs, run on a B200.

    python tests/golden/make_golden.py [output_dir]      # needs a GPU and oracle/_ref/libaxiom_ref.so

The fixture pins the CPU oracle (tests/test_golden.py, no GPU needed) and the CUDA path
(tests/test_gpu_golden.py) to the reference where the reference tree itself is not available.
Inputs are stored next to the outputs so nothing depends on a random-number generator's stream.
"""
import importlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import ref_cases as rc  # noqa: E402
import ref_lib  # noqa: E402

wl = importlib.import_module("axiom-kernel_b200.workloads")


def main():
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent
    out_dir.mkdir(parents=True, exist_ok=True)
    r = ref_lib.lib()
    fx = {}

    # 1. NVFP4 activation quantizer
    x = wl.quantize_input_np(16, 5120, seed=0)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(x)).max()))
    fx["q_in"], fx["q_G"] = x, np.float32(G)
    fx["q_codes"], fx["q_scales"] = rc.nvfp4_quantize(x, G, "row")
    c2, fx["q_plane_warp"] = rc.nvfp4_quantize(x, G, "warp")
    c3, plane_thread = rc.nvfp4_quantize(x, G, "thread")
    assert np.array_equal(c2, fx["q_codes"]) and np.array_equal(c3, c2) and np.array_equal(plane_thread, fx["q_plane_warp"])
    sp = rc.special_rows(64)
    fx["qs_in"] = sp
    for tag, Gs in (("a", 1.0), ("b", 74.6), ("c", 1e4)):
        fx[f"qs_G_{tag}"] = np.float32(Gs)
        fx[f"qs_codes_{tag}"], fx[f"qs_scales_{tag}"] = rc.nvfp4_quantize(sp, Gs, "row")

    # 2. residual add + RMSNorm (+ NVFP4 of the norm), and the norm-only kernel
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(8, 5120)
    fx["n_hidden"], fx["n_residual"], fx["n_gamma"] = hidden, residual, gamma
    fx["n_res_out"], fx["n_norm"] = rc.add_rmsnorm(hidden, residual, gamma)
    _, fx["n_norm_only"] = rc.add_rmsnorm(None, residual, gamma)
    Gn = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(fx["n_norm"])).max()))
    fx["n_G"] = np.float32(Gn)
    fx["n_codes"], fx["n_scales"] = rc.nvfp4_quantize(fx["n_norm"], Gn, "row")

    # 3. BF16 residual add
    rng = np.random.default_rng(1)
    a = wl.to_bf16_bits(rng.standard_normal(4096).astype(np.float32) * 4)
    b = wl.to_bf16_bits(rng.standard_normal(4096).astype(np.float32))
    fx["a_a"], fx["a_b"], fx["a_out"] = a, b, rc.add_bf16(a, b)

    # 4. FP8 per-token quantizers
    y = wl.quantize_input_np(8, 1024, seed=9)
    y[0] = 0
    fx["f_in"] = y
    fx["f_codes"], fx["f_scales"] = rc.fp8_quantize_f32(rc.f32_dev(y))
    y2 = y.copy()
    y2[1, 7] = 0x7F80
    fx["f2_in"] = y2
    fx["f2_codes"], fx["f2_scales"], st = rc.fp8_quantize_bf16(y2)
    fx["f2_status"] = np.uint32(st)

    # 5. SwiGLU
    gu = wl.swiglu_input_np(8, 2048, seed=4)
    gu[0, :8] = [0x0000, 0x8000, 0xC2C8, 0x42C8, 0x4300, 0xC300, 0x3F80, 0xBF80]
    fx["s_in"] = gu
    fx["s_y"] = rc.swiglu_f32(gu).cpu().numpy()
    fx["s_fp8_codes"], fx["s_fp8_scales"] = rc.swiglu_fp8(gu)
    Gs = wl.nvfp4_global_scale(float(np.abs(fx["s_y"]).max()))
    fx["s_G"] = np.float32(Gs)
    fx["s_nv_codes"], fx["s_nv_plane"] = rc.swiglu_nvfp4(gu, Gs, "warp")

    # 6. YaRN table and q/k norm + partial RoPE (reference geometry)
    fx["y_inv_freq"] = rc.yarn_inv_freq()
    for tag, base in (("lo", 1000), ("hi", 99992)):
        q, k, v, qg, kg = rc.qk_inputs(seed=base)
        fx[f"k_{tag}_q"], fx[f"k_{tag}_k"], fx[f"k_{tag}_v"], fx[f"k_{tag}_qg"], fx[f"k_{tag}_kg"] = q, k, v, qg, kg
        fx[f"k_{tag}_base"] = np.uint32(base)
        fx[f"k_{tag}_q_out"], fx[f"k_{tag}_k_out"], _, fx[f"k_{tag}_k_e4m3"] = rc.qk_temporal8(q, k, v, qg, kg, base)

    # 7. generic single-row F32 ops
    rng = np.random.default_rng(4)
    x = rng.standard_normal(5120).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(5120)).astype(np.float32)
    fx["g_x"], fx["g_w"] = x, w
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    for variant, tag in enumerate(("plain", "hp", "b1")):
        o = torch.zeros(5120, device="cuda")
        assert r.ref_rmsnorm_f32(wt.data_ptr(), xt.data_ptr(), o.data_ptr(), 5120, 1e-6, variant) == 0
        fx[f"g_rmsnorm_{tag}"] = o.cpu().numpy()
    heads, hd = 7, 128
    hx = rng.standard_normal(heads * hd).astype(np.float32)
    hw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    fx["g_hx"], fx["g_hw"] = hx, hw
    t = torch.from_numpy(hx).cuda()
    assert r.ref_head_rmsnorm_f32(t.data_ptr(), heads, hd, 1e-6) == 0
    fx["g_head_rmsnorm"] = t.cpu().numpy()
    t = torch.from_numpy(hx).cuda()
    hwt = torch.from_numpy(hw).cuda()
    assert r.ref_qk_rmsnorm_w_f32(t.data_ptr(), hwt.data_ptr(), heads, hd, 1e-6) == 0
    fx["g_qk_rmsnorm_w"] = t.cpu().numpy()
    for pos in (5, 4097):
        t = torch.from_numpy(hx).cuda()
        assert r.axiom_qknorm_rope_precise_launch(0, t.data_ptr(), hwt.data_ptr(), heads, hd, pos, 1e6, 1e-6) == 0
        fx[f"g_qknorm_rope_{pos}"] = t.cpu().numpy()
        t = torch.from_numpy(hx).cuda()
        assert r.axiom_rope_neox_partial_precise_launch(0, t.data_ptr(), heads, hd, 64, pos, 1e4) == 0
        fx[f"g_rope_partial_{pos}"] = t.cpu().numpy()
    ga = rng.standard_normal(1000).astype(np.float32) * 4
    gb = rng.standard_normal(1000).astype(np.float32)
    fx["g_a"], fx["g_b"] = ga, gb
    at, bt, ot = torch.from_numpy(ga).cuda(), torch.from_numpy(gb).cuda(), torch.zeros(1000, device="cuda")
    assert r.ref_add_f32(at.data_ptr(), bt.data_ptr(), ot.data_ptr(), 1000) == 0
    fx["g_add"] = ot.cpu().numpy()
    assert r.ref_silu_mul_f32(at.data_ptr(), bt.data_ptr(), ot.data_ptr(), 1000, 0.0) == 0
    fx["g_silu_mul"] = ot.cpu().numpy()
    assert r.ref_silu_mul_f32(at.data_ptr(), bt.data_ptr(), ot.data_ptr(), 1000, 3.0) == 0
    fx["g_silu_mul_clamp3"] = ot.cpu().numpy()

    # sigmoid output gate on the reference's fixed [8 x 6144] batch
    sg_rng = np.random.default_rng(12)
    attn = wl.to_bf16_bits(sg_rng.standard_normal((8, 6144), dtype=np.float32))
    gate = wl.to_bf16_bits(sg_rng.standard_normal((8, 6144), dtype=np.float32) * np.float32(3.0))
    gate.reshape(-1)[:8] = wl.to_bf16_bits(np.array([0.0, -0.0, 90.0, -90.0, 200.0, -200.0, 1e-30, np.inf], np.float32))
    a32 = torch.from_numpy(wl.from_bf16_bits(attn)).cuda()
    g32 = torch.from_numpy(wl.from_bf16_bits(gate)).cuda()
    o32 = torch.zeros_like(a32)
    assert r.ref_sigmoid_gate8(a32.data_ptr(), g32.data_ptr(), o32.data_ptr()) == 0
    fx["sg_attention"], fx["sg_gate"], fx["sg_out"] = attn, gate, wl.to_bf16_bits(o32.cpu().numpy())

    # 8. the BF16 ("draft") rounding convention of q/k norm + RoPE: qk_rmsnorm_rope_bf16_kernel + round_f32_to_bf16,
    #    40 query heads x 128 as in the draft, cos/sin from a host-built [position][cos | sin] table
    import oracle_lib as ol  # the table is an INPUT of both sides; it is stored with the fixture

    dr = np.random.default_rng(31)
    dq = wl.to_bf16_bits(dr.standard_normal((8, 40, 128), dtype=np.float32))
    dg = wl.to_bf16_bits(1.0 + 0.02 * dr.standard_normal(128, dtype=np.float32))
    d_first = 4090
    d_inv = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128, host_table=True)
    d_table = ol.rope_table_host(d_inv, 128, float(ol.o().axo_yarn_mscale(4.0)), d_first + 8)
    fx["d_q"], fx["d_gamma"], fx["d_first"], fx["d_table_rows"] = dq, dg, np.uint32(d_first), d_table[d_first:d_first + 8].copy()
    fx["d_out"] = rc.draft_qk_norm_rope(dq, dg, d_table, d_first)

    # 9. given-scale E4M3 quantizer (quantize_columns_static_e4m3_kernel), specials included
    sy = wl.quantize_input_np(8, 512, seed=17)
    sy[0, :6] = [0x7F80, 0xFF80, 0x7FC0, 0x8000, 0x0000, 0x7F7F]
    fx["fs_in"], fx["fs_scale"] = sy, np.float32(0.0123)
    fx["fs_codes"] = rc.fp8_quantize_static_f32(rc.f32_dev(sy), 0.0123)

    path = out_dir / "reference_b200.npz"
    if path.exists():  # every array of the committed fixture must come out the same: the kernels are deterministic
        old = np.load(path)
        for name in old.files:
            assert np.array_equal(old[name], fx[name]), f"{name} changed"
    np.savez_compressed(path, **fx)
    print(f"wrote {path} ({path.stat().st_size} bytes, {len(fx)} arrays) on {torch.cuda.get_device_name(0)}")


if __name__ == "__main__":
    main()

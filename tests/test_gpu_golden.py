"""The CUDA path against the committed fixture of the reference's own kernels' outputs
(tests/golden/reference_b200.npz): bit-exact, with no reference tree or oracle/_ref needed at run time."""
import importlib
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")
FIXTURE = Path(__file__).resolve().parent / "golden" / "reference_b200.npz"


@pytest.fixture(scope="module")
def fx():
    return np.load(FIXTURE)


def test_nvfp4_quantizer(axk, cuda_device, fx):
    import torch
    from gpu_util import dev, sync

    for key_in, cases in (("q_in", [("q_G", "q_codes", "q_scales")]),
                          ("qs_in", [(f"qs_G_{t}", f"qs_codes_{t}", f"qs_scales_{t}") for t in "abc"])):
        x = fx[key_in]
        rows, cols = x.shape
        xd = dev(x)
        for g, c, s in cases:
            codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
            scales = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
            assert axk.nvfp4_quantize(0, xd, rows, cols, float(fx[g]), codes, scales, 0) == 0
            sync()
            assert np.array_equal(codes.cpu().numpy(), fx[c]) and np.array_equal(scales.cpu().numpy(), fx[s])
    x = fx["q_in"]
    plane = torch.zeros(fx["q_plane_warp"].size, dtype=torch.uint8, device="cuda")
    codes = torch.zeros((16, 2560), dtype=torch.uint8, device="cuda")
    xd = dev(x)
    assert axk.nvfp4_quantize(0, xd, 16, 5120, float(fx["q_G"]), codes, plane, 1) == 0
    sync()
    assert np.array_equal(plane.cpu().numpy(), fx["q_plane_warp"])


def test_add_rmsnorm_nvfp4(axk, cuda_device, fx):
    import torch
    from gpu_util import dev, host, sync

    h, r, g = dev(fx["n_hidden"]), dev(fx["n_residual"]), dev(fx["n_gamma"])
    norm = torch.zeros((8, 5120), dtype=torch.int16, device="cuda")
    codes = torch.zeros((8, 2560), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((8, 320), dtype=torch.uint8, device="cuda")
    assert axk.add_rmsnorm_nvfp4(0, h, r, g, 1e-6, 8, 5120, float(fx["n_G"]), norm, codes, scales, 0) == 0
    sync()
    assert np.array_equal(host(r, np.uint16).reshape(8, 5120), fx["n_res_out"])
    assert np.array_equal(host(norm, np.uint16).reshape(8, 5120), fx["n_norm"])
    assert np.array_equal(codes.cpu().numpy(), fx["n_codes"]) and np.array_equal(scales.cpu().numpy(), fx["n_scales"])
    r2 = dev(fx["n_residual"])
    assert axk.add_rmsnorm_nvfp4(0, None, r2, g, 1e-6, 8, 5120, 1.0, norm, None, None, 0) == 0
    sync()
    assert np.array_equal(host(norm, np.uint16).reshape(8, 5120), fx["n_norm_only"])
    assert np.array_equal(host(r2, np.uint16).reshape(8, 5120), fx["n_residual"])
    out = torch.zeros(4096, dtype=torch.int16, device="cuda")
    a, b = dev(fx["a_a"]), dev(fx["a_b"])
    assert axk.add_bf16(0, a, b, out, 4096) == 0
    sync()
    assert np.array_equal(host(out, np.uint16), fx["a_out"])


def test_fp8_and_swiglu(axk, cuda_device, fx):
    import torch
    from gpu_util import dev, sync

    for key, c, s, st in (("f_in", "f_codes", "f_scales", 0), ("f2_in", "f2_codes", "f2_scales", 4)):
        x = dev(fx[key])
        codes = torch.zeros((8, 1024), dtype=torch.uint8, device="cuda")
        scales = torch.zeros(8, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert axk.fp8_quantize(0, x, 8, 1024, codes, scales, status) == 0
        sync()
        assert np.array_equal(codes.cpu().numpy(), fx[c]) and np.array_equal(scales.cpu().numpy(), fx[s])
        assert int(status.item()) == st
    gu = dev(fx["s_in"])
    codes = torch.zeros((8, 2048), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(8, dtype=torch.float32, device="cuda")
    assert axk.swiglu_fp8(0, gu, 8, 2048, codes, scales) == 0
    sync()
    assert np.array_equal(scales.cpu().numpy(), fx["s_fp8_scales"]) and np.array_equal(codes.cpu().numpy(), fx["s_fp8_codes"])
    c4 = torch.zeros((8, 1024), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(fx["s_nv_plane"].size, dtype=torch.uint8, device="cuda")
    assert axk.swiglu_nvfp4(0, gu, 8, 2048, float(fx["s_G"]), c4, plane, 1) == 0
    sync()
    assert np.array_equal(c4.cpu().numpy(), fx["s_nv_codes"]) and np.array_equal(plane.cpu().numpy(), fx["s_nv_plane"])


def test_yarn_table_and_qk_norm_rope(axk, cuda_device, fx):
    import torch
    from gpu_util import dev, host, sync

    inv = torch.zeros(32, dtype=torch.float32, device="cuda")
    assert axk.yarn_inv_freq(0, 64, 1e7, 4.0, 262144.0, 32.0, 1.0, inv) == 0
    sync()
    assert np.array_equal(inv.cpu().numpy().view(np.uint32), fx["y_inv_freq"].view(np.uint32))
    for tag in ("lo", "hi"):
        base = int(fx[f"k_{tag}_base"])
        qd, kd, vd = dev(fx[f"k_{tag}_q"]), dev(fx[f"k_{tag}_k"]), dev(fx[f"k_{tag}_v"])
        qg, kg = dev(fx[f"k_{tag}_qg"]), dev(fx[f"k_{tag}_kg"])
        pos = dev((base + np.arange(8)).astype(np.uint32))
        k_out = torch.zeros((8, 4, 256), dtype=torch.int16, device="cuda")
        args = axk.make_qk_args(tokens=8, q_heads=24, k_heads=4, head_dim=256, rope_dim=64, eps=1e-6,
                                mscale=float(np.float32(1.138629436111989)), q=qd, k=kd, q_gamma=qg, k_gamma=kg,
                                inv_freq=inv, positions=pos, k_out=k_out)
        assert axk.qk_norm_rope_paged(0, args) == 0
        sync()
        assert np.array_equal(host(qd, np.uint16).reshape(8, 24, 256), fx[f"k_{tag}_q_out"])
        assert np.array_equal(host(k_out, np.uint16).reshape(8, 4, 256), fx[f"k_{tag}_k_out"])


def test_sigmoid_gate_and_e4m3_cache(axk, cuda_device, fx):
    import torch
    from gpu_util import dev, sync

    a, g = dev(fx["sg_attention"]), dev(fx["sg_gate"])
    y = torch.zeros(fx["sg_out"].shape, dtype=torch.int16, device="cuda")
    assert axk.sigmoid_gate_nvfp4(0, a, g, 8, 6144, 1.0, y, None, None, 0) == 0
    sync()
    assert np.array_equal(y.cpu().numpy().view(np.uint16), fx["sg_out"])
    # E4M3 cache rows of the reference for the "lo" q/k case (positions base..base+7 -> one 8-token block)
    inv = dev(fx["y_inv_freq"])
    qd, kd, qgd, kgd = dev(fx["k_lo_q"]), dev(fx["k_lo_k"]), dev(fx["k_lo_qg"]), dev(fx["k_lo_kg"])
    base = int(fx["k_lo_base"])
    positions = dev((base + np.arange(8)).astype(np.uint32))
    table = dev(np.zeros((1, (base + 8) // 8 + 1), np.int32))
    k_cache = torch.zeros((8, 1024), dtype=torch.uint8, device="cuda")
    args = axk.make_qk_args(tokens=8, q_heads=24, k_heads=4, head_dim=256, rope_dim=64, eps=1e-6,
                            mscale=float(np.float32(1.138629436111989)), flags=axk.QK_FLAG_CACHE_E4M3 | axk.QK_FLAG_RING,
                            block_tokens=8, n_layers=1, layer=0, pool_stride=1024, tbl_stride=1, n_blocks=1, q=qd, k=kd,
                            q_gamma=qgd, k_gamma=kgd, inv_freq=inv, positions=positions, block_tables=table, k_pool=k_cache)
    assert axk.qk_norm_rope_paged(0, args) == 0
    sync()
    got = k_cache.cpu().numpy()
    want = fx["k_lo_k_e4m3"]
    # with an 8-token block and a one-entry ring, position p lands in row p % 8
    rows = [(base + t) % 8 for t in range(8)]
    assert np.array_equal(got[rows], want)

"""BF16 -> NVFP4 activation quantizer: CUDA path (through the C ABI) vs the CPU oracle, bit-exact."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


def run_quantize(axk, x_bits, G, layout):
    import torch
    from gpu_util import Guarded, dev, sync

    rows, cols = x_bits.shape
    x = dev(x_bits)
    codes = Guarded(rows * cols // 2)
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, layout))
    scales = Guarded(nscale)
    if layout == axk.SCALE_TILED:
        scales.raw[scales.pad:scales.pad + nscale] = 0  # the plane's padding cells are the caller's (zero-filled)
    rc = axk.nvfp4_quantize(0, x, rows, cols, G, codes.ptr, scales.ptr, layout)
    sync()
    assert rc == axk.AXIOM_OK
    assert codes.guards_intact() and scales.guards_intact()
    return codes.payload().reshape(rows, cols // 2), scales.payload()


@pytest.mark.parametrize("rows,cols", [(1, 16), (3, 48), (2, 32), (7, 5120), (8, 5120), (9, 5120), (15, 1024),
                                        (16, 1024), (17, 1024), (129, 5120), (33, 17408)])
@pytest.mark.parametrize("layout", [0, 1])
def test_matches_oracle_bit_exact(axk, cuda_device, rows, cols, layout):
    x = wl.quantize_input_np(rows, cols, seed=rows * 131 + cols)
    amax = float(np.abs(wl.from_bf16_bits(x)).max())
    G = wl.nvfp4_global_scale(amax)
    codes, scales = run_quantize(axk, x, G, layout)
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    assert np.array_equal(codes, want_codes)
    if layout == 0:
        assert np.array_equal(scales.reshape(rows, cols // 16), want_scales)
    else:
        assert np.array_equal(scales, ol.scales_to_tiled(want_scales))


@pytest.mark.parametrize("rows,cols,layout", [(129, 5120, 0), (300, 1072, 1), (5, 48, 0)])
def test_code_buffer_aligned_to_four_bytes_only(axk, cuda_device, rows, cols, layout):
    """The block-per-lane kernel stores 8-byte code words; a code buffer that is only 4-byte aligned takes the
    chunk-per-lane kernel instead.  Same bytes."""
    import torch
    from gpu_util import dev, sync

    x = wl.quantize_input_np(rows, cols, seed=rows + cols)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(x)).max()))
    backing = torch.full((rows * cols // 2 + 64,), 0xFF, dtype=torch.uint8, device="cuda")
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, layout))
    scales = torch.zeros(nscale, dtype=torch.uint8, device="cuda")
    assert axk.nvfp4_quantize(0, dev(x), rows, cols, G, backing.data_ptr() + 4, scales, layout) == axk.AXIOM_OK
    sync()
    raw = backing.cpu().numpy()
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    assert np.array_equal(raw[4:4 + rows * cols // 2].reshape(rows, cols // 2), want_codes)
    assert (raw[:4] == 0xFF).all() and (raw[4 + rows * cols // 2:] == 0xFF).all()
    want_plane = want_scales.reshape(-1) if layout == 0 else ol.scales_to_tiled(want_scales)
    assert np.array_equal(scales.cpu().numpy(), want_plane)
    assert axk.nvfp4_quantize(0, dev(x), rows, cols, G, backing.data_ptr() + 2, scales, layout) == axk.AXIOM_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("G", [1.0, 0.37, 123.456, 2688.0 / 7.3, 3.3e4, 1e-3])
def test_global_scale_sweep(axk, cuda_device, G):
    x = wl.quantize_input_np(64, 2048, seed=11)
    codes, scales = run_quantize(axk, x, G, 0)
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    assert np.array_equal(codes, want_codes)
    assert np.array_equal(scales.reshape(64, 128), want_scales)


def test_special_values(axk, cuda_device):
    """zeros, signed zeros, NaN, infinities, denormals, BF16 extremes and exact rounding ties."""
    rows, cols = 16, 64
    x = np.zeros((rows, cols), np.float32)
    x[1, :16] = -0.0
    x[2, 3] = np.nan
    x[2, 5] = 1.0
    x[3, :16] = np.nan                      # all-NaN block: maximum 0 -> guard scale
    x[4, 0] = np.inf
    x[4, 1] = -np.inf
    x[4, 2] = 2.0
    x[5, :] = 3.3895314e38                  # BF16 max
    x[6, :8] = 1e-40                        # FP32 denormals (BF16 keeps some)
    x[7, :16] = [6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25, -6, -5, -3.5, -2.5, -1.75, -1.25, -0.75, -0.25]
    x[8, :16] = np.array([6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25] * 2, np.float32) * 0.5
    x[9, :] = 9.1835e-41
    x[10, ::2] = 1e30
    x[10, 1::2] = -1e-30
    rng = np.random.default_rng(5)
    x[11:] = rng.standard_normal((rows - 11, cols)).astype(np.float32) * np.float32(1e-3)
    bits = wl.to_bf16_bits(x)
    bits[2, 3] = 0x7fc0
    bits[3, :16] = 0xffc0
    for G in (1.0, 74.6, 1e4):
        codes, scales = run_quantize(axk, bits, G, 0)
        want_codes, want_scales = ol.nvfp4_quantize_bf16(bits, G)
        assert np.array_equal(scales.reshape(rows, cols // 16), want_scales), G
        assert np.array_equal(codes, want_codes), G


def test_config1_full_size(axk, cuda_device):
    """4096 x 5120, N(0,1) + 0.1 % x20 outliers, seed 0: whole tensor bit-exact, both scale layouts."""
    x = wl.quantize_input_np(4096, 5120, seed=0)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(x)).max()))
    want_codes, want_scales = ol.nvfp4_quantize_bf16(x, G)
    codes, scales = run_quantize(axk, x, G, 0)
    assert np.array_equal(codes, want_codes)
    assert np.array_equal(scales.reshape(4096, 320), want_scales)
    codes, scales = run_quantize(axk, x, G, 1)
    assert np.array_equal(codes, want_codes)
    assert np.array_equal(scales, ol.scales_to_tiled(want_scales))


def test_reference_named_row_entry(axk, cuda_device):
    """axiom_qwen38_nvfp4_quantize_reference_f32: one F32 row, canonical scales, synchronous."""
    import torch
    from gpu_util import Guarded

    rng = np.random.default_rng(3)
    for cols in (16, 5120, 17408):
        x = (rng.standard_normal(cols) * 2).astype(np.float32)   # genuine F32 values, not BF16-valued
        G = 37.5
        xd = torch.from_numpy(x).cuda()
        codes, scales = Guarded(cols // 2, align=1), Guarded(cols // 16, align=1)
        rc = axk.lib().axiom_qwen38_nvfp4_quantize_reference_f32(0, xd.data_ptr(), G, codes.ptr + 1 - 1, scales.ptr, cols, None)
        assert rc == axk.AXIOM_OK  # no explicit synchronize: the entry synchronises its stream
        want_codes, want_scales = ol.nvfp4_quantize_f32(x.reshape(1, cols), G)
        assert np.array_equal(codes.payload(), want_codes[0]) and np.array_equal(scales.payload(), want_scales[0])
        assert codes.guards_intact() and scales.guards_intact()


def test_rejected_calls_leave_outputs_untouched(axk, cuda_device):
    from gpu_util import Guarded, dev, sync

    x = dev(wl.quantize_input_np(4, 64))
    codes, scales = Guarded(4 * 32), Guarded(4 * 4)
    assert axk.nvfp4_quantize(0, x, 4, 48 + 8, 1.0, codes.ptr, scales.ptr) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert axk.nvfp4_quantize(0, x, 4, 64, -1.0, codes.ptr, scales.ptr) == axk.AXIOM_ERR_INVALID_ARGUMENT
    assert axk.nvfp4_quantize(0, x, 0, 64, 1.0, codes.ptr, scales.ptr) == axk.AXIOM_ERR_INVALID_ARGUMENT
    sync()
    assert codes.untouched() and scales.untouched()

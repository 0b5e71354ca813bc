"""Fused residual add + RMSNorm + NVFP4: CUDA path vs the CPU oracle.

Bars: the updated residual is bit-exact; the normalised values are within
1 BF16 ulp of the oracle (the device rsqrtf is an approximation, the oracle's
is correctly rounded); the NVFP4 codes and block scales are bit-exact with the
oracle quantizer applied to the kernel's own normalised values, and the two
kernels behind the entry point (one warp per row / one CTA per row) agree
bit-for-bit with each other."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")
EPS = 1e-6


def run(axk, hidden, residual, gamma, G, layout=0, want_norm=True, want_codes=True):
    from gpu_util import Guarded, dev, host, sync

    rows, cols = residual.shape
    h = dev(hidden) if hidden is not None else None
    r = dev(residual)
    g = dev(gamma)
    norm = Guarded(rows * cols * 2) if want_norm else None
    codes = Guarded(rows * cols // 2) if want_codes else None
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, layout))
    scales = Guarded(nscale) if want_codes else None
    if want_codes and layout == 1:
        scales.raw[scales.pad:scales.pad + nscale] = 0
    rc = axk.add_rmsnorm_nvfp4(0, h, r, g, EPS, rows, cols, G, norm.ptr if norm else None,
                               codes.ptr if codes else None, scales.ptr if scales else None, layout)
    sync()
    assert rc == axk.AXIOM_OK
    for buf in (norm, codes, scales):
        assert buf is None or buf.guards_intact()
    return (host(r, np.uint16).reshape(rows, cols),
            norm.payload(np.uint16).reshape(rows, cols) if norm else None,
            codes.payload().reshape(rows, cols // 2) if codes else None,
            scales.payload() if scales else None)


def check_against_oracle(axk, rows, cols, layout=0, with_add=True):
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    if not with_add:
        hidden = None
    want_res, want_norm = ol.add_rmsnorm_bf16(hidden, residual, gamma, EPS)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(want_norm)).max()))
    res, norm, codes, scales = run(axk, hidden, residual, gamma, G, layout)
    assert np.array_equal(res, want_res)                       # residual: bit-exact
    a, b = wl.from_bf16_bits(norm), wl.from_bf16_bits(want_norm)
    assert np.all(np.abs(a - b) <= ol.bf16_ulp(b))             # norm: within 1 BF16 ulp
    assert np.mean(norm != want_norm) < 0.02
    own_codes, own_scales = ol.nvfp4_quantize_bf16(norm, G)    # codes: bit-exact on the kernel's own values
    assert np.array_equal(codes, own_codes)
    if layout == 0:
        assert np.array_equal(scales.reshape(rows, cols // 16), own_scales)
    else:
        assert np.array_equal(scales, ol.scales_to_tiled(own_scales))
    _, _, full_codes, full_scales = ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, EPS, G)
    assert np.mean(codes != full_codes) < 0.02                 # end-to-end oracle: only rsqrt-ulp effects differ
    return res, norm, codes, scales


@pytest.mark.parametrize("rows", [1, 2, 7, 8, 9, 64])
@pytest.mark.parametrize("cols", [5120, 1024, 48, 8192, 16384])
def test_wide_row_kernel(axk, cuda_device, rows, cols):
    check_against_oracle(axk, rows, cols)


@pytest.mark.parametrize("rows,cols", [(300, 5120), (333, 1024), (512, 2048), (297, 4096), (301, 7168), (299, 8192),
                                        (310, 48), (305, 3072), (320, 6144)])
def test_streaming_kernel(axk, cuda_device, rows, cols):
    check_against_oracle(axk, rows, cols)


def test_tiled_scale_layout_and_norm_only(axk, cuda_device):
    check_against_oracle(axk, 384, 5120, layout=1)
    check_against_oracle(axk, 40, 5120, layout=1)
    check_against_oracle(axk, 300, 5120, with_add=False)
    check_against_oracle(axk, 5, 5120, with_add=False)


def test_both_kernels_agree_bit_for_bit(axk, cuda_device):
    """Rows 0..199 through the CTA-per-row kernel equal the same rows inside a 1024-row launch."""
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(1024, 5120)
    G = 150.0
    big = run(axk, hidden, residual, gamma, G)
    small = run(axk, hidden[:200], residual[:200], gamma, G)
    for a, b in zip(big, small):
        assert np.array_equal(a[:200] if a.ndim == 2 else a[:200 * 320], b)


def test_optional_outputs(axk, cuda_device):
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(300, 5120)
    full = run(axk, hidden, residual, gamma, 100.0)
    only_norm = run(axk, hidden, residual, gamma, 100.0, want_codes=False)
    only_codes = run(axk, hidden, residual, gamma, 100.0, want_norm=False)
    assert np.array_equal(full[1], only_norm[1]) and np.array_equal(full[2], only_codes[2])
    assert np.array_equal(full[3], only_codes[3]) and np.array_equal(full[0], only_norm[0])


def test_config2_full_size_properties(axk, cuda_device):
    """8192 x 5120: residual bit-exact against the oracle, codes consistent with the kernel's own norm."""
    rows, cols = 8192, 5120
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    want_res, want_norm = ol.add_rmsnorm_bf16(hidden, residual, gamma, EPS)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(want_norm)).max()))
    res, norm, codes, scales = run(axk, hidden, residual, gamma, G)
    assert np.array_equal(res, want_res)
    a, b = wl.from_bf16_bits(norm), wl.from_bf16_bits(want_norm)
    assert np.all(np.abs(a - b) <= ol.bf16_ulp(b))
    own_codes, own_scales = ol.nvfp4_quantize_bf16(norm, G)
    assert np.array_equal(codes, own_codes) and np.array_equal(scales.reshape(rows, cols // 16), own_scales)


def test_no_bounded_wait_ran_out(axk, cuda_device):
    """The pipelined kernels poll their shared-memory barriers a bounded number of times; none may have given up."""
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(2048, 5120)
    run(axk, hidden, residual, gamma, 100.0)
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0


def test_a_wait_that_runs_out_skips_its_rows_and_raises_the_fault_word(axk, cuda_device):
    """The give-up path of the bounded waits, exercised without faulting anything: the test hook makes the first
    row of one team announce 16 bytes more than its copies deliver, so that team's barrier never completes and its
    wait runs out after 2000 polls.  The kernel must return, the fault word must be raised, the rows of that team
    must keep their old contents (nothing is computed from a slot that was never declared complete), every other
    row must be what an undisturbed launch produces — and the next launch must be clean."""
    import torch
    from gpu_util import dev, host, sync

    rows, cols, G = 5000, 5120, 80.0
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    lib = axk.lib()

    def launch(arm):
        h, r, g = dev(hidden), dev(residual), dev(gamma)
        codes = torch.full((rows, cols // 2), 0xEE, dtype=torch.uint8, device="cuda")
        scales = torch.full((rows, cols // 16), 0xEE, dtype=torch.uint8, device="cuda")
        if arm:
            assert lib.axiom_b200_test_arm_wait_timeout(16, 2000) == axk.AXIOM_OK
        assert axk.add_rmsnorm_nvfp4(0, h, r, g, wl.EPS, rows, cols, G, None, codes, scales, 0) == axk.AXIOM_OK
        sync()
        return host(r, np.uint16).reshape(rows, cols), host(codes, np.uint8).reshape(rows, -1), host(scales, np.uint8).reshape(rows, -1)

    assert lib.axiom_b200_pipeline_faults(0) == 0
    want_res, want_codes, want_scales = launch(arm=False)
    assert lib.axiom_b200_pipeline_faults(0) == 0
    got_res, got_codes, got_scales = launch(arm=True)
    assert lib.axiom_b200_pipeline_faults(0) != 0          # raised ...
    assert lib.axiom_b200_pipeline_faults(0) == 0          # ... and cleared by the read
    skipped = np.flatnonzero((got_codes == 0xEE).all(axis=1))
    assert 0 in skipped and 1 <= skipped.size <= 8 and np.all(skipped % 148 == 0)   # rows of CTA 0 only, row 0 among them
    assert np.array_equal(got_res[skipped], residual[skipped])                       # untouched: residual not merged,
    assert (got_scales[skipped] == 0xEE).all()                                       # nothing quantized
    done = np.setdiff1d(np.arange(rows), skipped)
    assert np.array_equal(got_res[done], want_res[done]) and np.array_equal(got_codes[done], want_codes[done])
    assert np.array_equal(got_scales[done], want_scales[done])
    # the hook is one-shot: the next launch is undisturbed
    again = launch(arm=False)
    assert lib.axiom_b200_pipeline_faults(0) == 0
    for a, b in zip(again, (want_res, want_codes, want_scales)):
        assert np.array_equal(a, b)
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_b200_test_arm_wait_timeout(8, 100) == inv


def test_residual_add_over_all_exponents(axk, cuda_device):
    """Random finite BF16 bit patterns (every exponent, both signs, denormals): the merged residual is
    bf16(f32(a) + f32(b)) bit for bit, in the pipelined kernel (packed BF16 add) and in the CTA kernel."""
    from gpu_util import dev, host, sync
    import torch

    rng = np.random.default_rng(99)
    for rows in (512, 40):
        a = rng.integers(0, 65536, (rows, 5120)).astype(np.uint16)
        b = rng.integers(0, 65536, (rows, 5120)).astype(np.uint16)
        for arr in (a, b):
            arr[(arr & 0x7F80) == 0x7F80] &= 0x807F       # no inf / NaN patterns: make them denormals
        b[:, ::7] = a[:, ::7] ^ 0x8000                     # exact cancellation
        b[:, 1::7] = ((a[:, 1::7].astype(np.int32) + rng.integers(-3, 4, a[:, 1::7].shape)) & 0xFFFF).astype(np.uint16)
        b[(b & 0x7F80) == 0x7F80] &= 0x807F
        gamma = wl.to_bf16_bits(np.ones(5120, np.float32))
        r = dev(b)
        norm = torch.zeros((rows, 5120), dtype=torch.int16, device="cuda")
        hd, gd = dev(a), dev(gamma)
        assert axk.add_rmsnorm_nvfp4(0, hd, r, gd, 1e-6, rows, 5120, 1.0, norm, None, None, 0) == axk.AXIOM_OK
        sync()
        assert np.array_equal(host(r, np.uint16).reshape(rows, 5120), ol.add_bf16(a, b))


@pytest.mark.parametrize("rows", [8, 600])
@pytest.mark.parametrize("with_addend", [True, False])
def test_layer_tap_is_a_copy_of_the_updated_residual(axk, cuda_device, rows, with_addend):
    """The tap entry gives the plain entry's outputs plus a second copy of the residual rows as they leave
    (both kernels, add and norm-only modes)."""
    import torch
    from gpu_util import dev, host, sync

    cols = 5120
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    outs = []
    for tap_entry in (False, True):
        h, r, g = dev(hidden), dev(residual), dev(gamma)
        norm = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
        codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
        scales = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
        tap = torch.full((rows, cols), 0x5555, dtype=torch.int16, device="cuda")
        addend = h if with_addend else None
        if tap_entry:
            assert axk.add_rmsnorm_nvfp4_tap(0, addend, r, g, 1e-6, rows, cols, 80.0, norm, codes, scales, 0, tap) == axk.AXIOM_OK
        else:
            assert axk.add_rmsnorm_nvfp4(0, addend, r, g, 1e-6, rows, cols, 80.0, norm, codes, scales, 0) == axk.AXIOM_OK
        sync()
        outs.append([host(x, np.uint8) for x in (r, norm, codes, scales)])
        if tap_entry:
            assert np.array_equal(host(tap, np.uint16), host(r, np.uint16))
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
    assert axk.add_rmsnorm_nvfp4_tap(0, None, dev(residual), dev(gamma), 1e-6, rows, cols, 80.0, None, None, None, 0,
                                     None) == axk.AXIOM_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("rows,cols", [(8, 5120), (1, 1024), (600, 5120), (333, 2048), (300, 7168)])
def test_fp8_gemm_epilogue_folded_into_the_prologue(axk, cuda_device, rows, cols):
    """Raw F32 accumulators + per-feature BF16 weight scales + per-token input scales as the addend: the result equals
    the epilogue evaluated separately (oracle) followed by the plain BF16 entry, bit for bit; and the epilogue
    expression itself equals the reference's kernel on its 8-column batch."""
    import torch
    import ref_lib
    from gpu_util import dev, host, sync

    rng = np.random.default_rng(rows + cols)
    raw = (rng.standard_normal((rows, cols)) * 37.0).astype(np.float32)
    wscale = wl.to_bf16_bits((0.01 + 0.005 * rng.random(cols)).astype(np.float32))
    iscale = (0.02 + 0.01 * rng.random(rows)).astype(np.float32)
    _, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    addend = ol.fp8_row_scale_epilogue_bf16(raw, wscale, iscale)
    if ref_lib.available() and rows == 8:
        r = ref_lib.lib()
        out = torch.from_numpy(raw.copy()).cuda()
        ws_d, is_d = dev(wscale), torch.from_numpy(iscale).cuda()
        assert r.ref_fp8_group_row_scale_bf16_epilogue(out.data_ptr(), ws_d.data_ptr(), is_d.data_ptr(), cols) == 0
        assert np.array_equal(wl.to_bf16_bits(out.cpu().numpy()), addend)
        assert np.array_equal(wl.from_bf16_bits(addend), out.cpu().numpy())
    outs = []
    for fused in (False, True):
        res, g = dev(residual), dev(gamma)
        norm = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
        codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
        scales = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
        if fused:
            raw_d, ws_d, is_d = torch.from_numpy(raw).cuda(), dev(wscale), torch.from_numpy(iscale).cuda()
            assert axk.fp8_epilogue_add_rmsnorm_nvfp4(0, raw_d, ws_d, is_d, res, g, 1e-6, rows, cols, 70.0, norm, codes,
                                                      scales, 0) == axk.AXIOM_OK
        else:
            assert axk.add_rmsnorm_nvfp4(0, dev(addend), res, g, 1e-6, rows, cols, 70.0, norm, codes, scales, 0) == axk.AXIOM_OK
        sync()
        outs.append([host(x, np.uint8) for x in (res, norm, codes, scales)])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)

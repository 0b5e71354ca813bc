"""The allocation-free host-I/O quantize entry (fixed device array inside the library) against
the existing host-I/O entry (staging buffers the runtime allocates): same bytes, on two calls
in a row of different shapes and scale layouts — the second call finds the first one's bytes
in the array — and the size ceiling is enforced before anything is touched.  The file sorts
last on purpose: it must pass alone and after every other test has used the device."""
import ctypes as C
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _static_call(axk, x, G, layout):
    rows, cols = x.shape
    codes = np.full((rows, cols // 2), 0xAB, np.uint8)
    plane = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, layout))
    scales = np.full(plane, 0xCD, np.uint8)
    rc = axk.lib().axiom_b200_nvfp4_quantize_bf16_host_static(0, _p(x), rows, cols, G, layout, _p(codes), _p(scales), None)
    return rc, codes, scales


def test_static_entry_matches_runtime_entry_on_two_calls_in_a_row(axk, cuda_device):
    import torch

    lib = axk.lib()
    rt = axk.Runtime(0)
    calls = 0
    try:
        # call 1: tiled scale plane with padding (rows % 128 != 0, groups % 4 != 0); call 2: canonical, larger
        for rows, cols, layout, seed in ((200, 1072, axk.SCALE_TILED, 0), (600, 5120, axk.SCALE_CANONICAL, 1),
                                         (64, 48, axk.SCALE_TILED, 2)):
            x = wl.quantize_input_np(rows, cols, seed=seed)
            G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(x)).max()))
            want_codes = np.empty((rows, cols // 2), np.uint8)
            want_scales = np.empty((rows, cols // 16), np.uint8)
            assert lib.axiom_runtime_nvfp4_quantize_bf16(rt.handle, _p(x), rows, cols, G, _p(want_codes), _p(want_scales)) == 0
            free_before = torch.cuda.mem_get_info(0)[0] if calls else None
            rc, codes, scales = _static_call(axk, x, G, layout)
            assert rc == axk.AXIOM_OK
            if calls:  # after the first call on the device (which loads the array's module) nothing is reserved any more
                assert torch.cuda.mem_get_info(0)[0] == free_before
            calls += 1
            assert np.array_equal(codes, want_codes)
            want_plane = want_scales.reshape(-1) if layout == axk.SCALE_CANONICAL else ol.scales_to_tiled(want_scales)
            assert np.array_equal(scales, want_plane)  # includes the zero padding of the tiled plane
            oracle_codes, oracle_scales = ol.nvfp4_quantize_bf16(x, G)
            assert np.array_equal(codes, oracle_codes) and np.array_equal(want_scales, oracle_scales)
    finally:
        rt.close()


def test_static_entry_enforces_its_ceiling_and_arguments(axk, cuda_device):
    lib = axk.lib()
    limit = int(lib.axiom_b200_static_scratch_bytes())
    assert limit == 8 << 20
    cols = 5120
    per_row = cols * 2 + cols // 2 + cols // 16
    rows = limit // per_row + 2                      # just over the ceiling
    x = np.zeros((rows, cols), np.uint16)
    rc, codes, scales = _static_call(axk, x, 1.0, axk.SCALE_CANONICAL)
    assert rc == axk.AXIOM_ERR_BUDGET
    assert (codes == 0xAB).all() and (scales == 0xCD).all()   # nothing was written
    small = np.zeros((4, 32), np.uint16)
    out = np.zeros(64, np.uint8)
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert lib.axiom_b200_nvfp4_quantize_bf16_host_static(0, None, 4, 32, 1.0, 0, _p(out), _p(out), None) == inv
    assert lib.axiom_b200_nvfp4_quantize_bf16_host_static(0, _p(small), 4, 24, 1.0, 0, _p(out), _p(out), None) == inv
    assert lib.axiom_b200_nvfp4_quantize_bf16_host_static(0, _p(small), 4, 32, 0.0, 0, _p(out), _p(out), None) == inv
    assert lib.axiom_b200_nvfp4_quantize_bf16_host_static(0, _p(small), 4, 32, 1.0, 2, _p(out), _p(out), None) == inv

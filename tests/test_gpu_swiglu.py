"""SwiGLU + FP8 / NVFP4 quantize and the plain BF16 FP8 quantizer vs the CPU oracle.

The plain quantizer has no transcendental and is bit-exact.  SwiGLU uses the
device expf (<= 2 ulp) where the oracle uses the C library's, so y may differ in
the last FP32 bits: the per-token scale must agree to 4 FP32 ulps, almost all
codes must be identical, and EVERY code must be a correct rounding of the
FP64-evaluated y/scale up to that FP32 slack."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


def e4m3_table():
    return np.array([ol.o().axo_e4m3_decode(c) for c in range(256)], np.float64)


def run_swiglu_fp8(axk, gu):
    from gpu_util import Guarded, dev, sync

    rows, two_w = gu.shape
    w = two_w // 2
    x = dev(gu)
    codes, scales = Guarded(rows * w), Guarded(rows * 4)
    rc = axk.swiglu_fp8(0, x, rows, w, codes.ptr, scales.ptr)
    sync()
    assert rc == axk.AXIOM_OK and codes.guards_intact() and scales.guards_intact()
    return codes.payload().reshape(rows, w), scales.payload(np.float32)


def silu_mul_f64(gu):
    w = gu.shape[1] // 2
    g = wl.from_bf16_bits(gu[:, :w]).astype(np.float64)
    u = wl.from_bf16_bits(gu[:, w:]).astype(np.float64)
    return g / (1.0 + np.exp(-g)) * u


def check_swiglu_fp8(axk, rows, width, seed=4):
    gu = wl.swiglu_input_np(rows, width, seed)
    codes, scales = run_swiglu_fp8(axk, gu)
    want_codes, want_scales = ol.swiglu_fp8_bf16(gu)
    assert np.all(np.abs(scales - want_scales) <= 4 * np.spacing(want_scales))
    assert np.mean(codes != want_codes) < 2e-3
    assert fp8_codes_are_correct_roundings(gu, codes, scales)
    return codes, scales


@pytest.mark.parametrize("rows,width", [(1, 17408), (8, 17408), (5, 64), (3, 8), (64, 4096), (256, 17408),
                                         (7, 11008), (4, 36864), (9, 4608 - 8)])
def test_swiglu_fp8(axk, cuda_device, rows, width):
    check_swiglu_fp8(axk, rows, width)


def test_swiglu_fp8_special_rows(axk, cuda_device):
    w = 256
    x = np.zeros((6, 2 * w), np.float32)
    x[1, :w] = 1.0                                     # up = 0 -> y = 0 -> scale 1
    x[2, :w] = np.linspace(-90, 90, w)
    x[2, w:] = 1.0
    x[3, 0] = np.inf; x[3, w] = 1.0; x[3, 1] = 2.0; x[3, w + 1] = 3.0   # y = inf -> scale falls back to 1
    x[4, 5] = np.nan; x[4, w:] = 1.0; x[4, 7] = 4.0
    x[5, :w] = -200.0; x[5, w:] = 5.0                  # expf overflow: g/inf = -0
    gu = wl.to_bf16_bits(x)
    codes, scales = run_swiglu_fp8(axk, gu)
    want_codes, want_scales = ol.swiglu_fp8_bf16(gu)
    assert np.allclose(scales, want_scales, rtol=1e-6)
    assert scales[0] == 1.0 and scales[1] == 1.0 and scales[3] == 1.0
    assert np.mean(codes != want_codes) < 0.01
    assert np.array_equal(codes[[0, 1, 3, 5]], want_codes[[0, 1, 3, 5]])


def test_swiglu_fp8_special_rows_at_the_mlp_width(axk, cuda_device):
    """The same special rows where the row kernel runs with its geometry as compile-time constants (width 17408,
    enough rows for persistent CTAs with the silu table): zero rows, an infinite product, a NaN, gates beyond
    both ends of the table.  Bit-equal with the reference's kernels when they are built."""
    import ref_lib

    rows, w = 300, wl.FFN
    gu = wl.swiglu_input_np(rows, w, seed=11)
    x = np.zeros((6, 2 * w), np.float32)
    x[1, :w] = 1.0
    x[2, :w] = np.linspace(-90, 90, w); x[2, w:] = 1.0
    x[3, 0] = np.inf; x[3, w] = 1.0; x[3, 1] = 2.0; x[3, w + 1] = 3.0
    x[4, 5] = np.nan; x[4, w:] = 1.0; x[4, 7] = 4.0
    x[5, :w] = -200.0; x[5, w:] = 5.0
    special = [0, 1, 150, 151, 298, 299]
    gu[special] = wl.to_bf16_bits(x)
    gu[7, 17] = 0x0001          # a subnormal gate (under the table)
    gu[8, w - 1] = 0x4300       # 128.0: the first magnitude past the table
    gu[9, 3] = 0x8000           # -0
    codes, scales = run_swiglu_fp8(axk, gu)
    want_codes, want_scales = ol.swiglu_fp8_bf16(gu)
    assert np.all(np.abs(scales - want_scales) <= 4 * np.spacing(want_scales))
    assert scales[0] == 1.0 and scales[1] == 1.0 and scales[151] == 1.0
    assert np.mean(codes != want_codes) < 2e-3
    assert np.array_equal(codes[[0, 1, 151, 299]], want_codes[[0, 1, 151, 299]])
    if ref_lib.available():
        import ref_cases as rc

        ref_codes, ref_scales = rc.swiglu_fp8(gu)
        assert np.array_equal(scales, ref_scales)
        assert np.array_equal(codes, ref_codes)


def test_plain_fp8_quantizer_bit_exact(axk, cuda_device):
    from gpu_util import Guarded, dev, sync
    import torch

    # from 4 x 148 rows on the launcher prefers more chunks per thread in smaller CTAs
    for rows, cols in [(1, 8), (3, 5120), (8, 17408), (130, 1024), (5, 36864), (700, 8192), (600, 5120), (593, 17408),
                       (640, 264), (1200, 4096 + 8)]:
        x = wl.quantize_input_np(rows, cols, seed=cols)
        if rows >= 3:
            x[1, :] = 0
            x[2, 3] = 0x7f80  # +inf: skipped by the maximum, raises the status word
        xd = dev(x)
        codes, scales = Guarded(rows * cols), Guarded(rows * 4)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = axk.fp8_quantize(0, xd, rows, cols, codes.ptr, scales.ptr, status)
        sync()
        assert rc == axk.AXIOM_OK
        want_codes, want_scales, want_status = ol.fp8_quantize_bf16(x)
        assert np.array_equal(scales.payload(np.float32), want_scales)
        assert np.array_equal(codes.payload().reshape(rows, cols), want_codes)
        assert int(status.item()) == want_status
        assert codes.guards_intact() and scales.guards_intact()


def test_plain_fp8_quantizer_every_bf16_value(axk, cuda_device):
    """Every finite BF16 value under a row maximum M, for maxima from the smallest subnormal to the largest finite
    value (rows of one sign each, zero padded): scales and codes bit-equal with the oracle.  Then every one of the
    65536 patterns, NaN and infinities included, through the given-scale flavour at several scales."""
    from gpu_util import Guarded, dev, sync
    import torch

    cols = 32768
    maxima = [0x0001, 0x007f, 0x0080, 0x0c00, 0x3b80, 0x3f80, 0x43e0, 0x43e1, 0x4400, 0x5000, 0x7000, 0x7f00, 0x7f7f]
    rows = []
    for m in maxima:
        mags = np.arange(0, m + 1, dtype=np.uint16)
        for sign in (0x0000, 0x8000):
            row = np.zeros(cols, np.uint16)
            row[: mags.size] = mags | sign
            rows.append(np.roll(row, 37 * len(rows)))   # the maximum is not always in the first thread's chunk
    x = np.stack(rows)
    codes, scales = Guarded(x.size), Guarded(x.shape[0] * 4)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert axk.fp8_quantize(0, dev(x), x.shape[0], cols, codes.ptr, scales.ptr, status) == axk.AXIOM_OK
    sync()
    want_codes, want_scales, want_status = ol.fp8_quantize_bf16(x)
    assert np.array_equal(scales.payload(np.float32), want_scales)
    assert np.array_equal(codes.payload().reshape(x.shape), want_codes)
    assert int(status.item()) == want_status == 0 and codes.guards_intact() and scales.guards_intact()

    every = np.arange(65536, dtype=np.uint16).reshape(2, cols)
    for scale in (1.0, 0.0123, 3.0e-3, 1.0e-30, 1.0e30, 2.0 ** -126, 448.0):
        out = Guarded(every.size)
        assert axk.fp8_quantize_static(0, dev(every), 2, cols, scale, out.ptr) == axk.AXIOM_OK
        sync()
        want = ol.fp8_quantize_static_f32(wl.from_bf16_bits(every), scale)
        assert np.array_equal(out.payload().reshape(every.shape), want), scale
        assert out.guards_intact()


@pytest.mark.parametrize("rows,cols,scale", [(1, 8, 1.0), (5, 5120, 0.0123), (300, 1024, 3.0e-3), (7, 36864, 2.5), (64, 264, 1.0e-30),
                                              (700, 8192, 0.02), (600, 5120, 1.5), (640, 264, 7.0e-3)])
def test_static_scale_fp8_quantizer_bit_exact(axk, cuda_device, rows, cols, scale):
    """Given-scale E4M3 quantizer (no transcendental): bit-exact with the oracle, specials included."""
    from gpu_util import Guarded, dev, sync

    x = wl.quantize_input_np(rows, cols, seed=cols + rows)
    flat = x.reshape(-1)
    flat[:12] = wl.to_bf16_bits(np.array([0.0, -0.0, 448.0 * scale, -448.0 * scale, 1e30, -1e30, np.inf, -np.inf, np.nan,
                                           464.0 * scale, 1e-38, 3.0e38], np.float32))[: min(12, flat.size)]
    codes = Guarded(rows * cols)
    assert axk.fp8_quantize_static(0, dev(x), rows, cols, scale, codes.ptr) == axk.AXIOM_OK
    sync()
    assert codes.guards_intact()
    want = ol.fp8_quantize_static_f32(wl.from_bf16_bits(x), scale)
    assert np.array_equal(codes.payload().reshape(rows, cols), want)
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert axk.fp8_quantize_static(0, dev(x), rows, cols, 0.0, codes.ptr) == inv
    assert axk.fp8_quantize_static(0, dev(x), rows, cols, float("nan"), codes.ptr) == inv


@pytest.mark.parametrize("rows,width,scale", [(3, 64, 0.01), (40, 17408, 0.02), (600, 2048, 0.004)])
def test_static_scale_swiglu_fp8(axk, cuda_device, rows, width, scale):
    """SwiGLU with a given scale: every code is a correct rounding of the FP64 y / scale, and almost all equal the
    oracle's (device expf vs the C library's)."""
    from gpu_util import Guarded, dev, sync

    gu = wl.swiglu_input_np(rows, width, seed=rows)
    codes = Guarded(rows * width)
    assert axk.swiglu_fp8_static(0, dev(gu), rows, width, scale, codes.ptr) == axk.AXIOM_OK
    sync()
    assert codes.guards_intact()
    got = codes.payload().reshape(rows, width)
    want = ol.fp8_quantize_static_f32(ol.swiglu_f32(gu), scale)
    assert np.mean(got != want) < 2e-3
    assert fp8_codes_are_correct_roundings(gu, got, np.full(rows, scale, np.float32))


@pytest.mark.parametrize("rows,width,layout", [(1, 17408, 0), (8, 17408, 1), (3, 16, 0), (70, 1024, 1), (256, 17408, 0),
                                                (300, 1024, 1), (1000, 17408, 0), (333, 4096 + 256, 1), (297, 512 + 16, 0)])
def test_swiglu_nvfp4(axk, cuda_device, rows, width, layout):
    from gpu_util import Guarded, dev, sync

    gu = wl.swiglu_input_np(rows, width, seed=9)
    y = ol.swiglu_f32(gu)
    G = wl.nvfp4_global_scale(float(np.abs(y).max()))
    x = dev(gu)
    codes = Guarded(rows * width // 2)
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, width // 16, layout))
    scales = Guarded(nscale)
    if layout == 1:
        scales.raw[scales.pad:scales.pad + nscale] = 0
    rc = axk.swiglu_nvfp4(0, x, rows, width, G, codes.ptr, scales.ptr, layout)
    sync()
    assert rc == axk.AXIOM_OK and codes.guards_intact() and scales.guards_intact()
    want_codes, want_scales = ol.swiglu_nvfp4_bf16(gu, G)
    want_plane = want_scales.reshape(-1) if layout == 0 else ol.scales_to_tiled(want_scales)
    assert np.mean(scales.payload() != want_plane) < 2e-3
    assert np.mean(codes.payload().reshape(rows, width // 2) != want_codes) < 2e-3
    if layout == 0:  # and no code or scale is off by more than the FP32 slack of y allows
        assert nvfp4_codes_are_correct_roundings(gu, G, codes.payload().reshape(rows, width // 2),
                                                 scales.payload().reshape(rows, width // 16))


def test_swiglu_flavours_agree_bitwise(axk, cuda_device):
    """Few rows evaluate silu directly, more rows read it from the tabulated copy (device table copied into
    shared memory, or filled per CTA): the same 600 rows in calls of 8, of 40 and at once must give the same
    bytes — the table holds the direct expression's bits.  Includes gates outside the table's range."""
    import torch
    from gpu_util import dev, sync

    rows, width = 600, 2048
    gu = wl.swiglu_input_np(rows, width, seed=21)
    rng = np.random.default_rng(5)
    specials = wl.to_bf16_bits(np.array([0.0, -0.0, 1e-30, -1e-30, 200.0, -200.0, np.inf, -np.inf, np.nan, 127.9, 2.0 ** -57,
                                         2.0 ** -58], np.float32))
    idx = rng.integers(0, rows * width, 4000)
    gu[idx // width, idx % width] = specials[rng.integers(0, specials.size, idx.size)]  # gate half of the rows
    x = dev(gu)
    outs = []
    for step in (8, 40, rows):
        c4 = torch.zeros((rows, width // 2), dtype=torch.uint8, device="cuda")
        s4 = torch.zeros((rows, width // 16), dtype=torch.uint8, device="cuda")
        c8 = torch.zeros((rows, width), dtype=torch.uint8, device="cuda")
        s8 = torch.zeros((rows,), dtype=torch.float32, device="cuda")
        for lo in range(0, rows, step):
            n = min(step, rows - lo)
            assert axk.swiglu_nvfp4(0, x[lo:], n, width, 37.0, c4[lo:], s4[lo:], 0) == axk.AXIOM_OK
            assert axk.swiglu_fp8(0, x[lo:], n, width, c8[lo:], s8[lo:]) == axk.AXIOM_OK
        sync()
        outs.append([t.cpu().numpy() for t in (c4, s4, c8)] + [s8.cpu().numpy().view(np.uint32)])
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert np.array_equal(a, b)


def fp8_codes_are_correct_roundings(gu, codes, scales):
    """Every E4M3 code is a correct rounding of the FP64-evaluated y/scale, up to the FP32 slack of y."""
    table = e4m3_table()
    q = silu_mul_f64(gu) / scales.astype(np.float64)[:, None]
    got = table[codes]
    mag = codes & 0x7f
    step = np.where(mag < 8, 2.0 ** -9, np.exp2(np.floor(np.log2(np.maximum(np.abs(got), 2.0 ** -9))) - 3))
    ok = np.abs(got - q) <= 0.5 * step + (np.abs(q) * 2.0 ** -21 + 1e-30)
    ok |= (np.abs(q) >= 448.0) & (mag == 0x7e)
    return bool(np.all(ok))


E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float64)
E2M1_STEP = np.array([0.5, 0.5, 0.5, 0.5, 1.0, 1.0, 2.0, 2.0], np.float64)  # width of the rounding cell around a code


def nvfp4_codes_are_correct_roundings(gu, G, codes, scales):
    """Per-code bound for SwiGLU -> NVFP4 against an FP64 evaluation of y (no mismatch fraction):
    every block scale is a correct E4M3 rounding of max|y|/6*G and every nibble a correct E2M1 rounding of
    y / (e4m3(scale)/G), both up to the FP32 slack of y (device expf and the C library's differ in the last bits)."""
    rows, w = codes.shape[0], codes.shape[1] * 2
    y = silu_mul_f64(gu)
    table = e4m3_table()
    block_max = np.abs(y).reshape(rows, w // 16, 16).max(axis=2)
    want = block_max / 6.0 * float(np.float32(G))
    got = table[scales]
    mag = scales & 0x7f
    step = np.where(mag < 8, 2.0 ** -9, np.exp2(np.floor(np.log2(np.maximum(got, 2.0 ** -9))) - 3))
    ok_scale = np.abs(got - want) <= 0.5 * step + want * 2.0 ** -20 + 1e-30
    ok_scale |= (want >= 448.0) & (scales == 0x7e)
    ok_scale |= (want < 2.0 ** -10) & (scales == 0x20)   # a zero magnitude is stored as +0.125
    ok_scale |= (want <= 2.0 ** -10 * (1 + 2.0 ** -20)) & (scales == 0x01)
    if not np.all(ok_scale):
        return False
    d = np.repeat(got / float(np.float32(G)), 16, axis=1)
    q = y / d
    lo, hi = codes & 0xF, codes >> 4
    nib = np.empty((rows, w), np.uint8)
    nib[:, 0::2], nib[:, 1::2] = lo, hi
    val = E2M1_VALUES[nib & 7] * np.where(nib & 8, -1.0, 1.0)
    ok = np.abs(val - q) <= 0.5 * E2M1_STEP[nib & 7] + np.abs(q) * 2.0 ** -20 + 1e-30
    ok |= (np.abs(q) >= 6.0) & ((nib & 7) == 7)
    ok &= (np.signbit(q) == ((nib & 8) != 0)) | (val == 0.0) | (np.abs(q) < 0.25 * (1 + 2.0 ** -20))
    return bool(np.all(ok))


CONFIG4_REFERENCE_ROWS = np.r_[0:40, 8190:8231, 16344:16384]


def test_config4_full_size_fp8(axk, cuda_device):
    """Config 4 at its stated size, T = 16384 x 2*17408 (1.14 GB in: byte offsets beyond 2^31, the persistent
    grid wraps many times).  EVERY row is checked: scale within 4 FP32 ulps of the oracle's and every code a
    correct rounding of the FP64 y/scale; rows at the start, across the middle and at the end are bit-equal
    with the reference's own kernels (silu_mul_batch + quantize_columns_e4m3, 8 rows per launch)."""
    import torch
    import ref_lib
    from gpu_util import sync

    T, W = 16384, wl.FFN
    gu_dev = wl.swiglu_input_torch(torch, torch.device("cuda", 0), T, W, seed=4)
    codes = torch.full((T, W), 0xFF, dtype=torch.uint8, device="cuda")
    scales = torch.full((T,), float("nan"), dtype=torch.float32, device="cuda")
    assert axk.swiglu_fp8(0, gu_dev, T, W, codes, scales) == axk.AXIOM_OK
    sync()
    got_scales = scales.cpu().numpy()
    assert np.all(np.isfinite(got_scales))
    for r0 in range(0, T, 1024):
        gu = gu_dev[r0:r0 + 1024].view(torch.int16).cpu().numpy().view(np.uint16)
        c, s = codes[r0:r0 + 1024].cpu().numpy(), got_scales[r0:r0 + 1024]
        want_codes, want_scales = ol.swiglu_fp8_bf16(gu)
        assert np.all(np.abs(s - want_scales) <= 4 * np.spacing(want_scales)), f"scales of rows {r0}.."
        assert np.mean(c != want_codes) < 2e-3
        assert fp8_codes_are_correct_roundings(gu, c, s), f"a code of rows {r0}.. is not a correct rounding"
    if ref_lib.available():
        import ref_cases as rc

        rows = torch.from_numpy(CONFIG4_REFERENCE_ROWS).cuda()
        gu = gu_dev[rows].view(torch.int16).cpu().numpy().view(np.uint16)
        ref_codes, ref_scales = rc.swiglu_fp8(gu)
        assert np.array_equal(got_scales[CONFIG4_REFERENCE_ROWS], ref_scales)
        assert np.array_equal(codes[rows].cpu().numpy(), ref_codes)


def test_config4_full_size_nvfp4(axk, cuda_device):
    """The same tensor through SwiGLU -> NVFP4 (the down-projection input), all 16384 rows: per-code and
    per-scale bounds against an FP64 evaluation, and the rows listed above bit-equal with the reference's
    silu_mul_quantize_batch_to_tc kernels (thread and warp variants)."""
    import torch
    import ref_lib
    from gpu_util import sync

    T, W = 16384, wl.FFN
    G = 37.0
    gu_dev = wl.swiglu_input_torch(torch, torch.device("cuda", 0), T, W, seed=4)
    codes = torch.full((T, W // 2), 0xFF, dtype=torch.uint8, device="cuda")
    scales = torch.full((T, W // 16), 0xFF, dtype=torch.uint8, device="cuda")
    assert axk.swiglu_nvfp4(0, gu_dev, T, W, G, codes, scales, 0) == axk.AXIOM_OK
    sync()
    for r0 in range(0, T, 1024):
        gu = gu_dev[r0:r0 + 1024].view(torch.int16).cpu().numpy().view(np.uint16)
        c, s = codes[r0:r0 + 1024].cpu().numpy(), scales[r0:r0 + 1024].cpu().numpy()
        assert nvfp4_codes_are_correct_roundings(gu, G, c, s), f"rows {r0}..: a code or scale is not a correct rounding"
        want_codes, want_scales = ol.swiglu_nvfp4_bf16(gu, G)
        assert np.mean(c != want_codes) < 2e-3 and np.mean(s != want_scales) < 2e-3
    if ref_lib.available():
        import ref_cases as rc

        rows = torch.from_numpy(CONFIG4_REFERENCE_ROWS).cuda()
        gu = gu_dev[rows].view(torch.int16).cpu().numpy().view(np.uint16)
        got_codes, got_scales = codes[rows].cpu().numpy(), scales[rows].cpu().numpy()
        for variant in ("thread", "warp"):
            ref_codes, ref_plane = rc.swiglu_nvfp4(gu, G, variant)
            assert np.array_equal(got_codes, ref_codes)
            assert np.array_equal(ol.scales_to_tiled(got_scales), ref_plane)


@pytest.mark.parametrize("rows,width,layout", [(1, 6144, 0), (8, 8192, 1), (3, 16, 0), (120, 6144, 1), (400, 2048, 0),
                                                (600, 4096, 1), (310, 8192, 1), (299, 256 + 16, 0)])
def test_sigmoid_gate_nvfp4(axk, cuda_device, rows, width, layout):
    """y = bf16(attention * sigmoid(gate)) and its NVFP4 image vs the oracle: y within one BF16 ulp (device
    expf), codes re-derived bit-exactly from the kernel's own y."""
    import torch
    from gpu_util import Guarded, dev, sync

    rng = np.random.default_rng(rows * 7 + width)
    attn = wl.to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32))
    gate = wl.to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32) * np.float32(2.0))
    want_y, _, _ = ol.sigmoid_gate_nvfp4_bf16(attn, gate, 1.0)
    G = wl.nvfp4_global_scale(float(np.abs(wl.from_bf16_bits(want_y)).max()))
    a, g = dev(attn), dev(gate)
    y = Guarded(rows * width * 2)
    codes = Guarded(rows * width // 2)
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, width // 16, layout))
    scales = Guarded(nscale)
    if layout == 1:
        scales.raw[scales.pad:scales.pad + nscale] = 0
    assert axk.sigmoid_gate_nvfp4(0, a, g, rows, width, G, y.ptr, codes.ptr, scales.ptr, layout) == axk.AXIOM_OK
    sync()
    assert y.guards_intact() and codes.guards_intact() and scales.guards_intact()
    got_y = y.payload(np.uint16).reshape(rows, width)
    diff = np.abs(wl.from_bf16_bits(got_y) - wl.from_bf16_bits(want_y))
    assert np.all(diff <= ol.bf16_ulp(np.abs(wl.from_bf16_bits(want_y))) * np.float32(1.01))
    assert np.mean(got_y != want_y) < 5e-3
    # the codes are the quantizer's image of the kernel's own BF16 values, bit for bit
    want_codes, want_scales = ol.nvfp4_quantize_bf16(got_y, G)
    want_plane = want_scales.reshape(-1) if layout == 0 else ol.scales_to_tiled(want_scales)
    assert np.array_equal(codes.payload().reshape(rows, width // 2), want_codes)
    assert np.array_equal(scales.payload(), want_plane)
    # BF16-only and codes-only calls
    y2 = torch.zeros((rows, width), dtype=torch.int16, device="cuda")
    assert axk.sigmoid_gate_nvfp4(0, a, g, rows, width, G, y2, None, None, layout) == axk.AXIOM_OK
    sync()
    assert np.array_equal(y2.cpu().numpy().view(np.uint16), got_y)
    assert axk.sigmoid_gate_nvfp4(0, a, g, rows, width, G, None, None, None, layout) == axk.AXIOM_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("rows,heads,head_dim,layout", [(1, 64, 128, 0), (8, 24, 256, 1), (120, 5, 64, 1),
                                                         (400, 64, 128, 1), (37, 3, 128, 0)])
def test_sigmoid_gate_reads_gate_behind_each_head(axk, cuda_device, rows, heads, head_dim, layout):
    """Gate taken from the q-projection output [rows][heads][2 * head_dim] (query values, then gate values, per head):
    every output is bit-identical to the plain call on the de-interleaved gate plane, and the source is not written."""
    from gpu_util import Guarded, dev, host, sync

    width = heads * head_dim
    rng = np.random.default_rng(rows * 11 + heads)
    attn = wl.to_bf16_bits(rng.standard_normal((rows, width), dtype=np.float32))
    gate = wl.to_bf16_bits(rng.standard_normal((rows, heads, head_dim), dtype=np.float32) * np.float32(2.0))
    query = rng.integers(0, 1 << 16, gate.shape).astype(np.uint16)  # never read: any bit pattern
    q_gate = np.concatenate([query, gate], axis=-1)
    G = 300.0
    a, g, qg = dev(attn), dev(gate.reshape(rows, width)), dev(q_gate)
    nscale = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, width // 16, layout))
    outs = []
    for strided in (False, True):
        y, codes, scales = Guarded(rows * width * 2), Guarded(rows * width // 2), Guarded(nscale)
        if layout == 1:
            scales.raw[scales.pad:scales.pad + nscale] = 0
        if strided:
            rc = axk.sigmoid_gate_heads_nvfp4(0, a, qg, rows, heads, head_dim, G, y.ptr, codes.ptr, scales.ptr, layout)
        else:
            rc = axk.sigmoid_gate_nvfp4(0, a, g, rows, width, G, y.ptr, codes.ptr, scales.ptr, layout)
        sync()
        assert rc == axk.AXIOM_OK
        assert y.guards_intact() and codes.guards_intact() and scales.guards_intact()
        outs.append((y.payload(np.uint16).copy(), codes.payload().copy(), scales.payload().copy()))
    for plain, strided in zip(*outs):
        assert np.array_equal(plain, strided)
    assert np.array_equal(host(qg, np.uint16).reshape(q_gate.shape), q_gate)
    assert axk.sigmoid_gate_heads_nvfp4(0, a, qg, rows, heads, 96, G, None, None, None, layout) == axk.AXIOM_ERR_INVALID_ARGUMENT

"""Differential test on adversarial inputs: the CUDA path against the reference's own kernels (oracle/_ref) on
BF16 tensors drawn to hit the rare paths — uniformly random bit patterns (every exponent, NaN, infinities,
subnormals), per-row magnitudes over the whole FP32 exponent range, many exact ties, sprinkled special values — at
random shapes on both sides of every kernel switch (few rows / streaming, table / direct silu, chunks per thread),
with global scales and given scales over many decades.  Every comparison is bit-exact."""
import importlib

import numpy as np
import pytest

import ref_lib

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref is built only where the reference tree is present")]
wl = importlib.import_module("axiom-kernel_b200.workloads")

SPECIALS = np.array([0x0000, 0x8000, 0x7f80, 0xff80, 0x7fc0, 0xffc0, 0x0001, 0x8001, 0x007f, 0x0080, 0x7f7f, 0xff7f,
                     0x3f80, 0x43e0, 0x40c0], np.uint16)


def adversarial(rng, rows, cols):
    kind = rng.integers(0, 5)
    if kind == 0:
        return rng.integers(0, 65536, (rows, cols), dtype=np.uint16)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    with np.errstate(all="ignore"):
        if kind == 1:
            x *= np.float32(10.0) ** rng.uniform(-38, 38, (rows, 1)).astype(np.float32)
        elif kind == 2:
            x *= np.float32(2.0) ** rng.integers(-8, 8, (rows, cols)).astype(np.float32)
        elif kind == 3:
            x *= np.float32(10.0) ** rng.uniform(-3, 3, (rows, 1)).astype(np.float32)
        else:
            x = np.round(x * 4) / 4
        bits = wl.to_bf16_bits(x)
    n = rng.integers(0, max(2, rows * cols // 2000))
    bits.reshape(-1)[rng.integers(0, rows * cols, n)] = SPECIALS[rng.integers(0, SPECIALS.size, n)]
    return bits


def dev(a):
    import torch

    return torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()


def decade(rng, lo, hi):
    return float(np.float32(10.0 ** rng.uniform(lo, hi)))


@pytest.mark.parametrize("seed", range(12))
def test_quantizers_on_adversarial_tensors(axk, cuda_device, seed):
    import torch
    import ref_cases as rc

    rng = np.random.default_rng(1000 + seed)
    # BF16 -> NVFP4, tiled scale plane (the reference's thread kernel: it agrees with the exported entry on all-NaN blocks)
    rows, cols = int(rng.choice([1, 3, 17, 129, 300, 700])), int(rng.choice([16, 528, 1024, 5120, 17408]))
    rows = min(rows, max(1, 3_000_000 // cols))
    bits, G = adversarial(rng, rows, cols), decade(rng, -4, 5)
    codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, 1)), dtype=torch.uint8, device="cuda")
    assert axk.nvfp4_quantize(0, dev(bits), rows, cols, G, codes, plane, 1) == 0
    torch.cuda.synchronize()
    ref_codes, ref_plane = rc.nvfp4_quantize(bits, G, "thread")
    assert np.array_equal(codes.cpu().numpy(), ref_codes) and np.array_equal(plane.cpu().numpy(), ref_plane), (rows, cols, G)

    # BF16 -> FP8 rows: per-row scale with status word, and a given scale
    rows, cols = int(rng.choice([1, 5, 64, 300, 650])), int(rng.choice([8, 264, 1024, 5120, 8192, 17408]))
    rows = min(rows, max(1, 4_000_000 // cols))
    bits = adversarial(rng, rows, cols)
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert axk.fp8_quantize(0, dev(bits), rows, cols, codes, scales, status) == 0
    torch.cuda.synchronize()
    ref_codes, ref_scales, ref_status = rc.fp8_quantize_bf16(bits)
    assert np.array_equal(codes.cpu().numpy(), ref_codes), (rows, cols)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), ref_scales.view(np.uint32)) and int(status.item()) == ref_status
    scale = decade(rng, -30, 30)
    assert axk.fp8_quantize_static(0, dev(bits), rows, cols, scale, codes) == 0
    torch.cuda.synchronize()
    assert np.array_equal(codes.cpu().numpy(), rc.fp8_quantize_static_f32(rc.f32_dev(bits), scale)), (rows, cols, scale)


@pytest.mark.parametrize("seed", range(12))
def test_swiglu_on_adversarial_tensors(axk, cuda_device, seed):
    import torch
    import ref_cases as rc

    rng = np.random.default_rng(2000 + seed)
    rows, w = int(rng.choice([1, 8, 95, 96, 300, 600])), int(rng.choice([16, 512, 2048, 4096 + 256, 17408]))
    rows = min(rows, max(1, 2_500_000 // w))
    gu = adversarial(rng, rows, 2 * w)
    if seed % 2:  # gates a model produces, next to arbitrary up values
        gu[:, :w] = wl.to_bf16_bits(rng.standard_normal((rows, w)).astype(np.float32) * np.float32(rng.choice([0.5, 1.5, 8.0, 60.0])))
    c8 = torch.zeros((rows, w), dtype=torch.uint8, device="cuda")
    s8 = torch.zeros(rows, dtype=torch.float32, device="cuda")
    assert axk.swiglu_fp8(0, dev(gu), rows, w, c8, s8) == 0
    torch.cuda.synchronize()
    ref_codes, ref_scales = rc.swiglu_fp8(gu)
    assert np.array_equal(c8.cpu().numpy(), ref_codes), (rows, w)
    assert np.array_equal(s8.cpu().numpy().view(np.uint32), ref_scales.view(np.uint32))
    scale = decade(rng, -6, 6)
    assert axk.swiglu_fp8_static(0, dev(gu), rows, w, scale, c8) == 0
    torch.cuda.synchronize()
    assert np.array_equal(c8.cpu().numpy(), rc.fp8_quantize_static_f32(rc.swiglu_f32(gu), scale)), (rows, w, scale)
    G = decade(rng, -3, 4)
    c4 = torch.zeros((rows, w // 2), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, w // 16, 1)), dtype=torch.uint8, device="cuda")
    assert axk.swiglu_nvfp4(0, dev(gu), rows, w, G, c4, plane, 1) == 0
    torch.cuda.synchronize()
    ref_c4, ref_plane = rc.swiglu_nvfp4(gu, G, "thread")
    assert np.array_equal(c4.cpu().numpy(), ref_c4) and np.array_equal(plane.cpu().numpy(), ref_plane), (rows, w, G)


@pytest.mark.parametrize("seed", range(8))
def test_add_rmsnorm_nvfp4_on_adversarial_tensors(axk, cuda_device, seed):
    import torch
    import ref_cases as rc

    rng = np.random.default_rng(3000 + seed)
    rows, cols = int(rng.choice([8, 64, 296, 304, 1024])), 5120
    hidden, residual = adversarial(rng, rows, cols), adversarial(rng, rows, cols)
    gamma = wl.to_bf16_bits((1 + rng.standard_normal(cols) * rng.choice([0.02, 1.0])).astype(np.float32))
    with_add = bool(seed % 2)
    ref_res, ref_norm = rc.add_rmsnorm(hidden if with_add else None, residual, gamma)
    G = decade(rng, -4, 5)
    ref_codes, ref_plane = rc.nvfp4_quantize(ref_norm, G, "thread")
    r = dev(residual)
    norm = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
    codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
    plane = torch.zeros(ref_plane.size, dtype=torch.uint8, device="cuda")
    assert axk.add_rmsnorm_nvfp4(0, dev(hidden) if with_add else None, r, dev(gamma), 1e-6, rows, cols, G, norm, codes, plane, 1) == 0
    torch.cuda.synchronize()
    assert np.array_equal(r.cpu().numpy().view(np.uint16).reshape(rows, cols), ref_res)
    assert np.array_equal(norm.cpu().numpy().view(np.uint16).reshape(rows, cols), ref_norm)
    assert np.array_equal(codes.cpu().numpy(), ref_codes) and np.array_equal(plane.cpu().numpy(), ref_plane), (rows, with_add, G)


@pytest.mark.parametrize("tokens,seed", [(8, 0), (40, 1), (304, 2), (600, 3)])
def test_qk_norm_rope_on_adversarial_tensors(axk, cuda_device, tokens, seed):
    """q/k RMSNorm + partial NeoX RoPE (YaRN) at the reference's geometry (24 q / 4 kv heads x 256, rope_dim 64): the
    per-token kernel (few tokens) and the streaming kernel (from 296 tokens) against the reference's temporal-8 kernel
    run group by group, eight consecutive positions per group from a random base."""
    import torch
    import ref_cases as rc

    rng = np.random.default_rng(4000 + seed)
    H, KH, D = rc.REF_Q_HEADS, rc.REF_K_HEADS, rc.REF_HEAD_DIM
    q = adversarial(rng, tokens, H * D).reshape(tokens, H, D)
    k = adversarial(rng, tokens, KH * D).reshape(tokens, KH, D)
    v = wl.to_bf16_bits(rng.standard_normal((tokens, KH, D), dtype=np.float32))  # V is not part of this call: the reference just carries it
    qg = wl.to_bf16_bits(1.0 + 0.3 * rng.standard_normal(D, dtype=np.float32))
    kg = wl.to_bf16_bits(1.0 + 0.3 * rng.standard_normal(D, dtype=np.float32))
    bases = rng.integers(0, 250000, tokens // 8)
    positions = (bases[:, None] + np.arange(8)[None, :]).reshape(-1).astype(np.uint32)
    ref_q, ref_k = np.empty_like(q), np.empty_like(k)
    for g, base in enumerate(bases):
        s = slice(8 * g, 8 * g + 8)
        ref_q[s], ref_k[s], ref_v, _ = rc.qk_temporal8(q[s], k[s], v[s], qg, kg, int(base))
        assert np.array_equal(ref_v, v[s])
    inv = torch.zeros(32, dtype=torch.float32, device="cuda")
    assert axk.yarn_inv_freq(0, 64, rc.REF_THETA, rc.REF_YARN_FACTOR, rc.REF_YARN_CTX, 32.0, 1.0, inv) == 0
    qd, kd, qgd, kgd, pd = dev(q), dev(k), dev(qg), dev(kg), dev(positions)
    k_out = torch.zeros((tokens, KH, D), dtype=torch.int16, device="cuda")
    args = axk.make_qk_args(tokens=tokens, q_heads=H, k_heads=KH, head_dim=D, rope_dim=64, eps=1e-6, mscale=rc.REF_MSCALE,
                            q=qd, k=kd, q_gamma=qgd, k_gamma=kgd, inv_freq=inv, positions=pd, k_out=k_out)
    assert axk.qk_norm_rope_paged(0, args) == 0
    torch.cuda.synchronize()
    assert np.array_equal(qd.cpu().numpy().view(np.uint16).reshape(q.shape), ref_q)
    assert np.array_equal(k_out.cpu().numpy().view(np.uint16).reshape(k.shape), ref_k)


@pytest.mark.parametrize("seed", range(6))
def test_sigmoid_gate_on_adversarial_tensors(axk, cuda_device, seed):
    """attention * sigmoid(gate) rounded to BF16 (qwen38_sigmoid_gate_kernel on its [8 x 6144] batch), direct and
    through the tabulated flavour (the same rows repeated until the call is large enough for the table)."""
    import torch

    r = ref_lib.lib()
    rng = np.random.default_rng(5000 + seed)
    rows, width = 8, 6144
    attn, gate = adversarial(rng, rows, width), adversarial(rng, rows, width)
    if seed % 2:
        gate = wl.to_bf16_bits(rng.standard_normal((rows, width)).astype(np.float32) * np.float32(rng.choice([1.0, 6.0, 40.0])))
    a32 = torch.from_numpy(wl.from_bf16_bits(attn)).cuda()
    g32 = torch.from_numpy(wl.from_bf16_bits(gate)).cuda()
    out32 = torch.zeros_like(a32)
    assert r.ref_sigmoid_gate8(a32.data_ptr(), g32.data_ptr(), out32.data_ptr()) == 0
    want = out32.cpu().numpy().view(np.uint32)
    assert not (want & 0xFFFF).any()
    want = (want >> 16).astype(np.uint16)
    for reps in (1, 50):
        a, g = dev(np.tile(attn, (reps, 1))), dev(np.tile(gate, (reps, 1)))
        y = torch.zeros((rows * reps, width), dtype=torch.int16, device="cuda")
        assert axk.sigmoid_gate_nvfp4(0, a, g, rows * reps, width, 1.0, y, None, None, 0) == axk.AXIOM_OK
        torch.cuda.synchronize()
        got = y.cpu().numpy().view(np.uint16)
        nan = lambda b: (b & 0x7FFF) > 0x7F80
        same = (got[:rows] == want) | (nan(got[:rows]) & nan(want))       # NaN payloads are not part of the contract
        assert same.all(), reps
        assert np.array_equal(got[-rows:], got[:rows])


@pytest.mark.parametrize("seed", range(4))
def test_top1_on_adversarial_logits(axk, cuda_device, seed):
    """Greedy selection over F32 bit patterns with many ties, infinities and NaN, against both reference paths."""
    import torch
    import oracle_lib as ol

    r = ref_lib.lib()
    rng = np.random.default_rng(6000 + seed)
    vocab = 248320
    if seed == 0:
        logits = rng.integers(0, 2 ** 32, (8, vocab), dtype=np.uint32).view(np.float32)          # every pattern
    elif seed == 1:
        logits = np.round(rng.standard_normal((8, vocab)).astype(np.float32) * 2) / 2             # ties at the maximum
    elif seed == 2:
        logits = rng.standard_normal((8, vocab)).astype(np.float32)
        logits[rng.integers(0, 8, 4000), rng.integers(0, vocab, 4000)] = np.float32(np.inf)
        logits[3] = np.float32(-np.inf)
        logits[5, ::2] = np.float32(np.nan)
    else:
        logits = np.full((8, vocab), np.float32(-3.0e38))
        logits[:, -1] = np.float32(-2.9e38)                                                        # the winner is the last element
        logits[2] = np.float32(7.0)                                                                # all equal: id 0 wins
    x = torch.from_numpy(np.ascontiguousarray(logits)).cuda()
    partials = torch.zeros(8 * 256 * 3, dtype=torch.int32, device="cuda")
    out = torch.full((8, 3), 0x55555555, dtype=torch.int32, device="cuda")
    assert axk.top1(0, x, 8, vocab, out) == axk.AXIOM_OK
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, ol.top1_f32(logits))
    for hierarchical in (0, 1):
        res = torch.zeros((8, 3), dtype=torch.int32, device="cuda")
        assert r.ref_top1_8(x.data_ptr(), partials.data_ptr(), res.data_ptr(), hierarchical) == 0
        assert np.array_equal(res.cpu().numpy().view(np.uint32), got), hierarchical


@pytest.mark.parametrize("seed", range(4))
def test_round_after_norm_convention_on_adversarial_tensors(axk, cuda_device, seed):
    """The draft / SGLang convention (AXIOM_QK_FLAG_ROUND_AFTER_NORM) against qk_rmsnorm_rope_bf16_kernel + the BF16
    rounding pass on adversarial heads."""
    import torch
    import oracle_lib as ol
    import ref_cases as rc

    rng = np.random.default_rng(7000 + seed)
    heads, tokens, first = 40, int(rng.choice([8, 64, 320])), int(rng.integers(0, 20000))
    q = adversarial(rng, tokens, heads * 128).reshape(tokens, heads, 128)
    qg = wl.to_bf16_bits(1.0 + 0.3 * rng.standard_normal(128, dtype=np.float32))
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128, host_table=True)
    table = ol.rope_table_host(inv_freq, 128, float(ol.o().axo_yarn_mscale(4.0)), first + tokens)
    positions = (first + np.arange(tokens)).astype(np.uint32)
    want = rc.draft_qk_norm_rope(q, qg, table, first)
    qd, qgd, td, pd = dev(q), dev(qg), dev(table), dev(positions)
    args = axk.make_qk_args(tokens=tokens, q_heads=heads, k_heads=0, head_dim=128, rope_dim=128,
                            flags=axk.QK_FLAG_ROUND_AFTER_NORM, eps=1e-6, mscale=1.0, q=qd, q_gamma=qgd, positions=pd,
                            rope_table=td, rope_table_positions=table.shape[0])
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
    torch.cuda.synchronize()
    assert np.array_equal(qd.cpu().numpy().view(np.uint16).reshape(q.shape), want)


@pytest.mark.parametrize("seed", range(6))
def test_e4m3_kv_cache_on_adversarial_tensors(axk, cuda_device, seed):
    """The E4M3 (scale 1) cache flavour: K after norm + RoPE and V as they land in the cache rows, against the
    reference kernel's own cache bytes, for arbitrary K and V values (NaN, infinities, values beyond +-448)."""
    import torch
    import ref_cases as rc

    r = ref_lib.lib()
    H, KH, D = rc.REF_Q_HEADS, rc.REF_K_HEADS, rc.REF_HEAD_DIM
    rng = np.random.default_rng(8000 + seed)
    q, k, v = (adversarial(rng, 8, n * D).reshape(8, n, D) for n in (H, KH, KH))
    qg = wl.to_bf16_bits(1.0 + 0.3 * rng.standard_normal(D, dtype=np.float32))
    kg = wl.to_bf16_bits(1.0 + 0.3 * rng.standard_normal(D, dtype=np.float32))
    q32, k32, v32, qw, kw = rc.f32_dev(q), rc.f32_dev(k), rc.f32_dev(v), rc.f32_dev(qg), rc.f32_dev(kg)
    kc = torch.zeros((8, KH * D), dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    kref = torch.zeros((8, KH * D), dtype=torch.float32, device="cuda")
    vref = torch.zeros_like(kref)
    assert r.ref_qk_norm_partial_rope_cache_temporal8(q32.data_ptr(), k32.data_ptr(), qw.data_ptr(), kw.data_ptr(), v32.data_ptr(),
                                                      kc.data_ptr(), vc.data_ptr(), kref.data_ptr(), vref.data_ptr(), 0, 8, 1) == 0
    inv = torch.zeros(32, dtype=torch.float32, device="cuda")
    assert axk.yarn_inv_freq(0, 64, rc.REF_THETA, rc.REF_YARN_FACTOR, rc.REF_YARN_CTX, 32.0, 1.0, inv) == 0
    qd, kd, vd, qgd, kgd = dev(q), dev(k), dev(v), dev(qg), dev(kg)
    k_cache = torch.zeros((8, KH * D), dtype=torch.uint8, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    table, positions = dev(np.zeros((1, 1), np.int32)), dev(np.arange(8, dtype=np.uint32))
    args = axk.make_qk_args(tokens=8, q_heads=H, k_heads=KH, head_dim=D, rope_dim=64, eps=1e-6, mscale=rc.REF_MSCALE,
                            flags=axk.QK_FLAG_CACHE_E4M3, block_tokens=8, n_layers=1, layer=0, pool_stride=KH * D,
                            tbl_stride=1, n_blocks=1, q=qd, k=kd, v=vd, q_gamma=qgd, k_gamma=kgd, inv_freq=inv,
                            positions=positions, block_tables=table, k_pool=k_cache, v_pool=v_cache)
    assert axk.qk_norm_rope_paged(0, args) == 0
    torch.cuda.synchronize()
    assert np.array_equal(k_cache.cpu().numpy(), kc.cpu().numpy())
    assert np.array_equal(v_cache.cpu().numpy(), vc.cpu().numpy())

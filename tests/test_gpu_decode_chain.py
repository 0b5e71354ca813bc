"""Decode-shape sweep (M in {1, 8, 64, 256}) of the whole chain on one stream:
gather -> add + RMSNorm + NVFP4 -> q/k norm + RoPE + paged KV -> SwiGLU + NVFP4, each stage checked
against the oracle fed with the previous stage's own device output."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

from test_gpu_qk_rope import tolerance as qk_tolerance
from test_gpu_swiglu import nvfp4_codes_are_correct_roundings

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


@pytest.mark.parametrize("m", [1, 8, 64, 256])
def test_chain(axk, cuda_device, m):
    import torch
    from gpu_util import dev, host, sync

    stream = torch.cuda.Stream()
    table, ids = wl.embedding_inputs_np(m, vocab=4096, hidden=wl.HIDDEN)
    _, residual, gamma = wl.add_rmsnorm_inputs_np(m)
    q, k, v, qg, kg, positions, btab = wl.qk_inputs_np(m)
    gu = wl.swiglu_input_np(m)
    inv_freq = ol.yarn_inv_freq(wl.ROPE_THETA, wl.YARN_FACTOR, wl.YARN_ORIGINAL_CONTEXT, 32.0, 1.0, wl.HEAD_DIM)
    mscale = axk.yarn_mscale(wl.YARN_FACTOR)

    d = {n: dev(a) for n, a in dict(table=table, ids=ids, residual=residual, gamma=gamma, q=q, k=k, qg=qg, kg=kg,
                                    positions=positions, btab=btab, gu=gu, inv_freq=inv_freq).items()}
    hidden = torch.empty((m, wl.HIDDEN), dtype=torch.int16, device="cuda")
    norm = torch.empty_like(hidden)
    codes = torch.empty((m, wl.HIDDEN // 2), dtype=torch.uint8, device="cuda")
    scales = torch.empty((m, wl.HIDDEN // 16), dtype=torch.uint8, device="cuda")
    pool = torch.full((wl.KV_BLOCKS * 16 * 1024,), -1, dtype=torch.int16, device="cuda")
    k_out = torch.empty((m, 8, 128), dtype=torch.int16, device="cuda")
    mlp_codes = torch.empty((m, wl.FFN // 2), dtype=torch.uint8, device="cuda")
    mlp_scales = torch.empty((m, wl.FFN // 16), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    G1, G2 = 90.0, 40.0
    args = axk.make_qk_args(tokens=m, q_heads=64, k_heads=8, head_dim=128, rope_dim=128, flags=axk.QK_FLAG_RING,
                            eps=1e-6, mscale=mscale, block_tokens=16, n_layers=1, layer=0, pool_stride=1024,
                            tbl_stride=wl.KV_BLOCKS, n_blocks=wl.KV_BLOCKS, q=d["q"], k=d["k"], q_gamma=d["qg"],
                            k_gamma=d["kg"], inv_freq=d["inv_freq"], positions=d["positions"], block_tables=d["btab"],
                            k_pool=pool, k_out=k_out, status_word=status)
    with torch.cuda.stream(stream):
        ok = axk.AXIOM_OK
        assert axk.embedding_gather(0, d["table"], 4096, wl.HIDDEN, d["ids"], m, hidden, status, stream) == ok
        assert axk.add_rmsnorm_nvfp4(0, hidden, d["residual"], d["gamma"], 1e-6, m, wl.HIDDEN, G1, norm, codes, scales, 0, stream) == ok
        assert axk.qk_norm_rope_paged(0, args, stream) == ok
        assert axk.swiglu_nvfp4(0, d["gu"], m, wl.FFN, G2, mlp_codes, mlp_scales, 0, stream) == ok
    stream.synchronize()
    assert int(status.item()) == 0

    got_hidden = host(hidden, np.uint16)
    assert np.array_equal(got_hidden, ol.embedding_gather_bf16(table, ids))
    want_res, want_norm = ol.add_rmsnorm_bf16(got_hidden, residual, gamma, 1e-6)
    assert np.array_equal(host(d["residual"], np.uint16), want_res)
    got_norm = host(norm, np.uint16)
    assert np.all(np.abs(wl.from_bf16_bits(got_norm) - wl.from_bf16_bits(want_norm)) <= ol.bf16_ulp(wl.from_bf16_bits(want_norm)))
    own_codes, own_scales = ol.nvfp4_quantize_bf16(got_norm, G1)
    assert np.array_equal(host(codes, np.uint8), own_codes) and np.array_equal(host(scales, np.uint8), own_scales)
    want_q, want_k, _ = ol.qk_norm_rope_paged(q, k, None, qg, kg, inv_freq, positions, btab, rope_dim=128, eps=1e-6,
                                              mscale=mscale, want_k_out=True)
    for got, want, src, g_bits in ((host(d["q"], np.uint16).reshape(q.shape), want_q, q, qg),
                                   (host(k_out, np.uint16).reshape(k.shape), want_k, k, kg)):
        # one BF16 ulp at the magnitude of the rotation terms, on every element (device cosf/sinf vs the C library's)
        bound = qk_tolerance(src, g_bits, inv_freq, positions, 128, mscale)
        assert np.all(np.abs(wl.from_bf16_bits(got) - wl.from_bf16_bits(want)) <= bound)
        assert np.mean(got != want) < 0.02
    cells = host(pool, np.uint16).reshape(wl.KV_BLOCKS, 16, 1024)
    lb = (positions // 16) % wl.KV_BLOCKS
    assert np.array_equal(cells[btab[0, lb], positions % 16], host(k_out, np.uint16).reshape(m, 1024))
    want_mc, want_ms = ol.swiglu_nvfp4_bf16(gu, G2)
    got_mc, got_ms = host(mlp_codes, np.uint8).reshape(want_mc.shape), host(mlp_scales, np.uint8).reshape(want_ms.shape)
    assert np.mean(got_mc != want_mc) < 2e-3 and np.mean(got_ms != want_ms) < 2e-3
    # and every code and block scale is a correct rounding of the FP64 value up to the FP32 slack of expf
    assert nvfp4_codes_are_correct_roundings(gu, G2, got_mc, got_ms)


@pytest.mark.parametrize("m,cols", [(1, 5120), (8, 5120), (64, 1024), (300, 5120), (700, 2048)])
def test_gather_fused_into_the_first_norm(axk, cuda_device, m, cols):
    """gather + add + RMSNorm + NVFP4 in one launch gives the bytes of the two-launch sequence, including rows
    whose token id is out of range (zero addend, status word raised)."""
    import torch
    from gpu_util import dev, host, sync

    table, ids = wl.embedding_inputs_np(m, vocab=2048, hidden=cols)
    bad = m >= 8
    if bad:
        ids[3] = 2048
        ids[m - 1] = 0xFFFFFFFF
    _, residual, gamma = wl.add_rmsnorm_inputs_np(m, cols)
    G = 75.0
    outs = []
    for fused in (False, True):
        t, i, r, g = dev(table), dev(ids), dev(residual), dev(gamma)
        norm = torch.zeros((m, cols), dtype=torch.int16, device="cuda")
        codes = torch.zeros((m, cols // 2), dtype=torch.uint8, device="cuda")
        scales = torch.zeros((m, cols // 16), dtype=torch.uint8, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        if fused:
            assert axk.gather_add_rmsnorm_nvfp4(0, t, 2048, i, r, g, 1e-6, m, cols, G, norm, codes, scales, 0, status) == axk.AXIOM_OK
        else:
            hidden = torch.zeros((m, cols), dtype=torch.int16, device="cuda")
            assert axk.embedding_gather(0, t, 2048, cols, i, m, hidden, status) == axk.AXIOM_OK
            assert axk.add_rmsnorm_nvfp4(0, hidden, r, g, 1e-6, m, cols, G, norm, codes, scales, 0) == axk.AXIOM_OK
        sync()
        assert int(status.item()) == (axk.STATUS_WORD_BAD_ADDRESS if bad else 0)
        outs.append([host(x, np.uint8) for x in (r, norm, codes, scales)])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def test_back_to_back_launches_respect_stream_order(axk, cuda_device):
    """Every kernel may be scheduled before its predecessor on the stream has finished (programmatic dependent
    launch) and must not touch memory before the dependency resolves.  Forty dependent launches — each adds the
    previous result into the residual in place, alternating the streaming and the wide-row kernel, and quantizes
    what the previous launch wrote — must give the bytes of forty synchronised launches."""
    import torch
    from gpu_util import dev, host, sync

    rows, cols = 600, 5120
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(rows, cols)
    small = 40  # rows of the wide-row launches
    results = []
    for synchronise in (True, False):
        h, r, g = dev(hidden), dev(residual), dev(gamma)
        norm = torch.zeros((rows, cols), dtype=torch.int16, device="cuda")
        codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
        scales = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
        q4 = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
        s4 = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
        for it in range(40):
            n = rows if it % 2 == 0 else small
            assert axk.add_rmsnorm_nvfp4(0, h, r, g, 1e-6, n, cols, 50.0, norm, codes, scales, 0) == axk.AXIOM_OK
            # the next launch reads what this one wrote (norm) and the one after overwrites it again
            assert axk.nvfp4_quantize(0, norm, n, cols, 50.0, q4, s4, 0) == axk.AXIOM_OK
            assert axk.add_bf16(0, norm, h, h, n * cols) == axk.AXIOM_OK  # and feeds the addend of the next round
            if synchronise:
                sync()
        sync()
        results.append([host(x, np.uint8) for x in (h, r, norm, codes, scales, q4, s4)])
    for a, b in zip(*results):
        assert np.array_equal(a, b)

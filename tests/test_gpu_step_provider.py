"""The step-engine forward_step provider on a ragged batch, the test playing the engine's part
(tools/axiom_engine.cpp: select the active sequences, upload their block-table rows and (cache length, position)
metadata, call ops.forward_step once; include/axiom/axiom_engine.h:183-198,218-225).

Every contraction hook is a stand-in that delivers a seeded BF16 tensor (the contractions are the integrator's), so
what is checked is everything the provider itself does, against the CPU oracle fed with the same tensors:
the embedding rows of next_tok, every norm, the NVFP4 operands handed to the MLP hooks, the residual stream after all
layers, the logits landing in each sequence's own host buffer — and, in the manner of the reference's paged-attention
parity tool (tools/axiom_paged_attn_parity_smoke.cpp:207-241), the paged KV pools: 0xFF-poisoned before the step,
afterwards every (layer, sequence) row sits at the address recomputed on the host from that sequence's own table row
and position, and every other byte still carries the poison."""
import ctypes as C
import importlib

import numpy as np
import pytest

import oracle_lib as ol

from test_gpu_qk_rope import tolerance as qk_tolerance

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")
eng = importlib.import_module("axiom-kernel_b200.engine")

LAYERS, HIDDEN, FFN, QH, KH, D, VOCAB = 3, 1024, 2048, 8, 2, 128, 4096
BT, NPHYS, CAP, TBL_STRIDE = 16, 40, 8, 12


def test_forward_step_on_a_ragged_batch(axk, cuda_device):
    import torch
    from gpu_util import dev, host, sync

    lib = axk.lib()
    cudart = C.CDLL("libcudart.so.12")
    cudart.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    rng = np.random.default_rng(77)
    bf = lambda *shape, s=1.0: wl.to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(s))
    gam = lambda *shape: wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(shape, dtype=np.float32))
    n = 5                                                     # active sequences of this step
    table = bf(VOCAB, HIDDEN, s=0.05)
    in_gamma, post_gamma, final_gamma = gam(LAYERS, HIDDEN), gam(LAYERS, HIDDEN), gam(HIDDEN)
    qg, kg = gam(LAYERS, D), gam(LAYERS, D)
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, D)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    G_in, G_mid = 70.0, 30.0
    # what the contraction hooks deliver, per layer
    stand = [dict(q=bf(n, QH, D), k=bf(n, KH, D), v=bf(n, KH, D), mixer=bf(n, HIDDEN), gate_up=bf(n, 2 * FFN, s=1.5),
                  mlp=bf(n, HIDDEN, s=0.5)) for _ in range(LAYERS)]
    logits = rng.standard_normal((n, VOCAB)).astype(np.float32)
    d_stand = [{k: dev(v) for k, v in L.items()} for L in stand]
    d_logits = torch.from_numpy(logits).cuda()
    seen = dict(norm=[], in_codes=[], in_scales=[], mid_codes=[], mid_scales=[], final=None, calls=[])

    def copy(dst, src_tensor, stream):
        return cudart.cudaMemcpyAsync(dst, src_tensor.data_ptr(), src_tensor.numel() * src_tensor.element_size(), 3, stream)

    def snapshot(ptr, nbytes, stream):
        t = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        assert cudart.cudaMemcpyAsync(t.data_ptr(), ptr, nbytes, 3, stream) == 0
        return t

    plane_in = int(lib.axiom_nvfp4_scale_plane_bytes(n, HIDDEN // 16, 1))
    plane_mid = int(lib.axiom_nvfp4_scale_plane_bytes(n, FFN // 16, 1))

    @eng.QKV_HOOK
    def qkv(user, layer, rows, norm, q, k, v, stream):
        seen["calls"].append(("qkv", layer, rows))
        seen["norm"].append(snapshot(norm, rows * HIDDEN * 2, stream))
        L = d_stand[layer]
        return copy(q, L["q"], stream) | copy(k, L["k"], stream) | copy(v, L["v"], stream)

    @eng.ATTENTION_HOOK
    def attention(user, layer, rows, q, dev_view, mixer_out, stream):
        seen["calls"].append(("attention", layer, rows))
        seen.setdefault("q_after", []).append(snapshot(q, rows * QH * D * 2, stream))
        assert dev_view.contents.cap == CAP and dev_view.contents.tbl_stride == TBL_STRIDE
        return copy(mixer_out, d_stand[layer]["mixer"], stream)

    @eng.NVFP4_GEMM_HOOK
    def gate_up(user, layer, rows, codes, scales, out, stream):
        seen["calls"].append(("gate_up", layer, rows))
        seen["in_codes"].append(snapshot(codes, rows * HIDDEN // 2, stream))
        seen["in_scales"].append(snapshot(scales, plane_in, stream))
        return copy(out, d_stand[layer]["gate_up"], stream)

    @eng.NVFP4_GEMM_HOOK
    def down(user, layer, rows, codes, scales, out, stream):
        seen["calls"].append(("down", layer, rows))
        seen["mid_codes"].append(snapshot(codes, rows * FFN // 2, stream))
        seen["mid_scales"].append(snapshot(scales, plane_mid, stream))
        return copy(out, d_stand[layer]["mlp"], stream)

    @eng.LM_HEAD_HOOK
    def lm_head(user, rows, final_norm, out, stream):
        seen["calls"].append(("lm_head", rows))
        seen["final"] = snapshot(final_norm, rows * HIDDEN * 2, stream)
        return copy(out, d_logits, stream)

    # ---- the engine's part: arena pools, block-table matrix, metadata, sequences ----
    rt = axk.Runtime(0)
    kv_dim = KH * D
    pool_bytes = NPHYS * LAYERS * BT * kv_dim * 2
    kpool, vpool = axk.DeviceBuffer(rt, pool_bytes), axk.DeviceBuffer(rt, pool_bytes)
    d_tbl, d_meta = axk.DeviceBuffer(rt, CAP * TBL_STRIDE * 4), axk.DeviceBuffer(rt, 2 * CAP * 4)
    poison = np.full(pool_bytes, 0xFF, np.uint8)
    kpool.upload(poison)
    vpool.upload(poison)
    positions = np.array([0, 17, 63, 100, 191], np.uint32)[:n]          # ragged cache lengths
    htbl = np.full((CAP, TBL_STRIDE), -1, np.int32)
    blocks = rng.permutation(NPHYS)
    used = 0
    for a in range(n):
        need = int(positions[a]) // BT + 1
        htbl[a, :need] = blocks[used:used + need]
        used += need
    hmeta = np.zeros(2 * CAP, np.uint32)
    hmeta[:n] = positions + 1
    hmeta[CAP:CAP + n] = positions
    d_tbl.upload(htbl)
    d_meta.upload(hmeta)
    ids = rng.integers(0, VOCAB, n).astype(np.uint32)
    seq_logits = [np.zeros(VOCAB, np.float32) for _ in range(n)]
    seqs = (eng.EngineSeq * n)()
    for a in range(n):
        seqs[a].sid = 100 + a
        seqs[a].pos = int(positions[a])
        seqs[a].next_tok = int(ids[a])
        seqs[a].seq_logits = seq_logits[a].ctypes.data_as(C.POINTER(C.c_float))
    active = (C.POINTER(eng.EngineSeq) * n)(*[C.pointer(seqs[a]) for a in range(n)])
    view = eng.EngineDev(rt.handle, kpool.handle, vpool.handle, d_tbl.handle, d_meta.handle, CAP, TBL_STRIDE, None, None)

    model = dict(table=dev(table), in_gamma=dev(in_gamma), post_gamma=dev(post_gamma), final_gamma=dev(final_gamma),
                 qg=dev(qg), kg=dev(kg), inv_freq=dev(inv_freq))
    hooks = eng.ContractionHooks(None, qkv, attention, gate_up, down, lm_head)
    cfg = eng.StepProviderConfig(axk.AXIOM_ABI_VERSION, C.sizeof(eng.StepProviderConfig), LAYERS, HIDDEN, FFN, QH, KH, D, D, VOCAB,
                                 CAP, BT, NPHYS, kv_dim, 1e-6, mscale, G_in, G_mid, model["table"].data_ptr(),
                                 model["in_gamma"].data_ptr(), model["post_gamma"].data_ptr(), model["final_gamma"].data_ptr(),
                                 model["qg"].data_ptr(), model["kg"].data_ptr(), model["inv_freq"].data_ptr(), hooks)
    provider = C.c_void_p()
    assert lib.axiom_b200_step_provider_create(rt.handle, C.byref(cfg), C.byref(provider)) == axk.AXIOM_OK
    try:
        rc = lib.axiom_b200_step_provider_forward_step(provider, active, n, C.byref(view))
        assert rc == axk.AXIOM_OK
        sync()
        order = [c[0] for c in seen["calls"]]
        assert order == ["qkv", "attention", "gate_up", "down"] * LAYERS + ["lm_head"] and all(c[-1] == n for c in seen["calls"])

        # ---- the residual stream and every norm / NVFP4 operand, against the oracle ----
        residual = ol.embedding_gather_bf16(table, ids)
        u16 = lambda t, *shape: t.cpu().numpy().view(np.uint16).reshape(*shape)
        want_k_rows, want_v_rows, k_bounds = [], [], []
        for L in range(LAYERS):
            _, want_norm = ol.add_rmsnorm_bf16(np.zeros_like(residual), residual, in_gamma[L], 1e-6)
            got_norm = u16(seen["norm"][L], n, HIDDEN)
            assert np.all(np.abs(wl.from_bf16_bits(got_norm) - wl.from_bf16_bits(want_norm)) <= ol.bf16_ulp(wl.from_bf16_bits(want_norm)))
            want_q, want_k, _ = ol.qk_norm_rope_paged(stand[L]["q"], stand[L]["k"], None, qg[L], kg[L], inv_freq, positions, None,
                                                      rope_dim=D, eps=1e-6, mscale=mscale, want_k_out=True)
            got_q = u16(seen["q_after"][L], n, QH, D)
            assert np.mean(got_q != want_q) < 0.02
            assert np.all(np.abs(wl.from_bf16_bits(got_q) - wl.from_bf16_bits(want_q)) <=
                          qk_tolerance(stand[L]["q"], qg[L], inv_freq, positions, D, mscale))
            want_k_rows.append(want_k)
            k_bounds.append(qk_tolerance(stand[L]["k"], kg[L], inv_freq, positions, D, mscale))
            want_v_rows.append(stand[L]["v"])
            residual, post_norm = ol.add_rmsnorm_bf16(stand[L]["mixer"], residual, post_gamma[L], 1e-6)
            codes, scales = ol.nvfp4_quantize_bf16(post_norm, G_in)
            got_codes = seen["in_codes"][L].cpu().numpy().reshape(n, HIDDEN // 2)
            assert np.mean(got_codes != codes) < 0.02           # the norm under the codes is within one BF16 ulp
            assert np.mean(seen["in_scales"][L].cpu().numpy() != ol.scales_to_tiled(scales)) < 0.02
            mid_codes, mid_scales = ol.swiglu_nvfp4_bf16(stand[L]["gate_up"], G_mid)
            assert np.mean(seen["mid_codes"][L].cpu().numpy().reshape(n, FFN // 2) != mid_codes) < 2e-3
            assert np.mean(seen["mid_scales"][L].cpu().numpy() != ol.scales_to_tiled(mid_scales)) < 2e-3
            residual = ol.add_bf16(residual, stand[L]["mlp"])
        scratch = lambda name: lib.axiom_b200_step_provider_scratch(provider, eng.SCRATCH[name])
        got_res = torch.empty((n, HIDDEN), dtype=torch.int16, device="cuda")
        assert cudart.cudaMemcpyAsync(got_res.data_ptr(), scratch("residual"), n * HIDDEN * 2, 3, None) == 0
        sync()
        assert np.array_equal(host(got_res, np.uint16).reshape(n, HIDDEN), residual)       # adds are exact: bit for bit
        _, want_final = ol.add_rmsnorm_bf16(np.zeros_like(residual), residual, final_gamma, 1e-6)
        got_final = u16(seen["final"], n, HIDDEN)
        assert np.all(np.abs(wl.from_bf16_bits(got_final) - wl.from_bf16_bits(want_final)) <= ol.bf16_ulp(wl.from_bf16_bits(want_final)))
        for a in range(n):
            assert np.array_equal(seq_logits[a], logits[a])
        assert lib.axiom_b200_step_provider_scratch(provider, 99) is None

        # ---- paged pools: host-recomputed addresses, everything else still poisoned ----
        raw_k, raw_v = np.empty(pool_bytes, np.uint8), np.empty(pool_bytes, np.uint8)
        kpool.download(raw_k)
        vpool.download(raw_v)
        got_k, got_v = raw_k.view(np.uint16), raw_v.view(np.uint16)
        expect_k = np.full(pool_bytes // 2, 0xFFFF, np.uint16)
        expect_v = expect_k.copy()
        touched = np.zeros(pool_bytes // 2, bool)
        bound_k = np.zeros(pool_bytes // 2, np.float32)
        for L in range(LAYERS):
            for a in range(n):
                pos = int(positions[a])
                pb = int(htbl[a, pos // BT])
                base = ((pb * LAYERS + L) * BT + pos % BT) * kv_dim
                touched[base:base + kv_dim] = True
                expect_v[base:base + kv_dim] = want_v_rows[L][a].reshape(-1)
                expect_k[base:base + kv_dim] = want_k_rows[L][a].reshape(-1)
                bound_k[base:base + kv_dim] = k_bounds[L][a].reshape(-1)
        assert np.array_equal(got_v, expect_v)                                   # V is a copy: bit for bit
        assert np.array_equal(got_k[~touched], expect_k[~touched])              # nothing outside the step's cells
        a_, b_ = wl.from_bf16_bits(got_k[touched]), wl.from_bf16_bits(expect_k[touched])
        assert np.mean(got_k[touched] != expect_k[touched]) < 0.02 and np.all(np.abs(a_ - b_) <= bound_k[touched])

        # ---- a position whose block is outside its table row: that KV write is skipped, the step reports it ----
        hmeta[CAP + 1] = TBL_STRIDE * BT + 3
        d_meta.upload(hmeta)
        kpool.upload(poison)
        assert lib.axiom_b200_step_provider_forward_step(provider, active, n, C.byref(view)) == axk.AXIOM_ERR_RUNTIME
        kpool.download(raw_k)
        again = raw_k.view(np.uint16)
        written_rows = (again.reshape(-1, kv_dim) != 0xFFFF).any(axis=1).sum()
        assert written_rows == LAYERS * (n - 1)
        # argument checks
        inv = axk.AXIOM_ERR_INVALID_ARGUMENT
        assert lib.axiom_b200_step_provider_forward_step(provider, active, CAP + 1, C.byref(view)) == inv
        assert lib.axiom_b200_step_provider_forward_step(provider, active, 0, C.byref(view)) == inv
        assert lib.axiom_b200_step_provider_forward_step(provider, active, n, None) == inv
    finally:
        lib.axiom_b200_step_provider_destroy(provider)
        for b in (kpool, vpool, d_tbl, d_meta):
            b.close()
        rt.close()

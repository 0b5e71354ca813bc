"""The elementwise launches of decoder layers at the reference's M = 8, in the reference's order
(qwen38_model_forward_batch8_internal, src/axiom_qwen38_model.cu:1357-1418, top-1 :509-610): the reference's own
kernels run launch by launch through oracle/_ref on F32 tensors, this library's three calls per layer run from ONE
captured CUDA graph on BF16 tensors, and every stage is compared bit for bit.  The contractions between the stages
(mixer, gate_up, down, LM head) are the reference's library calls and out of scope: seeded BF16-valued tensors stand
in for their outputs, identical on both sides, so the stages are chained through the residual stream only."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol
import ref_lib

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_lib.available(), reason="reference harness library not built")]
wl = importlib.import_module("axiom-kernel_b200.workloads")

HIDDEN, FFN, M, LAYERS, VOCAB = 5120, 17408, 8, 3, 248320


def test_three_layers_and_the_tail_replay_from_one_graph_bit_exact_with_the_reference(axk, cuda_device):
    import torch
    import ref_cases as rc
    from gpu_util import dev, host, sync

    r = ref_lib.lib()
    rng = np.random.default_rng(2024)
    bf = lambda *shape, s=1.0: wl.to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(s))
    hidden0 = bf(M, HIDDEN)
    layers = [dict(mixer=bf(M, HIDDEN), post_gamma=wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(HIDDEN, dtype=np.float32)),
                   gate_up=bf(M, 2 * FFN, s=1.5), mlp=bf(M, HIDDEN, s=0.7),
                   next_gamma=wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(HIDDEN, dtype=np.float32)))
              for _ in range(LAYERS)]
    G_in, G_mid = 85.0, 41.0
    logits = rng.standard_normal((M, VOCAB)).astype(np.float32) * 4
    logits[3, 17] = logits[3, 200001] = 77.0     # a tie: the smaller id wins

    # ---------------- the reference, launch by launch, in its order
    ref = []
    hid = rc.f32_dev(hidden0)
    taps = torch.zeros((5, M, HIDDEN), dtype=torch.float32, device="cuda")
    for li, L in enumerate(layers):
        norm = torch.zeros_like(hid)
        # every device tensor is named: a temporary would be freed, and its block reused, before the launch reads it
        mixer32, post_w32, mlp32 = rc.f32_dev(L["mixer"]), rc.f32_dev(L["post_gamma"]), rc.f32_dev(L["mlp"])
        rc.ok(r.ref_add_bf16_rmsnorm8(hid.data_ptr(), mixer32.data_ptr(), post_w32.data_ptr(), norm.data_ptr(), M), "add_bf16_rmsnorm8")
        after_mixer = rc.bits_of(hid)
        in_codes, in_plane = rc.nvfp4_quantize(rc.bits_of(norm), G_in, "warp")
        mid_codes, mid_plane = rc.swiglu_nvfp4(L["gate_up"], G_mid, "warp")
        rc.ok(r.ref_add_bf16_inplace(hid.data_ptr(), mlp32.data_ptr(), hid.numel()), "add_bf16_inplace")
        rc.ok(r.ref_capture_tap8(hid.data_ptr(), taps.data_ptr(), li), "capture_tap8")
        # the norm that reads the residual next: the attention flavour for layer 0, the model flavour otherwise
        nxt = torch.zeros_like(hid)
        w = rc.f32_dev(L["next_gamma"])
        if li == 0:
            rc.ok(r.ref_attention_rmsnorm8(w.data_ptr(), hid.data_ptr(), nxt.data_ptr()), "attention_rmsnorm8")
        else:
            rc.ok(r.ref_rmsnorm_bf16_8(w.data_ptr(), hid.data_ptr(), nxt.data_ptr(), M), "rmsnorm_bf16_8")
        ref.append(dict(after_mixer=after_mixer, in_codes=in_codes, in_plane=in_plane, mid_codes=mid_codes, mid_plane=mid_plane,
                        after_mlp=rc.bits_of(hid), tap=rc.bits_of(taps[li]), next_norm=rc.bits_of(nxt)))
    x = torch.from_numpy(logits).cuda()
    partials = torch.zeros(M * 256 * 3, dtype=torch.int32, device="cuda")
    ref_top = torch.zeros((M, 3), dtype=torch.int32, device="cuda")
    rc.ok(r.ref_top1_8(x.data_ptr(), partials.data_ptr(), ref_top.data_ptr(), 1), "top1 (hierarchical)")

    # ---------------- this library: three launches per layer + top-1, captured once, replayed
    plane_in = int(axk.lib().axiom_nvfp4_scale_plane_bytes(M, HIDDEN // 16, 1))
    plane_mid = int(axk.lib().axiom_nvfp4_scale_plane_bytes(M, FFN // 16, 1))
    residual = dev(hidden0)
    bufs, glues = [], []
    for L in layers:
        b = dict(mixer=dev(L["mixer"]), post_gamma=dev(L["post_gamma"]), gate_up=dev(L["gate_up"]), mlp=dev(L["mlp"]),
                 next_gamma=dev(L["next_gamma"]),
                 in_codes=torch.zeros((M, HIDDEN // 2), dtype=torch.uint8, device="cuda"),
                 in_plane=torch.zeros(plane_in, dtype=torch.uint8, device="cuda"),
                 mid_codes=torch.zeros((M, FFN // 2), dtype=torch.uint8, device="cuda"),
                 mid_plane=torch.zeros(plane_mid, dtype=torch.uint8, device="cuda"),
                 tap=torch.zeros((M, HIDDEN), dtype=torch.int16, device="cuda"),
                 next_norm=torch.zeros((M, HIDDEN), dtype=torch.int16, device="cuda"))
        bufs.append(b)
        glues.append(axk.make_layer_glue(columns=M, hidden=HIDDEN, ffn=FFN, scale_layout=axk.SCALE_TILED, eps=1e-6,
                                         gate_up_input_scale=G_in, down_input_scale=G_mid, residual=residual,
                                         mixer_out=b["mixer"], post_norm_gamma=b["post_gamma"], mlp_in_codes=b["in_codes"],
                                         mlp_in_scales=b["in_plane"], gate_up=b["gate_up"], mlp_mid_codes=b["mid_codes"],
                                         mlp_mid_scales=b["mid_plane"], mlp_out=b["mlp"], tap_out=b["tap"],
                                         next_norm_gamma=b["next_gamma"], next_norm_out=b["next_norm"]))
    top = torch.zeros((M, 3), dtype=torch.int32, device="cuda")
    assert axk.lib().axiom_b200_prepare(0) == axk.AXIOM_OK

    def enqueue(stream):
        for b, g in zip(bufs, glues):
            assert axk.layer_post_mixer(0, g, stream) == axk.AXIOM_OK
            assert axk.layer_mlp_mid(0, g, stream) == axk.AXIOM_OK
            assert axk.layer_post_mlp(0, g, stream) == axk.AXIOM_OK
        assert axk.top1(0, x, M, VOCAB, top, stream) == axk.AXIOM_OK

    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        enqueue(torch.cuda.current_stream())
    for replay in range(2):                       # the second replay starts from a fresh residual: same bytes again
        residual.copy_(dev(hidden0))
        sync()
        graph.replay()
        sync()
        for b, want in zip(bufs, ref):
            assert np.array_equal(host(b["in_codes"], np.uint8).reshape(M, -1), want["in_codes"])
            assert np.array_equal(host(b["in_plane"], np.uint8), want["in_plane"])
            assert np.array_equal(host(b["mid_codes"], np.uint8).reshape(M, -1), want["mid_codes"])
            assert np.array_equal(host(b["mid_plane"], np.uint8), want["mid_plane"])
            assert np.array_equal(host(b["tap"], np.uint16).reshape(M, HIDDEN), want["tap"])
            assert np.array_equal(want["tap"], want["after_mlp"])
            assert np.array_equal(host(b["next_norm"], np.uint16).reshape(M, HIDDEN), want["next_norm"])
        assert np.array_equal(host(residual, np.uint16).reshape(M, HIDDEN), ref[-1]["after_mlp"])
        assert np.array_equal(top.cpu().numpy().view(np.uint32), ref_top.cpu().numpy().view(np.uint32))
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0
    # the residual right after the mixer add is an intermediate of the fused call: checked through an eager run
    residual.copy_(dev(hidden0))
    assert axk.layer_post_mixer(0, glues[0]) == axk.AXIOM_OK
    sync()
    assert np.array_equal(host(residual, np.uint16).reshape(M, HIDDEN), ref[0]["after_mixer"])


def test_layer_glue_argument_checks(axk, cuda_device):
    import torch

    t = torch.zeros((8, 5120), dtype=torch.int16, device="cuda")
    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    g = axk.make_layer_glue(columns=8, hidden=5120, ffn=17408, residual=t)
    assert axk.layer_post_mixer(0, g) == inv and axk.layer_mlp_mid(0, g) == inv and axk.layer_post_mlp(0, g) == inv
    g2 = axk.make_layer_glue(columns=8, hidden=5120, ffn=17408, residual=t, mlp_out=t, next_norm_gamma=t, next_norm_out=t, tap_out=t)
    assert axk.layer_post_mlp(0, g2) == inv            # the tap may not alias the residual
    g3 = axk.make_layer_glue(columns=8, hidden=5100, ffn=17408, residual=t, mlp_out=t, next_norm_gamma=t, next_norm_out=t)
    assert axk.layer_post_mlp(0, g3) == inv            # hidden % 16
    assert not t.any().item()

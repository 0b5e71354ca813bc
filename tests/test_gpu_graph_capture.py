"""Stream-explicit entries inside a CUDA graph: no allocation, no synchronisation and no device-to-host read may
happen in a call that is being captured (the reference's contract for graph-replayed stages,
include/axiom/qwen38_mtp_device_control.h:4-10).  The stages of one layer are captured once and replayed on new
input contents; every output must equal the eager calls' output bit for bit."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


@pytest.mark.parametrize("m", [8, 600])
def test_layer_stages_replay_from_a_graph(axk, cuda_device, m):
    """m = 8 takes the latency-shaped kernels, m = 600 the persistent streaming ones (the q/k stage with its
    tensor-map flavour: the map is encoded on the host at capture time and replayed as a kernel parameter)."""
    import torch
    from gpu_util import dev

    heads, kv_heads, D = 16, 4, 128
    width, ffn = heads * D, 4096
    inv_freq = dev(ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, D))
    mscale = axk.yarn_mscale(4.0)
    n_blocks = 64
    plane = lambda cols: int(axk.lib().axiom_nvfp4_scale_plane_bytes(m, cols // 16, 1))  # tiled scale plane, bytes

    def inputs(seed):
        rng = np.random.default_rng(seed)
        bf = lambda *shape, s=1.0: wl.to_bf16_bits((rng.standard_normal(shape, dtype=np.float32) * np.float32(s)))
        return dict(hidden=bf(m, width), residual=bf(m, width), gamma=bf(width, s=0.02) , q_gate=bf(m, heads, 2 * D),
                    k=bf(m, kv_heads, D), v=bf(m, kv_heads, D), attn=bf(m, width), gu=bf(m, 2 * ffn, s=1.5),
                    logits=rng.standard_normal((8, 5000), dtype=np.float32),
                    positions=rng.permutation(n_blocks * 16)[:m].astype(np.uint32) if m <= n_blocks * 16 else None)

    first, second = inputs(1), inputs(2)
    d = {k: dev(v) for k, v in first.items()}
    qg, kg = dev(wl.to_bf16_bits(np.ones(D, np.float32))), dev(wl.to_bf16_bits(np.ones(D, np.float32)))
    table = dev(np.random.default_rng(5).permutation(n_blocks).astype(np.int32)[None, :])
    out = dict(
        norm=torch.zeros((m, width), dtype=torch.int16, device="cuda"),
        codes=torch.zeros((m, width // 2), dtype=torch.uint8, device="cuda"),
        scales=torch.zeros((plane(width),), dtype=torch.uint8, device="cuda"),
        q=torch.zeros((m, heads, D), dtype=torch.int16, device="cuda"),
        k_pool=torch.zeros((n_blocks * 16 * kv_heads * D,), dtype=torch.int16, device="cuda"),
        v_pool=torch.zeros((n_blocks * 16 * kv_heads * D,), dtype=torch.int16, device="cuda"),
        gate_codes=torch.zeros((m, width // 2), dtype=torch.uint8, device="cuda"),
        gate_scales=torch.zeros((plane(width),), dtype=torch.uint8, device="cuda"),
        mlp_codes=torch.zeros((m, ffn // 2), dtype=torch.uint8, device="cuda"),
        mlp_scales=torch.zeros((plane(ffn),), dtype=torch.uint8, device="cuda"),
        fp8=torch.zeros((m, ffn), dtype=torch.uint8, device="cuda"),
        fp8_scales=torch.zeros((m,), dtype=torch.float32, device="cuda"),
        top=torch.zeros((8, 3), dtype=torch.int32, device="cuda"),
        status=torch.zeros(1, dtype=torch.int32, device="cuda"),
    )
    args = axk.make_qk_args(tokens=m, q_heads=heads, k_heads=kv_heads, head_dim=D, rope_dim=D,
                            flags=axk.QK_FLAG_RING | axk.QK_FLAG_Q_GATE_INTERLEAVED, eps=1e-6, mscale=mscale,
                            block_tokens=16, n_layers=1, layer=0, pool_stride=kv_heads * D, tbl_stride=n_blocks,
                            n_blocks=n_blocks, q=d["q_gate"], k=d["k"], v=d["v"], q_gamma=qg, k_gamma=kg,
                            inv_freq=inv_freq, positions=d["positions"], block_tables=table, k_pool=out["k_pool"],
                            v_pool=out["v_pool"], status_word=out["status"], q_out=out["q"])

    def stages(stream):
        ok = axk.AXIOM_OK
        assert axk.add_rmsnorm_nvfp4(0, d["hidden"], d["residual"], d["gamma"], 1e-6, m, width, 80.0, out["norm"],
                                     out["codes"], out["scales"], 1, stream) == ok
        assert axk.qk_norm_rope_paged(0, args, stream) == ok
        assert axk.sigmoid_gate_heads_nvfp4(0, d["attn"], d["q_gate"], m, heads, D, 60.0, None, out["gate_codes"],
                                            out["gate_scales"], 1, stream) == ok
        assert axk.swiglu_nvfp4(0, d["gu"], m, ffn, 40.0, out["mlp_codes"], out["mlp_scales"], 1, stream) == ok
        assert axk.swiglu_fp8(0, d["gu"], m, ffn, out["fp8"], out["fp8_scales"], stream) == ok
        assert axk.top1(0, d["logits"], 8, 5000, out["top"], stream) == ok

    def load(values):
        for name, value in values.items():
            if value is not None:
                d[name].copy_(dev(value))
        for t in out.values():
            t.zero_()
        torch.cuda.synchronize()  # the copies above ran on the default stream, the stages use their own

    def snapshot():
        torch.cuda.synchronize()
        return {name: t.cpu().numpy().copy() for name, t in list(out.items()) + [("residual", d["residual"])]}

    stream = torch.cuda.Stream()
    # eager results for both input sets (the tables of the gated kernels are made ready by these calls)
    eager = []
    for values in (first, second):
        load(values)
        with torch.cuda.stream(stream):
            stages(stream)
        eager.append(snapshot())

    load(first)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        stages(stream)
    for values, want in ((first, eager[0]), (second, eager[1]), (first, eager[0])):
        load(values)
        graph.replay()
        got = snapshot()
        for name in want:
            assert np.array_equal(got[name], want[name]), name
    assert int(out["status"].item()) == 0
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0


PREPARE_PROBE = r"""
import importlib, sys, torch
sys.path.insert(0, {root!r})
axk = importlib.import_module("axiom-kernel_b200")
lib = axk.lib()
torch.cuda.set_device(0)
rows, width = 320, 1024
a = torch.randn((rows, width), device="cuda").to(torch.bfloat16)
g = torch.randn((rows, width), device="cuda").to(torch.bfloat16)
gu = torch.randn((rows, 2 * width), device="cuda").to(torch.bfloat16)
codes = torch.empty((rows, width // 2), dtype=torch.uint8, device="cuda")
scales = torch.empty((rows, width // 16), dtype=torch.uint8, device="cuda")
c8 = torch.empty((rows, width), dtype=torch.uint8, device="cuda")
s8 = torch.empty(rows, dtype=torch.float32, device="cuda")
torch.cuda.synchronize()
if {prepare}:
    assert lib.axiom_b200_prepare(0) == 0
before = int(lib.axiom_b200_kernel_launch_count())
assert axk.sigmoid_gate_nvfp4(0, a, g, rows, width, 50.0, None, codes, scales, 0) == 0
assert axk.swiglu_fp8(0, gu, rows, width, c8, s8) == 0
torch.cuda.synchronize()
print(int(lib.axiom_b200_kernel_launch_count()) - before)
"""


def test_prepare_takes_the_lazy_set_up_out_of_the_first_calls(axk, cuda_device):
    """In a fresh process the first sigmoid-gate and SwiGLU calls that use the gate tables each launch a fill kernel
    (and synchronise their stream) before their own kernel; after axiom_b200_prepare they launch their own kernel only."""
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parent.parent)
    counts = {}
    for prepare in (False, True):
        res = subprocess.run([sys.executable, "-c", PREPARE_PROBE.format(root=root, prepare=prepare)], capture_output=True,
                             text=True, timeout=300)
        assert res.returncode == 0, res.stderr[-2000:]
        counts[prepare] = int(res.stdout.strip().splitlines()[-1])
    assert counts[True] == 2       # the two kernels themselves
    assert counts[False] == 4      # plus one table fill each

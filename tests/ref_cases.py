"""Runs the reference's own kernels (oracle/_ref) on seeded inputs.  Used twice: live by the
-m gpu parity tests, and by tests/golden/make_golden.py to write the committed fixtures."""
from __future__ import annotations

import importlib

import numpy as np
import torch

import ref_lib

wl = importlib.import_module("axiom-kernel_b200.workloads")

REF_Q_HEADS, REF_K_HEADS, REF_HEAD_DIM, REF_ROPE_DIM = 24, 4, 256, 64
REF_THETA, REF_YARN_FACTOR, REF_YARN_CTX = 1.0e7, 4.0, 262144.0
REF_MSCALE = float(np.float32(1.138629436111989))


def f32_dev(bits: np.ndarray) -> torch.Tensor:
    """BF16 bit patterns -> F32 device tensor holding the same values (the reference's storage)."""
    return torch.from_numpy(wl.from_bf16_bits(bits)).cuda()


def bits_of(t: torch.Tensor) -> np.ndarray:
    """F32 device tensor of BF16-valued numbers -> BF16 bit patterns (asserts nothing is lost)."""
    a = t.detach().cpu().numpy().view(np.uint32)
    assert not (a & 0xFFFF).any(), "reference output is not BF16-valued"
    return (a >> 16).astype(np.uint16)


def ok(rc, what):
    assert rc == 0, f"reference launcher {what} failed with {rc}"


def special_rows(cols: int) -> np.ndarray:
    x = np.zeros((12, cols), np.float32)
    x[1, :16] = -0.0
    x[2, 5] = 1.0
    x[4, 2] = 2.0
    x[5, :] = 3.3895314e38
    x[6, :8] = 1e-40
    x[7, :16] = [6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25, -6, -5, -3.5, -2.5, -1.75, -1.25, -0.75, -0.25]
    x[8, :16] = np.array([6, 5, 3.5, 2.5, 1.75, 1.25, 0.75, 0.25] * 2, np.float32) * 0.5
    x[9, :] = 9.1835e-41
    x[10, ::2] = 1e30
    x[10, 1::2] = -1e-30
    x[11] = np.random.default_rng(5).standard_normal(cols).astype(np.float32) * np.float32(1e-3)
    bits = wl.to_bf16_bits(x)
    bits[2, 3] = 0x7FC0          # NaN
    bits[3, :16] = 0xFFC0        # all-NaN block
    bits[4, 0] = 0x7F80          # +inf
    bits[4, 1] = 0xFF80          # -inf
    return bits


def nvfp4_quantize(x_bits: np.ndarray, G: float, variant: str):
    """variant: 'row' (exported oracle entry, canonical scales), 'thread' or 'warp' (tiled scales)."""
    r = ref_lib.lib()
    rows, cols = x_bits.shape
    x = f32_dev(x_bits)
    codes = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
    if variant == "row":
        scales = torch.zeros((rows, cols // 16), dtype=torch.uint8, device="cuda")
        for i in range(rows):
            ok(r.axiom_qwen38_nvfp4_quantize_reference_f32(0, x[i].data_ptr(), G, codes[i].data_ptr(), scales[i].data_ptr(), cols, None), "row entry")
    else:
        plane = ((rows + 127) // 128) * ((cols // 16 + 3) // 4) * 512
        scales = torch.zeros(plane, dtype=torch.uint8, device="cuda")
        ok(r.ref_quantize_batch_to_tc(x.data_ptr(), G, codes.data_ptr(), scales.data_ptr(), cols, rows, int(variant == "warp")), variant)
    return codes.cpu().numpy(), scales.cpu().numpy()


def add_rmsnorm(hidden_bits, residual_bits, gamma_bits):
    """hidden may be None.  Returns (residual', norm) as BF16 bits.  rows % 8 == 0, cols == 5120."""
    r = ref_lib.lib()
    rows = residual_bits.shape[0]
    res = f32_dev(residual_bits)
    w = f32_dev(gamma_bits)
    norm = torch.zeros_like(res)
    if hidden_bits is None:
        ok(r.ref_rmsnorm_bf16_8(w.data_ptr(), res.data_ptr(), norm.data_ptr(), rows), "rmsnorm8")
    else:
        hidden = f32_dev(hidden_bits)
        ok(r.ref_add_bf16_rmsnorm8(res.data_ptr(), hidden.data_ptr(), w.data_ptr(), norm.data_ptr(), rows), "add_rmsnorm8")
    return bits_of(res), bits_of(norm)


def add_bf16(a_bits, b_bits):
    a, b = f32_dev(a_bits), f32_dev(b_bits)
    ok(ref_lib.lib().ref_add_bf16_inplace(a.data_ptr(), b.data_ptr(), a.numel()), "add_bf16_inplace")
    return bits_of(a)


def fp8_quantize_f32(x: torch.Tensor):
    rows, cols = x.shape
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, dtype=torch.float32, device="cuda")
    ok(ref_lib.lib().ref_quantize_columns_e4m3(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), cols, rows), "quantize_columns_e4m3")
    return codes.cpu().numpy(), scales.cpu().numpy()


def fp8_quantize_bf16(x_bits: np.ndarray):
    rows, cols = x_bits.shape
    x = torch.from_numpy(x_bits.view(np.int16)).cuda()
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ok(ref_lib.lib().ref_quantize_bf16_rows_e4m3(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols, status.data_ptr()), "quantize_bf16_rows")
    return codes.cpu().numpy(), scales.cpu().numpy(), int(status.item())


def swiglu_f32(gu_bits: np.ndarray) -> torch.Tensor:
    rows, two_w = gu_bits.shape
    w = two_w // 2
    gate = f32_dev(np.ascontiguousarray(gu_bits[:, :w]))
    up = f32_dev(np.ascontiguousarray(gu_bits[:, w:]))
    out = torch.zeros_like(gate)
    ok(ref_lib.lib().ref_silu_mul_batch(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel()), "silu_mul_batch")
    return out


def swiglu_fp8(gu_bits: np.ndarray):
    return fp8_quantize_f32(swiglu_f32(gu_bits))


def swiglu_nvfp4(gu_bits: np.ndarray, G: float, variant: str):
    rows, two_w = gu_bits.shape
    w = two_w // 2
    x = f32_dev(gu_bits)
    codes = torch.zeros((rows, w // 2), dtype=torch.uint8, device="cuda")
    plane = ((rows + 127) // 128) * ((w // 16 + 3) // 4) * 512
    scales = torch.zeros(plane, dtype=torch.uint8, device="cuda")
    ok(ref_lib.lib().ref_silu_mul_quantize_batch_to_tc(x.data_ptr(), G, codes.data_ptr(), scales.data_ptr(), w, rows, int(variant == "warp")), "silu_mul_quantize")
    return codes.cpu().numpy(), scales.cpu().numpy()


def yarn_inv_freq() -> np.ndarray:
    out = torch.zeros(32, dtype=torch.float32, device="cuda")
    ok(ref_lib.lib().ref_yarn_inv_frequency(out.data_ptr()), "yarn_inv_frequency")
    return out.cpu().numpy()


def qk_inputs(seed: int):
    rng = np.random.default_rng(seed)
    q = wl.to_bf16_bits(rng.standard_normal((8, REF_Q_HEADS, REF_HEAD_DIM), dtype=np.float32))
    k = wl.to_bf16_bits(rng.standard_normal((8, REF_K_HEADS, REF_HEAD_DIM), dtype=np.float32))
    v = wl.to_bf16_bits(rng.standard_normal((8, REF_K_HEADS, REF_HEAD_DIM), dtype=np.float32))
    qg = wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(REF_HEAD_DIM, dtype=np.float32))
    kg = wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(REF_HEAD_DIM, dtype=np.float32))
    return q, k, v, qg, kg


def qk_temporal8(q_bits, k_bits, v_bits, qg_bits, kg_bits, base_position: int, yarn: bool = True):
    """8 tokens at positions base..base+7.  Returns rotated Q bits, rotated K bits [8,4,256], V bits as cached."""
    r = ref_lib.lib()
    q, k, v = f32_dev(q_bits), f32_dev(k_bits), f32_dev(v_bits)
    qw, kw = f32_dev(qg_bits), f32_dev(kg_bits)  # named: a temporary would be freed (and its block reused) before the launch
    max_context = base_position + 8
    kc = torch.zeros((max_context, 1024), dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    kref = torch.zeros((max_context, 1024), dtype=torch.float32, device="cuda")
    vref = torch.zeros_like(kref)
    ok(r.ref_qk_norm_partial_rope_cache_temporal8(q.data_ptr(), k.data_ptr(), qw.data_ptr(), kw.data_ptr(),
                                                  v.data_ptr(), kc.data_ptr(), vc.data_ptr(), kref.data_ptr(), vref.data_ptr(),
                                                  base_position, max_context, int(yarn)), "qk temporal8")
    k_rows = bits_of(kref[base_position:base_position + 8]).reshape(8, REF_K_HEADS, REF_HEAD_DIM)
    v_rows = bits_of(vref[base_position:base_position + 8]).reshape(8, REF_K_HEADS, REF_HEAD_DIM)
    return bits_of(q), k_rows, v_rows, kc[base_position:base_position + 8].cpu().numpy()


def draft_qk_norm_rope(x_bits: np.ndarray, gamma_bits: np.ndarray, rope_table: np.ndarray, first_position: int):
    """The reference's BF16-convention q/k kernel followed by its BF16 rounding pass; x_bits [T, H, 128], token t at
    position first_position + t.  Returns the BF16 bits of the result."""
    tokens, heads, _ = x_bits.shape
    x = f32_dev(x_bits)
    w = torch.from_numpy(gamma_bits.view(np.int16)).cuda()
    table = torch.from_numpy(np.ascontiguousarray(rope_table, np.float32)).cuda()
    ok(ref_lib.lib().ref_dspark_qk_norm_rope_round(w.data_ptr(), x.data_ptr(), table.data_ptr(), table.shape[0], heads, tokens,
                                                   first_position), "dspark qk_norm_rope + round")
    return bits_of(x)


def fp8_quantize_static_f32(x: torch.Tensor, scale: float):
    rows, cols = x.shape
    codes = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
    ok(ref_lib.lib().ref_quantize_columns_static_e4m3(x.data_ptr(), codes.data_ptr(), scale, cols, rows), "quantize_columns_static_e4m3")
    return codes.cpu().numpy()

"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (stand-ins for real activations; no dataset is used).

numpy flavours (`*_np`) serve the parity tests at small sizes; torch flavours
build the full-size tensors directly on the device for the benchmark.
All BF16 data is carried as uint16 bit patterns on the numpy side.
"""
from __future__ import annotations

import numpy as np

HIDDEN = 5120
FFN = 17408
Q_HEADS = 64
K_HEADS = 8
HEAD_DIM = 128
VOCAB = 151936
ROPE_THETA = 1.0e6
YARN_FACTOR = 4.0
YARN_ORIGINAL_CONTEXT = 32768.0
YARN_BETA_FAST = 32.0
YARN_BETA_SLOW = 1.0
KV_BLOCK_TOKENS = 16
KV_BLOCKS = 4096
EPS = 1.0e-6


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def nvfp4_global_scale(amax: float) -> float:
    """G = 1/s with s = amax/(6*448), both in FP32 (the multiplier convention of the quantizer)."""
    s = np.float32(amax) / np.float32(6.0 * 448.0)
    return float(np.float32(1.0) / s)


# ---------------------------------------------------------------------------
# numpy (tests)
# ---------------------------------------------------------------------------

def quantize_input_np(rows: int, cols: int = HIDDEN, seed: int = 0) -> np.ndarray:
    """N(0,1) with 0.1 % of the elements scaled by 20 (config 1)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    mask = rng.random((rows, cols)) < 0.001
    x[mask] *= np.float32(20.0)
    return to_bf16_bits(x)


def add_rmsnorm_inputs_np(rows: int, cols: int = HIDDEN):
    """hidden (seed 0), residual (seed 1) ~N(0,1); gamma (seed 2) = 1 + N(0,0.02) (config 2)."""
    hidden = to_bf16_bits(np.random.default_rng(0).standard_normal((rows, cols), dtype=np.float32))
    residual = to_bf16_bits(np.random.default_rng(1).standard_normal((rows, cols), dtype=np.float32))
    gamma = to_bf16_bits(1.0 + 0.02 * np.random.default_rng(2).standard_normal(cols, dtype=np.float32))
    return hidden, residual, gamma


def qk_inputs_np(tokens: int, q_heads: int = Q_HEADS, k_heads: int = K_HEADS, head_dim: int = HEAD_DIM,
                 n_blocks: int = KV_BLOCKS, seed: int = 3, max_base: int = 100000):
    """Q, K, V ~N(0,1); gammas 1+N(0,0.02); positions base+t; block table = permutation (config 3)."""
    rng = np.random.default_rng(seed)
    q = to_bf16_bits(rng.standard_normal((tokens, q_heads, head_dim), dtype=np.float32))
    k = to_bf16_bits(rng.standard_normal((tokens, k_heads, head_dim), dtype=np.float32))
    v = to_bf16_bits(rng.standard_normal((tokens, k_heads, head_dim), dtype=np.float32))
    q_gamma = to_bf16_bits(1.0 + 0.02 * rng.standard_normal(head_dim, dtype=np.float32))
    k_gamma = to_bf16_bits(1.0 + 0.02 * rng.standard_normal(head_dim, dtype=np.float32))
    base = int(rng.integers(0, max_base))
    positions = (base + np.arange(tokens)).astype(np.uint32)
    table = rng.permutation(n_blocks).astype(np.int32).reshape(1, n_blocks)
    return q, k, v, q_gamma, k_gamma, positions, table


def swiglu_input_np(rows: int, width: int = FFN, seed: int = 4) -> np.ndarray:
    """[gate ~N(0,1.5) | up ~N(0,1)] (config 4)."""
    rng = np.random.default_rng(seed)
    gate = rng.standard_normal((rows, width), dtype=np.float32) * np.float32(1.5)
    up = rng.standard_normal((rows, width), dtype=np.float32)
    return to_bf16_bits(np.concatenate([gate, up], axis=1))


def embedding_inputs_np(tokens: int, vocab: int = VOCAB, hidden: int = HIDDEN, seed: int = 5):
    rng = np.random.default_rng(seed)
    table = to_bf16_bits(rng.standard_normal((vocab, hidden), dtype=np.float32) * np.float32(0.02))
    ids = rng.integers(0, vocab, tokens).astype(np.uint32)
    return table, ids


# ---------------------------------------------------------------------------
# torch (benchmark): tensors created on `device`
# ---------------------------------------------------------------------------

def _gen(torch, device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def quantize_input_torch(torch, device, rows: int, cols: int = HIDDEN, seed: int = 0):
    g = _gen(torch, device, seed)
    x = torch.randn((rows, cols), generator=g, device=device, dtype=torch.float32)
    mask = torch.rand((rows, cols), generator=g, device=device) < 0.001
    x = torch.where(mask, x * 20.0, x)
    return x.to(torch.bfloat16)


def add_rmsnorm_inputs_torch(torch, device, rows: int, cols: int = HIDDEN):
    hidden = torch.randn((rows, cols), generator=_gen(torch, device, 0), device=device).to(torch.bfloat16)
    residual = torch.randn((rows, cols), generator=_gen(torch, device, 1), device=device).to(torch.bfloat16)
    gamma = (1.0 + 0.02 * torch.randn((cols,), generator=_gen(torch, device, 2), device=device)).to(torch.bfloat16)
    return hidden, residual, gamma


def qk_inputs_torch(torch, device, tokens: int, q_heads: int = Q_HEADS, k_heads: int = K_HEADS,
                    head_dim: int = HEAD_DIM, n_blocks: int = KV_BLOCKS, seed: int = 3):
    g = _gen(torch, device, seed)
    q = torch.randn((tokens, q_heads, head_dim), generator=g, device=device).to(torch.bfloat16)
    k = torch.randn((tokens, k_heads, head_dim), generator=g, device=device).to(torch.bfloat16)
    v = torch.randn((tokens, k_heads, head_dim), generator=g, device=device).to(torch.bfloat16)
    q_gamma = (1.0 + 0.02 * torch.randn((head_dim,), generator=g, device=device)).to(torch.bfloat16)
    k_gamma = (1.0 + 0.02 * torch.randn((head_dim,), generator=g, device=device)).to(torch.bfloat16)
    base = int(torch.randint(0, 100000, (1,), generator=g, device=device).item())
    positions = (base + torch.arange(tokens, device=device)).to(torch.int32)
    table = torch.randperm(n_blocks, generator=g, device=device).to(torch.int32).reshape(1, n_blocks)
    return q, k, v, q_gamma, k_gamma, positions, table


def swiglu_input_torch(torch, device, rows: int, width: int = FFN, seed: int = 4):
    g = _gen(torch, device, seed)
    out = torch.empty((rows, 2 * width), device=device, dtype=torch.bfloat16)
    step = 2048
    for r0 in range(0, rows, step):  # bounded FP32 temporaries
        n = min(step, rows - r0)
        out[r0:r0 + n, :width] = (torch.randn((n, width), generator=g, device=device) * 1.5).to(torch.bfloat16)
        out[r0:r0 + n, width:] = torch.randn((n, width), generator=g, device=device).to(torch.bfloat16)
    return out


def embedding_inputs_torch(torch, device, tokens: int, vocab: int = VOCAB, hidden: int = HIDDEN, seed: int = 5):
    g = _gen(torch, device, seed)
    table = torch.empty((vocab, hidden), device=device, dtype=torch.bfloat16)
    step = 16384
    for r0 in range(0, vocab, step):
        n = min(step, vocab - r0)
        table[r0:r0 + n] = (torch.randn((n, hidden), generator=g, device=device) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (tokens,), generator=g, device=device).to(torch.int32)
    return table, ids

"""Token-row sharding across the GPUs of one box.

Every op of the fused path is independent per token row (RMSNorm, q/k norm and
the FP8 scale reduce within a row, NVFP4 blocks within 16 elements, gather and
the KV write are per token), so N GPUs split the rows and never exchange data.
The only collectives are in the harness: a max over ranks of the step time and
a gather of per-row digests for verification.  The NVFP4 global scale is a
calibrated input (reference src/axiom_qwen38_nvfp4_mlp.cu:1059-1081), the same
number on every rank.

Nothing here touches the GPU; the callers hand in a `torch.distributed` module
whose process group is already initialised (nccl on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import zlib

import numpy as np


def row_range(total_rows: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """Contiguous rows [lo, hi) of `rank`.  Boundaries fall on multiples of `align` (a KV page is
    16 tokens: no page is shared between two GPUs), the tail goes to the last rank that has rows,
    and the ranges of all ranks tile [0, total_rows) exactly; a rank may get an empty range."""
    if world <= 0 or not 0 <= rank < world or total_rows < 0 or align <= 0:
        raise ValueError("row_range: bad arguments")
    units = (total_rows + align - 1) // align          # whole pages, the last one possibly short
    base, extra = divmod(units, world)
    lo_u = rank * base + min(rank, extra)
    hi_u = lo_u + base + (1 if rank < extra else 0)
    return min(lo_u * align, total_rows), min(hi_u * align, total_rows)


def row_digests(*arrays: np.ndarray) -> np.ndarray:
    """One CRC32 per row over the bytes of that row in every array (arrays share their first axis)."""
    rows = arrays[0].shape[0]
    out = np.zeros(rows, dtype=np.uint32)
    views = [np.ascontiguousarray(a).reshape(rows, -1).view(np.uint8) for a in arrays]
    for r in range(rows):
        crc = 0
        for v in views:
            crc = zlib.crc32(v[r].tobytes(), crc)
        out[r] = crc
    return out


def max_over_ranks(dist, value: float, device=None) -> float:
    """Max of a per-rank scalar (the step time: a multi-GPU number is the slowest rank's)."""
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_row_digests(dist, local: np.ndarray, total_rows: int, align: int = 16, device=None):
    """All ranks contribute the digests of their row range; every rank gets the digest vector of
    all `total_rows` rows (ranges are ragged, so the exchange is padded to the widest range)."""
    import torch

    world, rank = dist.get_world_size(), dist.get_rank()
    ranges = [row_range(total_rows, world, r, align) for r in range(world)]
    lo, hi = ranges[rank]
    if local.shape != (hi - lo,):
        raise ValueError(f"rank {rank}: expected {hi - lo} digests, got {local.shape}")
    widest = max(h - l for l, h in ranges)
    send = torch.zeros(max(widest, 1), dtype=torch.int64, device=device)
    send[: hi - lo] = torch.from_numpy(local.astype(np.int64)).to(send.device)
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send)
    out = np.zeros(total_rows, dtype=np.uint32)
    for (l, h), t in zip(ranges, recv):
        out[l:h] = t[: h - l].cpu().numpy().astype(np.uint32)
    return out


def sharded_digests(dist, total_rows: int, compute, align: int = 16, device=None):
    """Runs `compute(lo, hi)` (-> tuple of arrays whose first axis is hi - lo) on this rank's rows
    and returns the digest vector of the whole job, identical on every rank."""
    lo, hi = row_range(total_rows, dist.get_world_size(), dist.get_rank(), align)
    if hi > lo:
        local = row_digests(*compute(lo, hi))
    else:
        local = np.zeros(0, dtype=np.uint32)
    return gather_row_digests(dist, local, total_rows, align, device)

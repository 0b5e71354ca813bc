"""Helpers shared by the -m gpu tests: device tensors from numpy bit patterns,
poisoned outputs with guard bands, and the BF16 tolerance used for float results."""
from __future__ import annotations

import numpy as np
import torch

GUARD = 256  # bytes of 0xFF on both sides of every output


def dev(array: np.ndarray) -> torch.Tensor:
    """Copy a numpy array to cuda:0 keeping its bytes (uint16/uint32 go through same-width ints)."""
    a = np.ascontiguousarray(array)
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32}.get(a.dtype)
    if view is not None:
        a = a.view(view)
    return torch.from_numpy(a).cuda()


def host(t: torch.Tensor, dtype) -> np.ndarray:
    return t.detach().cpu().numpy().view(dtype)


class Guarded:
    """A byte buffer on the device filled with 0xFF, with guard bands around the payload."""

    def __init__(self, nbytes: int, align: int = 256):
        self.nbytes = nbytes
        self.pad = (GUARD + align - 1) // align * align
        self.raw = torch.full((self.pad + nbytes + GUARD,), 0xFF, dtype=torch.uint8, device="cuda")

    @property
    def ptr(self) -> int:
        return self.raw.data_ptr() + self.pad

    def payload(self, dtype=np.uint8) -> np.ndarray:
        return self.raw[self.pad:self.pad + self.nbytes].cpu().numpy().view(dtype)

    def guards_intact(self) -> bool:
        r = self.raw.cpu().numpy()
        return bool((r[:self.pad] == 0xFF).all() and (r[self.pad + self.nbytes:] == 0xFF).all())

    def untouched(self) -> bool:
        return bool((self.raw.cpu().numpy() == 0xFF).all())


def sync():
    torch.cuda.synchronize()

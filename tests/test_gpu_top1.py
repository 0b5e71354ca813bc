"""Greedy selection (largest finite logit, smallest id among equals, invalid flag) through the C ABI against the
oracle, and against both of the reference's top-1 paths on its fixed [8 x 248320] shape."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol
import ref_lib

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


def run(axk, logits):
    import torch
    from gpu_util import sync

    rows, vocab = logits.shape
    x = torch.from_numpy(np.ascontiguousarray(logits)).cuda()
    out = torch.full((rows, 3), 0x55555555, dtype=torch.int32, device="cuda")
    assert axk.top1(0, x, rows, vocab, out) == axk.AXIOM_OK
    sync()
    return out.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("rows,vocab", [(1, 248320), (8, 151936), (3, 7), (5, 4099), (64, 32000), (2, 33),
                                         (127, 4100), (128, 4100), (130, 7), (200, 151936), (300, 4099)])
def test_top1_matches_oracle(axk, cuda_device, rows, vocab):
    rng = np.random.default_rng(rows * 131 + vocab)
    logits = rng.standard_normal((rows, vocab)).astype(np.float32) * 3
    # ties at the maximum (the smaller id wins), a winner in the last element, non-finite entries
    logits[0, vocab // 2] = logits[0].max() + 1
    logits[0, vocab // 3] = logits[0, vocab // 2]
    if rows > 1:
        logits[1, vocab - 1] = 50.0
        logits[1, 0] = np.inf
    if rows > 2:
        logits[2, :] = np.nan
    if rows > 3:
        logits[3, vocab // 5] = -np.inf
    assert np.array_equal(run(axk, logits), ol.top1_f32(logits))


def test_top1_unaligned_rows_take_the_scalar_path(axk, cuda_device):
    import torch
    from gpu_util import sync

    rng = np.random.default_rng(4)
    backing = rng.standard_normal(4 * 1000 + 1).astype(np.float32)
    x = torch.from_numpy(backing).cuda()
    out = torch.zeros((4, 3), dtype=torch.int32, device="cuda")
    assert axk.top1(0, x[1:], 4, 1000, out) == axk.AXIOM_OK   # base 4-byte aligned only
    sync()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ol.top1_f32(backing[1:].reshape(4, 1000)))
    # the same with enough rows for one CTA per row
    backing = rng.standard_normal(150 * 1000 + 1).astype(np.float32)
    x = torch.from_numpy(backing).cuda()
    out = torch.zeros((150, 3), dtype=torch.int32, device="cuda")
    assert axk.top1(0, x[1:], 150, 1000, out) == axk.AXIOM_OK
    sync()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ol.top1_f32(backing[1:].reshape(150, 1000)))


@pytest.mark.skipif(not ref_lib.available(), reason="reference harness library not built")
def test_top1_matches_both_reference_paths(axk, cuda_device):
    import torch

    r = ref_lib.lib()
    rng = np.random.default_rng(9)
    logits = rng.standard_normal((8, 248320)).astype(np.float32) * 4
    logits[2, 1000] = logits[2, 200000] = 99.0
    logits[5, 77] = np.nan
    x = torch.from_numpy(logits).cuda()
    partials = torch.zeros(8 * 256 * 3, dtype=torch.int32, device="cuda")
    want = ol.top1_f32(logits)
    for hierarchical in (0, 1):
        res = torch.zeros((8, 3), dtype=torch.int32, device="cuda")
        assert r.ref_top1_8(x.data_ptr(), partials.data_ptr(), res.data_ptr(), hierarchical) == 0
        assert np.array_equal(res.cpu().numpy().view(np.uint32), want)
    assert np.array_equal(run(axk, logits), want)

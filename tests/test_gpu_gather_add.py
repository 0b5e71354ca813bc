"""Embedding gather and BF16 residual add: bit-exact against the CPU oracle."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


@pytest.mark.parametrize("tokens", [1, 8, 64, 256, 1000])
def test_gather_matches_oracle(axk, cuda_device, tokens):
    import torch
    from gpu_util import Guarded, dev, sync

    table, ids = wl.embedding_inputs_np(tokens, vocab=3000, hidden=5120)
    out = Guarded(tokens * 5120 * 2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = axk.embedding_gather(0, dev(table), 3000, 5120, dev(ids), tokens, out.ptr, status)
    sync()
    assert rc == axk.AXIOM_OK and out.guards_intact() and int(status.item()) == 0
    assert np.array_equal(out.payload(np.uint16).reshape(tokens, 5120), ol.embedding_gather_bf16(table, ids))


def test_gather_invalid_id_gives_zero_row_and_status(axk, cuda_device):
    import torch
    from gpu_util import Guarded, dev, sync

    table, ids = wl.embedding_inputs_np(9, vocab=500, hidden=64)
    ids[4] = 500
    ids[7] = 0xFFFFFFFF
    out = Guarded(9 * 64 * 2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert axk.embedding_gather(0, dev(table), 500, 64, dev(ids), 9, out.ptr, status) == axk.AXIOM_OK
    sync()
    got = out.payload(np.uint16).reshape(9, 64)
    assert np.array_equal(got, ol.embedding_gather_bf16(table, ids))
    assert not got[4].any() and not got[7].any()
    assert int(status.item()) == axk.STATUS_WORD_BAD_ADDRESS


@pytest.mark.parametrize("count", [1, 7, 8, 9, 5120, 8 * 5120 + 3, 1 << 20])
def test_add_matches_oracle(axk, cuda_device, count):
    from gpu_util import Guarded, dev, sync

    rng = np.random.default_rng(count)
    a = wl.to_bf16_bits(rng.standard_normal(count).astype(np.float32) * 3)
    b = wl.to_bf16_bits(rng.standard_normal(count).astype(np.float32))
    out = Guarded(count * 2)
    assert axk.add_bf16(0, dev(a), dev(b), out.ptr, count) == axk.AXIOM_OK
    sync()
    assert out.guards_intact()
    assert np.array_equal(out.payload(np.uint16), ol.add_bf16(a, b))

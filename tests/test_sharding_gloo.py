"""Row sharding across ranks: partition properties, and a world_size-2 gloo run on CPU in which
each rank computes its row range with the CPU oracle and the gathered per-row digests must equal
those of the unsharded computation."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sharding = importlib.import_module("axiom-kernel_b200.sharding")


@pytest.mark.parametrize("total", [0, 1, 15, 16, 17, 100, 4096, 8192, 8200])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_row_ranges_tile_the_job_on_page_boundaries(total, world):
    ranges = [sharding.row_range(total, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == total
    for (lo, hi), (lo2, _) in zip(ranges, ranges[1:]):
        assert hi == lo2
    for lo, hi in ranges:
        assert 0 <= lo <= hi <= total
        assert (lo % 16 == 0 or lo == total) and (hi % 16 == 0 or hi == total)
    sizes = [hi - lo for lo, hi in ranges]
    assert max(sizes) - min(sizes) <= 16 + 15  # balanced to one page (+ the short tail)


def test_row_range_rejects_bad_arguments():
    for bad in ((10, 0, 0), (10, 2, 2), (10, 2, -1), (-1, 2, 0)):
        with pytest.raises(ValueError):
            sharding.row_range(*bad)


def test_row_digests_see_every_byte():
    a = np.arange(64, dtype=np.uint16).reshape(4, 16)
    b = np.arange(8, dtype=np.uint8).reshape(4, 2)
    base = sharding.row_digests(a, b)
    a2 = a.copy(); a2[2, 5] ^= 1
    b2 = b.copy(); b2[3, 1] ^= 0x80
    assert (sharding.row_digests(a2, b) != base).tolist() == [False, False, True, False]
    assert (sharding.row_digests(a, b2) != base).tolist() == [False, False, False, True]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total_rows, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch.distributed as dist
    import oracle_lib as ol

    wl = importlib.import_module("axiom-kernel_b200.workloads")
    sh = importlib.import_module("axiom-kernel_b200.sharding")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(total_rows, 512)

    def compute(lo, hi):
        res, norm, codes, scales = ol.add_rmsnorm_nvfp4_bf16(hidden[lo:hi], residual[lo:hi], gamma, 1e-6, 64.0)
        return res, codes, scales

    digests = sh.sharded_digests(dist, total_rows, compute)
    slowest = sh.max_over_ranks(dist, float(rank + 1))
    np.save(Path(out_dir) / f"digests_{rank}.npy", digests)
    (Path(out_dir) / f"max_{rank}.txt").write_text(str(slowest))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total_rows", [100, 16])
def test_two_ranks_reproduce_the_unsharded_job(tmp_path, total_rows):
    import torch.multiprocessing as mp

    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib as ol

    wl = importlib.import_module("axiom-kernel_b200.workloads")
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, total_rows, str(tmp_path)), nprocs=world, join=True)
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(total_rows, 512)
    res, norm, codes, scales = ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, 64.0)
    want = sharding.row_digests(res, codes, scales)
    for rank in range(world):
        got = np.load(tmp_path / f"digests_{rank}.npy")
        assert np.array_equal(got, want)
        assert float((tmp_path / f"max_{rank}.txt").read_text()) == float(world)

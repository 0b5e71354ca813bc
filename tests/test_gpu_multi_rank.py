"""Row sharding on real GPUs: two ranks (one process per GPU, NCCL) each run the CUDA path on their page-aligned
row range; the gathered per-row digests must equal those of one GPU doing the whole job.  Needs two GPUs."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _compute(axk, wl, torch, device_index, hidden, residual, gamma, lo, hi, G):
    """add + RMSNorm + NVFP4 on rows [lo, hi) on the given GPU -> (residual, codes, scales) as numpy."""
    dev = torch.device("cuda", device_index)
    n, cols = hi - lo, hidden.shape[1]
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev)
    h, r, g = to(hidden[lo:hi]), to(residual[lo:hi]), to(gamma)
    codes = torch.empty((n, cols // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((n, cols // 16), dtype=torch.uint8, device=dev)
    assert axk.add_rmsnorm_nvfp4(device_index, h, r, g, 1e-6, n, cols, G, None, codes, scales, 0) == axk.AXIOM_OK
    torch.cuda.synchronize(dev)
    return r.cpu().numpy().view(np.uint16), codes.cpu().numpy(), scales.cpu().numpy()


def _worker(rank, world, port, total_rows, cols, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    axk = importlib.import_module("axiom-kernel_b200")
    wl = importlib.import_module("axiom-kernel_b200.workloads")
    sh = importlib.import_module("axiom-kernel_b200.sharding")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(total_rows, cols)
    digests = sh.sharded_digests(dist, total_rows,
                                 lambda lo, hi: _compute(axk, wl, torch, rank, hidden, residual, gamma, lo, hi, 64.0),
                                 device=torch.device("cuda", rank))
    np.save(Path(out_dir) / f"digests_{rank}.npy", digests)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_reproduce_one(axk, cuda_device, tmp_path):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    wl = importlib.import_module("axiom-kernel_b200.workloads")
    sh = importlib.import_module("axiom-kernel_b200.sharding")
    total_rows, cols, world = 1000, 5120, 2
    mp.spawn(_worker, args=(world, _free_port(), total_rows, cols, str(tmp_path)), nprocs=world, join=True)
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(total_rows, cols)
    want = sh.row_digests(*_compute(axk, wl, torch, 0, hidden, residual, gamma, 0, total_rows, 64.0))
    for rank in range(world):
        assert np.array_equal(np.load(tmp_path / f"digests_{rank}.npy"), want)

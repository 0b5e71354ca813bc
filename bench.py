#!/usr/bin/env python
"""Benchmark of the fused elementwise / reduction / quantize path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (one "step" = one pass of the hot path over one batch):
fused residual-add + RMSNorm + NVFP4 quantize over BF16 [8192 x 5120] per GPU
(hidden, residual ~N(0,1); gamma = 1+N(0,0.02); eps 1e-6).  Rows are
independent, so N GPUs each process their own 8192 rows (weak scaling, no
collective in the data path; NCCL only carries the timing reduction).

The JSON line carries, besides the contract keys:
  ops            device-timed figures of the other benchmark configurations (NVFP4 quantize,
                 q/k-norm + RoPE + paged KV, SwiGLU + FP8, decode chain ...): microseconds, GB/s,
                 fraction of the measured HBM peak, and the same bytes moved by dst.copy_(src)
                 (`copy_us`, `vs_copy` = copy time / kernel time) as a size-matched ceiling
  strong         strong scaling: ONE global job (8192 rows of configuration 2, 16384 rows of
                 configuration 4) split by rows over the ranks, time = slowest rank
  reference_gpu  the reference's own CUDA kernels (compiled for sm_100a into oracle/_ref) issued the
                 way the reference issues them — 8 rows per launch on F32 tensors — over the same rows
  roofline       HBM roofline of the dominant kernel (algorithmic bytes / CUDA-event time)
  e2e            same metric through the host-I/O C-ABI entry (pinned host buffers,
                 H2D + kernel + D2H inside the timed region)
  cpu_baseline   the CPU oracle timed on a bounded sample on this box's host cores

With --impl reference the CPU restatement of the reference's arithmetic (the
reference has no CPU path of its own for these ops) is timed on all host cores,
all rows of the workload per step.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ROWS = 8192
COLS = 5120
NSETS = 4  # rotating buffer sets so no step finds its inputs in L2 (126 MB)
HEADLINE_PROFILE = ROOT / "profiles" / "add_rmsnorm_nvfp4_8192x5120.md"
METRIC = "fused_add_rmsnorm_nvfp4_tokens_per_s"
UNIT = "tokens/s"


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def profiled_dram_bytes():
    """dram__bytes_read.sum + dram__bytes_write.sum of one headline launch, read from the committed ncu summary
    (None when the file or the figures are missing): the run itself does not measure DRAM traffic."""
    try:
        text = HEADLINE_PROFILE.read_text()
    except OSError:
        return None
    total = 0.0
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        for line in text.splitlines():
            if f"`{key}`" in line:
                cell = line.split("|")[2].strip().replace(",", "").split()
                scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(cell[1] if len(cell) > 1 else "byte")
                if scale is None:
                    return None
                total += float(cell[0]) * scale
                break
        else:
            return None
    return int(total)


def workload_config(rows, cols):
    algo = bytes_add_rmsnorm_nvfp4(rows, cols)
    return {"workload": f"fused residual-add + RMSNorm + NVFP4 quantize, BF16 [{rows}x{cols}] per GPU, "
                        f"eps 1e-6, gamma 1+N(0,0.02)",
            "rows_per_gpu": rows, "cols": cols,
            "l2": f"inputs larger than L2: {NSETS} rotating buffer sets of {algo / 1e6:.0f} MB",
            "partition": "token rows, no collective"}


def bytes_add_rmsnorm_nvfp4(rows, cols):
    # hidden R + residual R + residual W + codes W + scales W + gamma R
    return 3 * rows * cols * 2 + rows * cols // 2 + rows * cols // 16 + cols * 2


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons during the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def event_time_ms(torch, stream, fn, iters):
    """Time `iters` calls of fn (each enqueues on `stream`) with CUDA events on that stream."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for i in range(iters):
        fn(i)
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def rounded(x, digits=4):
    """Floats of the ops / strong / reference_gpu blocks to a few significant digits: the line stays short."""
    if isinstance(x, float):
        return float(f"{x:.{digits}g}")
    if isinstance(x, dict):
        return {k: rounded(v, digits) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [rounded(v, digits) for v in x]
    return x


def load_reference_kernels():
    """oracle/_ref/libaxiom_ref.so (the reference's own kernels built for sm_100a), or None.  Benchmark baseline only."""
    import ctypes as C

    path = ROOT / "oracle" / "_ref" / "libaxiom_ref.so"
    if not path.exists():
        return None
    try:
        lib = C.CDLL(str(path))
        vp, u32, f32 = C.c_void_p, C.c_uint32, C.c_float
        lib.ref_time_add_rmsnorm_then_quantize.argtypes = [vp, vp, vp, vp, f32, vp, vp, u32, u32, u32, vp, vp]
        lib.ref_time_quantize.argtypes = [vp, f32, vp, vp, u32, u32, u32, u32, vp, vp]
        lib.ref_time_swiglu_then_fp8.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, vp, vp]
        return lib
    except (OSError, AttributeError):
        return None


def reference_gpu_baseline(torch, wl, device, G, configs=("add_rmsnorm_nvfp4", "nvfp4_quantize", "swiglu_fp8")):
    """The reference's own CUDA kernels over the same rows, issued as the reference issues them: 8 token rows per
    launch (its fixed batch), F32 tensors holding BF16 values, one launch per fused step.  Outside every product
    timed region.  Returns None where oracle/_ref has not been built."""
    import ctypes as C

    ref = load_reference_kernels()
    if ref is None:
        return None
    out = {"kind": "oracle/_ref: reference kernels compiled for sm_100a, 8 rows per launch, F32 storage", "unit": UNIT}
    ms, launches = C.c_float(0.0), C.c_uint32(0)
    with torch.cuda.device(device):
        if "add_rmsnorm_nvfp4" in configs:
            hidden, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, ROWS, COLS)
            res32, add32, w32 = residual.float(), hidden.float(), gamma.float()
            norm32 = torch.empty_like(res32)
            codes = torch.empty((ROWS, COLS // 2), dtype=torch.uint8, device=device)
            planes = torch.zeros((ROWS // 8) * ((COLS // 16 + 3) // 4) * 512, dtype=torch.uint8, device=device)
            torch.cuda.synchronize()
            rc = ref.ref_time_add_rmsnorm_then_quantize(res32.data_ptr(), add32.data_ptr(), w32.data_ptr(), norm32.data_ptr(), G,
                                                        codes.data_ptr(), planes.data_ptr(), ROWS, 1, 3, C.byref(ms), C.byref(launches))
            if rc == 0 and ms.value > 0:
                out["add_rmsnorm_nvfp4"] = {"rows": ROWS, "ms": ms.value, "value": ROWS / (ms.value * 1e-3), "launches": launches.value}
                out["value"] = out["add_rmsnorm_nvfp4"]["value"]
                out["launches"] = launches.value
            del res32, add32, w32, norm32, codes, planes
        if "nvfp4_quantize" in configs:
            rows = 4096
            x32 = wl.quantize_input_torch(torch, device, rows, COLS, seed=0).float()
            codes = torch.empty((rows, COLS // 2), dtype=torch.uint8, device=device)
            planes = torch.zeros((rows // 8) * ((COLS // 16 + 3) // 4) * 512, dtype=torch.uint8, device=device)
            torch.cuda.synchronize()
            rc = ref.ref_time_quantize(x32.data_ptr(), G, codes.data_ptr(), planes.data_ptr(), rows, COLS, 1, 3, C.byref(ms), C.byref(launches))
            if rc == 0 and ms.value > 0:
                out["nvfp4_quantize"] = {"rows": rows, "ms": ms.value, "value": rows / (ms.value * 1e-3), "launches": launches.value}
            del x32, codes, planes
        if "swiglu_fp8" in configs:
            rows, W = 16384, wl.FFN
            gu = wl.swiglu_input_torch(torch, device, rows, W)
            gate32, up32 = gu[:, :W].float().contiguous(), gu[:, W:].float().contiguous()
            del gu
            mid = torch.empty((8, W), dtype=torch.float32, device=device)
            codes = torch.empty((rows, W), dtype=torch.uint8, device=device)
            scales = torch.empty(rows, dtype=torch.float32, device=device)
            torch.cuda.synchronize()
            rc = ref.ref_time_swiglu_then_fp8(gate32.data_ptr(), up32.data_ptr(), mid.data_ptr(), codes.data_ptr(), scales.data_ptr(),
                                              rows, W, 1, 2, C.byref(ms), C.byref(launches))
            if rc == 0 and ms.value > 0:
                out["swiglu_fp8"] = {"rows": rows, "ms": ms.value, "value": rows / (ms.value * 1e-3), "launches": launches.value}
            del gate32, up32, mid, codes, scales
        torch.cuda.empty_cache()
    return rounded(out)


def host_cores():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def reference_arm(args):
    """CPU restatement of the reference's arithmetic for the headline op: every row of the workload per step, all
    host threads.  (The reference has no CPU implementation of these ops; its CUDA kernels are timed as
    `reference_gpu` where a GPU and oracle/_ref are present.)"""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle_lib as ol

    wl = importlib.import_module("axiom-kernel_b200.workloads")
    hidden, residual, gamma = wl.add_rmsnorm_inputs_np(ROWS, COLS)
    pristine = residual.copy()
    # all host cores, also under torchrun, which exports OMP_NUM_THREADS=1 to its workers
    ol.o().axo_set_threads(host_cores())
    threads = ol.o().axo_get_threads()
    G = 100.0
    for _ in range(max(args.warmup, 1)):
        ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
    dt = (time.perf_counter() - t0) / args.steps
    del pristine
    value = ROWS / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(ROWS, COLS),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"all {ROWS} rows per step, OpenMP over rows",
                         "note": "CPU restatement of the reference's arithmetic; the reference has no CPU "
                                 "implementation of this op"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        import torch

        if torch.cuda.is_available():
            line["reference_gpu"] = reference_gpu_baseline(torch, wl, torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))), G,
                                                           configs=("add_rmsnorm_nvfp4",))
    except Exception as exc:  # the CPU figure stands on its own
        line["reference_gpu"] = {"unavailable": str(exc)[:120]}
    print(json.dumps(line), flush=True)
    return 0


def bind_to_gpu_numa_node(torch, local):
    """Keep this rank's threads (and so its page-locked buffers, placed by first touch) on the NUMA node the GPU hangs
    off, as numactl would in a deployment; with several ranks per host the host-I/O leg otherwise crosses sockets.
    Returns the node, or None when the topology cannot be read."""
    try:
        props = torch.cuda.get_device_properties(local)
        address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{address}/numa_node").read_text())
        if node < 0:
            return None
        cpus = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-ops", action="store_true", help="only the headline workload")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-reference-gpu", action="store_true", help="leave the reference's own kernels out (profiling aid)")
    ap.add_argument("--only", default=None,
                    choices=["add_rmsnorm", "add_rmsnorm_tiled", "fp8_epilogue", "nvfp4_quantize", "qk", "swiglu_fp8", "swiglu_nvfp4", "sigmoid_gate", "fp8_quantize",
                             "top1", "chain"],
                    help="run one configuration alone (profiling aid): device-timed, no e2e / CPU legs")
    ap.add_argument("--rows", type=int, default=0, help="with --only: override the token count")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import numpy as np
    import torch

    axk = importlib.import_module("axiom-kernel_b200")
    wl = importlib.import_module("axiom-kernel_b200.workloads")
    sharding = importlib.import_module("axiom-kernel_b200.sharding")
    lib = axk.lib()  # raises if the CUDA library is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    numa_node = bind_to_gpu_numa_node(torch, local) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    device = torch.device("cuda", local)
    stream = torch.cuda.Stream(device)
    peak, peak_kind = measured_peak_gbs()
    if args.only and args.only != "add_rmsnorm":
        res = bench_other_ops(torch, axk, wl, local, device, stream, peak, only=args.only, rows_override=args.rows,
                              iters=args.steps, warm=args.warmup)
        print(json.dumps({"only": args.only, "result": res}), flush=True)
        return 0
    global ROWS
    if args.only == "add_rmsnorm":
        args.skip_e2e = args.skip_ops = args.skip_cpu = True
        if args.rows:
            ROWS = args.rows

    # ---- headline: add + RMSNorm + NVFP4, device resident ---------------------------------
    sets = []
    for s in range(NSETS):
        hidden, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, ROWS, COLS)
        if s:
            hidden = hidden.roll(s, 0)
            residual = residual.roll(s, 0)
        sets.append(dict(hidden=hidden, residual=residual, gamma=gamma,
                         codes=torch.empty((ROWS, COLS // 2), dtype=torch.uint8, device=device),
                         scales=torch.empty((ROWS, COLS // 16), dtype=torch.uint8, device=device)))
    pristine = [s["residual"].clone() for s in sets]
    # global scale from the normalised tensor of set 0 (calibration step, outside any timed region)
    norm0 = torch.empty((ROWS, COLS), dtype=torch.bfloat16, device=device)
    rc = axk.add_rmsnorm_nvfp4(local, sets[0]["hidden"], sets[0]["residual"], sets[0]["gamma"], wl.EPS, ROWS, COLS, 1.0,
                               norm0, None, None, 0, stream)
    axk.check(rc, "calibration")
    torch.cuda.synchronize()
    G = wl.nvfp4_global_scale(float(norm0.float().abs().max().item()))
    sets[0]["residual"].copy_(pristine[0])
    del norm0

    def step(i):
        s = sets[i % NSETS]
        rc = axk.add_rmsnorm_nvfp4(local, s["hidden"], s["residual"], s["gamma"], wl.EPS, ROWS, COLS, G, None,
                                   s["codes"], s["scales"], 0, stream)
        if rc:
            axk.check(rc, "add_rmsnorm_nvfp4")

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    for s, p in zip(sets, pristine):
        s["residual"].copy_(p)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def keep_loaded(seconds):
        # the same kernel, untimed: the timed region is a few milliseconds, shorter than one nvidia-smi
        # sampling period, so the clocks are sampled over a window of identical load around it
        t_end = time.perf_counter() + seconds
        i = 0
        while time.perf_counter() < t_end:
            for _ in range(32):
                step(i)
                i += 1
            torch.cuda.synchronize()

    keep_loaded(0.5)
    launches0 = int(lib.axiom_b200_kernel_launch_count())
    ms = event_time_ms(torch, stream, step, args.steps)
    launches = int(lib.axiom_b200_kernel_launch_count()) - launches0
    keep_loaded(0.3)
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "0.5 s of the same launches before and 0.3 s after the timed region"
    if dist:
        ms = sharding.max_over_ranks(dist, ms, device)  # a multi-GPU step takes as long as its slowest rank
        dist.barrier()
    value = world * ROWS / (ms * 1e-3)
    algo = bytes_add_rmsnorm_nvfp4(ROWS, COLS)
    achieved = algo / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "io_dtype": "bf16 in; bf16 residual, e2m1 codes + e4m3 block scales out", "data": "synthetic",
        "config": workload_config(ROWS, COLS),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": profiled_dram_bytes() if (ROWS, COLS) == (8192, 5120) else None,
                     "traffic_source": "not measured by this run: dram__bytes_read.sum + dram__bytes_write.sum of one ncu "
                                       "capture of this launch, read from profiles/" + HEADLINE_PROFILE.name,
                     "peak_kind": peak_kind, "kernel": "add_rmsnorm_stream_kernel<kBf16, true, 5120>",
                     "algorithmic_bytes_per_launch": algo},
        "gpu_launches": launches,
        "clocks": clocks,
    }

    # ---- e2e through the host-I/O C-ABI entry ------------------------------------------------
    if not args.skip_e2e:
        rt = axk.Runtime(local)
        h_hidden = sets[0]["hidden"].cpu().pin_memory()
        h_res = pristine[0].cpu().pin_memory()
        h_gamma = sets[0]["gamma"].cpu().pin_memory()
        h_codes = torch.empty((ROWS, COLS // 2), dtype=torch.uint8).pin_memory()
        h_scales = torch.empty((ROWS, COLS // 16), dtype=torch.uint8).pin_memory()

        def e2e_step():
            rc = lib.axiom_runtime_add_rmsnorm_nvfp4_bf16(rt.handle, h_hidden.data_ptr(), h_res.data_ptr(),
                                                          h_gamma.data_ptr(), wl.EPS, ROWS, COLS, G,
                                                          h_codes.data_ptr(), h_scales.data_ptr())
            if rc:
                axk.check(rc, "host-I/O add_rmsnorm_nvfp4")

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        e2e_steps = max(5, min(args.steps, 30))
        solo_ms = None
        if dist:
            # rank 0 alone first: what one rank gets from the host link when nobody shares it
            dist.barrier()
            if rank == 0:
                t0 = time.perf_counter()
                for _ in range(e2e_steps):
                    e2e_step()
                torch.cuda.synchronize()
                solo_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
        if dist:
            e2e_ms = sharding.max_over_ranks(dist, e2e_ms, device)
        # the same leg with every buffer forced through the staging slots and the copy engines (informative)
        os.environ["AXIOM_B200_HOST_IO"] = "staged"
        e2e_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            e2e_step()
        torch.cuda.synchronize()
        staged_ms = (time.perf_counter() - t0) / 5 * 1e3
        del os.environ["AXIOM_B200_HOST_IO"]
        if dist:
            staged_ms = sharding.max_over_ranks(dist, staged_ms, device)
        # the bare transfers of one step (inputs host -> device on one stream, results device -> host on another, both
        # directions at once, nothing computed): what the host link allows for these bytes, every rank at the same time
        d_in = [torch.empty_like(h_hidden, device=device), torch.empty_like(h_res, device=device)]
        d_out = [torch.empty_like(h_res, device=device), torch.empty_like(h_codes, device=device), torch.empty_like(h_scales, device=device)]
        h_res_out = torch.empty_like(h_res).pin_memory()
        up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)

        def bare_transfers():
            with torch.cuda.stream(up):
                d_in[0].copy_(h_hidden, non_blocking=True)
                d_in[1].copy_(h_res, non_blocking=True)
            with torch.cuda.stream(down):
                h_res_out.copy_(d_out[0], non_blocking=True)
                h_codes.copy_(d_out[1], non_blocking=True)
                h_scales.copy_(d_out[2], non_blocking=True)

        bare_transfers()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            bare_transfers()
        torch.cuda.synchronize()
        link_ms = (time.perf_counter() - t0) / 5 * 1e3
        if dist:
            link_ms = sharding.max_over_ranks(dist, link_ms, device)
        del d_in, d_out, h_res_out
        line["e2e"] = {"value": world * ROWS / (e2e_ms * 1e-3), "unit": UNIT,
                       "h2d_bytes_per_step": 2 * ROWS * COLS * 2 + COLS * 2,
                       "d2h_bytes_per_step": ROWS * COLS * 2 + ROWS * COLS // 2 + ROWS * COLS // 16,
                       "ms_per_step": e2e_ms, "steps": e2e_steps, "staged_copy_engine_ms_per_step": staged_ms,
                       "bare_transfers_ms_per_step": link_ms,
                       "numa_node": numa_node,
                       "api": "axiom_runtime_add_rmsnorm_nvfp4_bf16, pinned host buffers; the kernel reads and writes mapped host memory over PCIe"}
        if solo_ms:
            # efficiency of the host-I/O leg at this N against one rank alone on the same host in the same run:
            # the ranks share one host's memory and PCIe root, so this falls with N although the GPUs share nothing
            line["e2e"]["one_rank_alone_ms_per_step"] = solo_ms
            line["e2e"]["efficiency_vs_one_rank"] = (solo_ms / e2e_ms)
        rt.close()
        del h_hidden, h_res, h_codes, h_scales

    # ---- the other configurations, device timed (rank 0 reports) ----------------------------------
    del sets, pristine
    torch.cuda.empty_cache()
    if not args.skip_ops:
        line["ops"] = rounded(bench_other_ops(torch, axk, wl, local, device, stream, peak))
        # strong scaling: one global job split by rows over the ranks (every rank takes part)
        line["strong"] = rounded(bench_strong(torch, axk, wl, sharding, dist, world, rank, local, device, stream, G, peak,
                                              iters=max(20, min(args.steps, 100)), warm=max(args.warmup, 3)))
        # the reference's own kernels on the same rows (rank 0; outside every product timed region)
        if rank == 0 and not args.skip_reference_gpu:
            try:
                line["reference_gpu"] = reference_gpu_baseline(torch, wl, device, G)
            except Exception as exc:
                line["reference_gpu"] = {"unavailable": str(exc)[:120]}
        if dist:
            dist.barrier()

    # ---- CPU baseline: the oracle on a bounded sample, rank 0 at N=1 only -------------------------
    if rank == 0 and world == 1 and not args.skip_cpu:
        sys.path.insert(0, str(ROOT / "tests"))
        import oracle_lib as ol

        sample_rows = 2048
        hidden, residual, gamma = wl.add_rmsnorm_inputs_np(sample_rows, COLS)
        threads = ol.o().axo_get_threads()
        ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 200):
            ol.add_rmsnorm_nvfp4_bf16(hidden, residual, gamma, 1e-6, G)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": sample_rows / dt, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{sample_rows} of {ROWS} rows, {reps} repetitions, OpenMP over rows"}
    elif rank == 0:
        line["cpu_baseline"] = None

    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        # the long per-configuration block goes first, the short judged blocks last (a truncated log keeps them)
        order = ["ops"] + [k for k in line if k not in ("ops", "strong", "reference_gpu", "roofline", "e2e", "cpu_baseline", "clocks")]
        order += ["strong", "reference_gpu", "e2e", "cpu_baseline", "clocks", "roofline"]
        print(json.dumps({k: line[k] for k in order if k in line}), flush=True)
    return 0


def bench_other_ops(torch, axk, wl, local, device, stream, peak, only=None, rows_override=0, iters=50, warm=5):
    """Device-timed throughput of configurations 1, 3, 4 and the decode chain (5)."""
    out = {}

    def want(name):
        return only is None or only == name

    def timed(fn, n=None):
        n = min(n, iters) if n else iters
        # Inputs are generated on torch's current stream and the kernels run on `stream`: without this, the warm-up
        # launches would overlap the generation, and torch's allocator may have handed an output tensor the block of
        # a generation temporary that is still in flight on the other stream (the kernel's writes then corrupt the
        # input being generated, and a garbage input takes the kernels' slow paths).
        torch.cuda.synchronize()
        for i in range(warm):
            fn(i)
        return event_time_ms(torch, stream, fn, n)

    copy_cache = {}

    def matched_copy_ms(algo):
        """dst.copy_(src) of algo/2 bytes (so the copy moves the same bytes: half read, half written), rotating
        buffer pairs larger than L2 in total, timed with the same events on the same stream."""
        if algo in copy_cache:
            return copy_cache[algo]
        half = max(16, algo // 2 // 16 * 16)
        nsets = max(2, min(16, -(-400_000_000 // algo)))
        src = [torch.empty(half, dtype=torch.uint8, device=device).random_(0, 255) for _ in range(nsets)]
        dst = [torch.empty(half, dtype=torch.uint8, device=device) for _ in range(nsets)]

        def step(i):
            dst[i % nsets].copy_(src[i % nsets])

        with torch.cuda.stream(stream):
            for i in range(max(warm, 3)):
                step(i)
            ms = event_time_ms(torch, stream, step, max(20, min(iters, 100)))
        del src, dst
        copy_cache[algo] = ms
        return ms

    def report(name, ms, algo, rows, note):
        # `note` documents the call site only: the line carries numbers
        gbs = algo / (ms * 1e-3) / 1e9
        out[name] = {"us": ms * 1e3, "gbs": gbs, "frac": gbs / peak, "tokens_per_s": rows / (ms * 1e-3), "bytes": algo}
        if algo >= (1 << 20):
            cms = matched_copy_ms(algo)
            out[name]["copy_us"] = cms * 1e3
            out[name]["vs_copy"] = cms / ms

    if only is None or only == "add_rmsnorm_tiled":
        bench_add_rmsnorm_tiled(torch, axk, wl, local, device, stream, timed, report, rows_override or 8192)
    if want("fp8_epilogue"):
        bench_fp8_epilogue(torch, axk, wl, local, device, stream, timed, report, rows_override or 8192)
    if want("nvfp4_quantize"):
        bench_nvfp4_quantize(torch, axk, wl, local, device, stream, timed, report, rows_override or 4096)
    if want("qk"):
        bench_qk(torch, axk, wl, local, device, stream, timed, report, rows_override or 8192)
    if want("swiglu_fp8") or want("swiglu_nvfp4"):
        bench_swiglu(torch, axk, wl, local, device, stream, timed, report, rows_override or 16384, want)
    if want("sigmoid_gate"):
        bench_sigmoid_gate(torch, axk, wl, local, device, stream, timed, report, rows_override or 8192)
    if want("fp8_quantize"):
        bench_fp8_quantize(torch, axk, wl, local, device, stream, timed, report, rows_override or 16384)
    if want("top1"):
        bench_top1(torch, axk, wl, local, device, stream, timed, report)
    if want("chain"):
        out["decode_chain"] = bench_chain(torch, axk, wl, local, device, stream, timed, peak)
    return out


def bench_strong(torch, axk, wl, sharding, dist, world, rank, local, device, stream, G, peak, iters=50, warm=5):
    """Strong scaling: ONE global job split by token rows over the ranks (sharding.row_range, 16-row granules so no
    KV page is shared), no data-path collective; time = the slowest rank.  Configuration 2 at 8192 global rows and
    configuration 4 at 16384.  `full_us` is the whole job on one GPU measured in the same run (every rank measures it,
    the slowest counts), so `efficiency` = full_us / (n_gpus * shard_us) needs no other run; `floor_us` is the same
    kernel on 16 rows, the launch-bound time a shard converges to as N grows."""
    out = {"n_gpus": world}

    def timed(fn, n):
        # Shards are short (tens of microseconds) and each measurement follows allocations and frees, during which
        # the GPU idles and drops its clocks; a long run of the heavier kernels, on the other hand, reaches the power
        # cap.  So: warm up by TIME, briefly (60 ms of the same launches), then take the median of seven batches of a
        # few milliseconds each.
        torch.cuda.synchronize()  # inputs are generated on torch's stream, the kernels run on another: order them
        t_end = time.perf_counter() + 0.06
        i = 0
        while time.perf_counter() < t_end or i < warm:
            for _ in range(8):
                fn(i)
                i += 1
            torch.cuda.synchronize()
        probe = event_time_ms(torch, stream, fn, 8)
        n = max(8, min(n, int(3.0 / max(probe, 1e-3))))
        batches = sorted(event_time_ms(torch, stream, fn, n) for _ in range(7))
        return batches[3]

    def slowest(ms):
        return sharding.max_over_ranks(dist, ms, device) if dist else ms

    def every_rank(ms):
        if not dist:
            return [ms * 1e3]
        t = torch.tensor([ms * 1e3], dtype=torch.float64, device=device)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return [float(x.item()) for x in parts]

    def sets_for(bytes_per_set):
        return max(2, min(16, -(-400_000_000 // max(bytes_per_set, 1))))  # rotating sets: 400 MB and more in total

    # ---- configuration 2: add + RMSNorm + NVFP4, 8192 global rows
    total = 8192
    lo, hi = sharding.row_range(total, world, rank)

    def norm_sets(rows):
        n = sets_for(bytes_add_rmsnorm_nvfp4(rows, COLS))
        hidden, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, rows, COLS)
        return [(hidden.roll(k, 0) if k else hidden, residual.roll(k, 0) if k else residual, gamma,
                 torch.empty((rows, COLS // 2), dtype=torch.uint8, device=device),
                 torch.empty((rows, COLS // 16), dtype=torch.uint8, device=device)) for k in range(n)]

    def norm_time(rows):
        sets = norm_sets(rows)

        def step(i):
            h, r, g, c, sc = sets[i % len(sets)]
            axk.add_rmsnorm_nvfp4(local, h, r, g, wl.EPS, rows, COLS, G, None, c, sc, 0, stream)

        return timed(step, iters)

    mine = norm_time(hi - lo) if hi > lo else 0.0
    per_rank = every_rank(mine)
    shard_ms = slowest(mine)
    full_ms = slowest(norm_time(total)) if world > 1 else shard_ms
    floor_ms = norm_time(16)
    out["add_rmsnorm_nvfp4"] = {"global_rows": total, "rows_per_rank": hi - lo, "shard_us": shard_ms * 1e3,
                                "tokens_per_s": total / (shard_ms * 1e-3), "full_us": full_ms * 1e3,
                                "efficiency": full_ms / (world * shard_ms), "floor_us": floor_ms * 1e3,
                                "shard_us_per_rank": per_rank,
                                "kernel": "stream kernel from 296 rows per rank, one CTA per row below"}
    torch.cuda.empty_cache()

    # ---- configuration 4: SwiGLU + FP8, 16384 global rows
    total, W = 16384, wl.FFN
    lo, hi = sharding.row_range(total, world, rank)

    def swiglu_time(rows):
        n = 1 if rows * W * 5 + rows * 4 > 400_000_000 else sets_for(rows * W * 5)
        sets = [(wl.swiglu_input_torch(torch, device, rows, W, seed=4 + k), torch.empty((rows, W), dtype=torch.uint8, device=device),
                 torch.empty((rows,), dtype=torch.float32, device=device)) for k in range(n)]

        def step(i):
            gu, c, sc = sets[i % n]
            axk.swiglu_fp8(local, gu, rows, W, c, sc, stream)

        return timed(step, min(iters, 30))

    mine = swiglu_time(hi - lo) if hi > lo else 0.0
    per_rank = every_rank(mine)
    shard_ms = slowest(mine)
    torch.cuda.empty_cache()
    full_ms = slowest(swiglu_time(total)) if world > 1 else shard_ms
    torch.cuda.empty_cache()
    floor_ms = swiglu_time(16)
    out["swiglu_fp8"] = {"global_rows": total, "rows_per_rank": hi - lo, "shard_us": shard_ms * 1e3,
                         "tokens_per_s": total / (shard_ms * 1e-3), "full_us": full_ms * 1e3,
                         "efficiency": full_ms / (world * shard_ms), "floor_us": floor_ms * 1e3, "shard_us_per_rank": per_rank}
    torch.cuda.empty_cache()
    return out


def bench_add_rmsnorm_tiled(torch, axk, wl, local, device, stream, timed, report, rows):
    # config 2 with the block scales written straight into the cuBLASLt VEC16_UE4M3 tile layout (what the next GEMM reads)
    cols = COLS
    sets = []
    for s in range(NSETS):
        hidden, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, rows, cols)
        plane = int(axk.lib().axiom_nvfp4_scale_plane_bytes(rows, cols // 16, 1))
        sets.append((hidden, residual, gamma, torch.empty((rows, cols // 2), dtype=torch.uint8, device=device),
                     torch.zeros(plane, dtype=torch.uint8, device=device)))

    def step(i):
        h, r, g, c, s = sets[i % NSETS]
        axk.add_rmsnorm_nvfp4(local, h, r, g, wl.EPS, rows, cols, 90.0, None, c, s, 1, stream)

    ms = timed(step)
    report("add_rmsnorm_nvfp4_tiled_scales", ms, bytes_add_rmsnorm_nvfp4(rows, cols), rows,
           "config 2, block scales in the cuBLASLt tile layout")


def bench_fp8_epilogue(torch, axk, wl, local, device, stream, timed, report, rows):
    # config 2 with the addend taken as raw F32 accumulators of an FP8 GEMM (scale epilogue folded into the prologue)
    cols = COLS
    sets = []
    for s in range(NSETS):
        _, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, rows, cols)
        g = torch.Generator(device=device).manual_seed(70 + s)
        raw = torch.randn((rows, cols), generator=g, device=device, dtype=torch.float32) * 40.0
        wscale = (0.01 + 0.005 * torch.rand(cols, generator=g, device=device)).to(torch.bfloat16)
        iscale = 0.02 + 0.01 * torch.rand(rows, generator=g, device=device, dtype=torch.float32)
        sets.append((raw, wscale, iscale, residual, gamma, torch.empty((rows, cols // 2), dtype=torch.uint8, device=device),
                     torch.empty((rows, cols // 16), dtype=torch.uint8, device=device)))

    def step(i):
        raw, ws, isc, r, g, c, s = sets[i % NSETS]
        axk.fp8_epilogue_add_rmsnorm_nvfp4(local, raw, ws, isc, r, g, wl.EPS, rows, cols, 90.0, None, c, s, 0, stream)

    ms = timed(step)
    report("fp8_epilogue_add_rmsnorm_nvfp4", ms, rows * cols * 4 + 2 * rows * cols * 2 + rows * cols // 2 + rows * cols // 16 +
           cols * 4 + rows * 4, rows, "raw F32 GEMM accumulators + weight/token scales as the addend (FP8 path)")


def bench_nvfp4_quantize(torch, axk, wl, local, device, stream, timed, report, rows):
    # config 1: BF16 -> NVFP4, [4096 x 5120]; 8 rotating inputs (8 x 42 MB > L2)
    cols = 5120
    xs = [wl.quantize_input_torch(torch, device, rows, cols, seed=s) for s in range(8)]
    codes = [torch.empty((rows, cols // 2), dtype=torch.uint8, device=device) for _ in range(8)]
    scales = [torch.empty((rows, cols // 16), dtype=torch.uint8, device=device) for _ in range(8)]
    G = wl.nvfp4_global_scale(float(xs[0].float().abs().max().item()))
    for layout, tag in ((0, "canonical"), (1, "tiled")):
        ms = timed(lambda i: axk.nvfp4_quantize(local, xs[i % 8], rows, cols, G, codes[i % 8], scales[i % 8], layout, stream))
        report(f"nvfp4_quantize_{tag}", ms, rows * cols * 2 + rows * cols // 2 + rows * cols // 16, rows,
               "config 1, 8 rotating buffer sets")


def bench_qk(torch, axk, wl, local, device, stream, timed, report, T):
    # config 3: q/k norm + RoPE + paged KV, T = 8192; 2 rotating sets (2 x 302 MB)
    qk_sets = []
    inv_freq = torch.empty(64, dtype=torch.float32, device=device)
    axk.check(axk.yarn_inv_freq(local, 128, wl.ROPE_THETA, wl.YARN_FACTOR, wl.YARN_ORIGINAL_CONTEXT, 32.0, 1.0, inv_freq, stream), "yarn")
    pool = torch.empty((wl.KV_BLOCKS * 16 * 1024,), dtype=torch.bfloat16, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for s in range(2):
        q, k, v, qg, kg, pos, tab = wl.qk_inputs_torch(torch, device, T, seed=3 + s)
        keep = (q, k, qg, kg, pos, tab)
        args = axk.make_qk_args(tokens=T, q_heads=64, k_heads=8, head_dim=128, rope_dim=128, flags=axk.QK_FLAG_RING,
                                eps=1e-6, mscale=axk.yarn_mscale(4.0), block_tokens=16, n_layers=1, layer=0,
                                pool_stride=1024, tbl_stride=wl.KV_BLOCKS, n_blocks=wl.KV_BLOCKS, q=q, k=k, q_gamma=qg,
                                k_gamma=kg, inv_freq=inv_freq, positions=pos, block_tables=tab, k_pool=pool,
                                status_word=status)
        qk_sets.append((args, keep))
    ms = timed(lambda i: axk.qk_norm_rope_paged(local, qk_sets[i % 2][0], stream))
    report("qk_norm_rope_paged_kv", ms, 2 * T * 64 * 128 * 2 + 2 * T * 8 * 128 * 2 + T * 4 + 4096 * 4 + 512, T,
           "config 3, Q in place, K to 16-token BF16 pages")
    # the same tokens with Q read from a q|gate-interleaved projection output and written to q_out (same algorithmic
    # bytes: the gate halves are not touched)
    split_sets = []
    for args, keep in qk_sets:
        q = keep[0]
        source = torch.cat([q.view(T, 64, 128), torch.zeros_like(q.view(T, 64, 128))], dim=2).contiguous()
        out = torch.empty_like(q)
        a2 = axk.QkRopeArgs.from_buffer_copy(args)
        a2.flags |= axk.QK_FLAG_Q_GATE_INTERLEAVED
        a2.q_bf16, a2.q_out_bf16 = source.data_ptr(), out.data_ptr()
        split_sets.append((a2, source, out))
    ms = timed(lambda i: axk.qk_norm_rope_paged(local, split_sets[i % 2][0], stream))
    report("qk_norm_rope_paged_kv_split_q_gate", ms, 2 * T * 64 * 128 * 2 + 2 * T * 8 * 128 * 2 + T * 4 + 4096 * 4 + 512, T,
           "config 3 with the query halves read from a [T][64][2*128] q|gate projection output")


def bench_swiglu(torch, axk, wl, local, device, stream, timed, report, T, want):
    # config 4: SwiGLU + FP8, T = 16384 (1.43 GB per pass: larger than L2 by itself)
    W = wl.FFN
    gu = wl.swiglu_input_torch(torch, device, T, W)
    if want("swiglu_fp8"):
        c8 = torch.empty((T, W), dtype=torch.uint8, device=device)
        s8 = torch.empty((T,), dtype=torch.float32, device=device)
        ms = timed(lambda i: axk.swiglu_fp8(local, gu, T, W, c8, s8, stream), n=20)
        report("swiglu_fp8", ms, T * 2 * W * 2 + T * W + T * 4, T, "config 4")
    if want("swiglu_nvfp4"):
        c4 = torch.empty((T, W // 2), dtype=torch.uint8, device=device)
        s4 = torch.empty((T, W // 16), dtype=torch.uint8, device=device)
        ms = timed(lambda i: axk.swiglu_nvfp4(local, gu, T, W, 40.0, c4, s4, 0, stream), n=20)
        report("swiglu_nvfp4", ms, T * 2 * W * 2 + T * W // 2 + T * W // 16, T, "SwiGLU -> NVFP4 (down-projection input)")


def bench_sigmoid_gate(torch, axk, wl, local, device, stream, timed, report, T):
    # attention output gate + o_proj activation quantize: [T x 64*128] attention and gate planes, 2 rotating sets
    W = 64 * 128
    sets = []
    for s in range(2):
        g = torch.Generator(device=device).manual_seed(40 + s)
        attn = torch.randn((T, W), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        gate = (torch.randn((T, W), generator=g, device=device, dtype=torch.float32) * 2).to(torch.bfloat16)
        sets.append((attn, gate, torch.empty((T, W // 2), dtype=torch.uint8, device=device),
                     torch.empty((T, W // 16), dtype=torch.uint8, device=device)))
    ms = timed(lambda i: axk.sigmoid_gate_nvfp4(local, sets[i % 2][0], sets[i % 2][1], T, W, 60.0, None, sets[i % 2][2],
                                                sets[i % 2][3], 1, stream))
    report("sigmoid_gate_nvfp4", ms, 2 * T * W * 2 + T * W // 2 + T * W // 16, T,
           "attention * sigmoid(gate) -> NVFP4 with tiled scales (o_proj input), 64 heads x 128")


def bench_fp8_quantize(torch, axk, wl, local, device, stream, timed, report, T):
    # plain BF16 -> FP8 E4M3 rows (the activation quantizer in front of an FP8 contraction): per-row scale, and a given one
    W = 8192
    n = 2
    xs = [wl.quantize_input_torch(torch, device, T, W, seed=70 + s) for s in range(n)]
    cs = [torch.empty((T, W), dtype=torch.uint8, device=device) for _ in range(n)]
    sc = torch.empty((T,), dtype=torch.float32, device=device)
    ms = timed(lambda i: axk.fp8_quantize(local, xs[i % n], T, W, cs[i % n], sc, None, stream))
    report("fp8_quantize", ms, T * W * 3 + T * 4, T, "BF16 -> FP8 E4M3 with a per-row scale, [T x 8192]")
    ms = timed(lambda i: axk.fp8_quantize_static(local, xs[i % n], T, W, 0.01, cs[i % n], stream))
    report("fp8_quantize_static", ms, T * W * 3, T, "BF16 -> FP8 E4M3 with a given scale, [T x 8192]")


def bench_top1(torch, axk, wl, local, device, stream, timed, report):
    # greedy selection over F32 logits: the decode-step tail (8 rows) and a prefill-sized batch
    for rows, vocab in ((8, 151936), (8, 248320), (256, 151936)):
        logits = torch.randn((rows, vocab), device=device, dtype=torch.float32)
        res = torch.empty((rows, 3), dtype=torch.int32, device=device)
        ms = timed(lambda i: axk.top1(local, logits, rows, vocab, res, stream))
        report(f"top1_{rows}x{vocab}", ms, rows * vocab * 4 + rows * 12, rows,
               "one launch, 8-CTA clusters; logits stay in L2 between iterations at 8 rows (latency figure)")


def bench_chain(torch, axk, wl, local, device, stream, timed, peak):
    # config 5: decode chain, microseconds per layer-chain, eager launches and one CUDA graph replay
    table, _ = wl.embedding_inputs_torch(torch, device, 1)
    inv_freq = torch.empty(64, dtype=torch.float32, device=device)
    axk.check(axk.yarn_inv_freq(local, 128, wl.ROPE_THETA, wl.YARN_FACTOR, wl.YARN_ORIGINAL_CONTEXT, 32.0, 1.0, inv_freq, stream), "yarn")
    status = torch.zeros(1, dtype=torch.int32, device=device)
    chain = {}
    # the launch floor of this box, measured the same way: the smallest kernel of the library (a 64-element BF16 add,
    # one CTA) three times per "chain", back to back and as eight chains per graph
    fa, fb = torch.zeros(64, dtype=torch.bfloat16, device=device), torch.zeros(64, dtype=torch.bfloat16, device=device)
    fo = torch.empty(64, dtype=torch.bfloat16, device=device)

    def floor_chain(_i, s=stream):
        for _ in range(3):
            axk.add_bf16(local, fa, fb, fo, 64, s)

    floor_eager_us = timed(floor_chain, n=200) * 1e3
    floor_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(floor_graph, stream=stream):
        for _ in range(8):
            floor_chain(0, torch.cuda.current_stream())
    for _ in range(3):
        floor_graph.replay()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    f0.record()
    for _ in range(50):
        floor_graph.replay()
    f1.record()
    torch.cuda.synchronize()
    chain["launch_floor"] = {"eager_us": floor_eager_us, "graph8_us_per_chain": f0.elapsed_time(f1) / (50 * 8) * 1e3,
                             "what": "three launches of a one-CTA kernel (64-element BF16 add) in place of the three stages"}
    del floor_graph
    for m in (1, 8, 64, 256):
        ids = torch.randint(0, wl.VOCAB, (m,), device=device).to(torch.int32)
        _, residual, gamma = wl.add_rmsnorm_inputs_torch(torch, device, m)
        q, k, v, qg, kg, pos, tab = wl.qk_inputs_torch(torch, device, m)
        gu = wl.swiglu_input_torch(torch, device, m)
        codes = torch.empty((m, wl.HIDDEN // 2), dtype=torch.uint8, device=device)
        scales = torch.empty((m, wl.HIDDEN // 16), dtype=torch.uint8, device=device)
        pool = torch.empty((wl.KV_BLOCKS * 16 * 1024,), dtype=torch.bfloat16, device=device)
        mc = torch.empty((m, wl.FFN // 2), dtype=torch.uint8, device=device)
        msc = torch.empty((m, wl.FFN // 16), dtype=torch.uint8, device=device)
        args = axk.make_qk_args(tokens=m, q_heads=64, k_heads=8, head_dim=128, rope_dim=128, flags=axk.QK_FLAG_RING,
                                eps=1e-6, mscale=axk.yarn_mscale(4.0), block_tokens=16, n_layers=1, layer=0,
                                pool_stride=1024, tbl_stride=wl.KV_BLOCKS, n_blocks=wl.KV_BLOCKS, q=q, k=k, q_gamma=qg,
                                k_gamma=kg, inv_freq=inv_freq, positions=pos, block_tables=tab, k_pool=pool,
                                status_word=status)

        stages = {
            # the gather is folded into the first norm of the chain: three launches per chain
            "gather_add_rmsnorm_nvfp4": lambda _i, s=stream: axk.gather_add_rmsnorm_nvfp4(
                local, table, wl.VOCAB, ids, residual, gamma, wl.EPS, m, wl.HIDDEN, 90.0, None, codes, scales, 0, status, s),
            "qk_norm_rope_paged_kv": lambda _i, s=stream: axk.qk_norm_rope_paged(local, args, s),
            "swiglu_nvfp4": lambda _i, s=stream: axk.swiglu_nvfp4(local, gu, m, wl.FFN, 40.0, mc, msc, 0, s),
        }

        def run_chain(_i, s=stream):
            for fn in stages.values():
                fn(_i, s)

        eager_us = timed(run_chain, n=200) * 1e3
        # each stage alone: 24 launches of it in one graph (device-side time per launch; eager launches of kernels
        # this short are bound by the host's launch rate)
        stage_us = {}
        for name, fn in stages.items():
            sg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(sg, stream=stream):
                for _ in range(24):
                    fn(0, torch.cuda.current_stream())
            for _ in range(3):
                sg.replay()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s0.record()
            for _ in range(20):
                sg.replay()
            s1.record()
            torch.cuda.synchronize()
            stage_us[name] = s0.elapsed_time(s1) / (20 * 24) * 1e3
            del sg
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run_chain(0, torch.cuda.current_stream())
        for _ in range(5):
            graph.replay()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(200):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        graph_us = start.elapsed_time(end) / 200 * 1e3
        # eight chains in ONE graph (a model forward is captured whole, as the reference does for its verify cycle): the
        # drain and launch gap between two graph launches, which no programmatic edge spans, is paid once per eight chains
        graph8 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph8, stream=stream):
            for _ in range(8):
                run_chain(0, torch.cuda.current_stream())
        for _ in range(3):
            graph8.replay()
        torch.cuda.synchronize()
        start.record()
        for _ in range(50):
            graph8.replay()
        end.record()
        torch.cuda.synchronize()
        graph8_us = start.elapsed_time(end) / (50 * 8) * 1e3
        del graph8
        algo = m * (wl.HIDDEN * 2 * 2 + (3 * wl.HIDDEN * 2 + wl.HIDDEN // 2 + wl.HIDDEN // 16) +
                    (2 * 64 * 128 * 2 + 2 * 8 * 128 * 2 + 4) + (2 * wl.FFN * 2 + wl.FFN // 2 + wl.FFN // 16)) + wl.HIDDEN * 2
        chain[str(m)] = {"eager_us": eager_us, "graph_us": graph_us, "graph8_us_per_chain": graph8_us,
                         "stage_us": list(stage_us.values()), "bytes": algo,
                         "frac_graph8": algo / (graph8_us * 1e-6) / 1e9 / peak}
        del graph
    return chain


if __name__ == "__main__":
    sys.exit(main())

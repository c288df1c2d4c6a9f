#!/usr/bin/env python
"""Benchmark of the cross-entropy hot path (forward + backward in one sweep) on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A "step" is one pass of the fused cross entropy over one batch of synthetic
logits: valid-row count, fused forward+backward sweep, deterministic loss sum.  With N GPUs the rows of
the configuration are sharded over the ranks (strong scaling: rows / N each) and the two scalars of the
mean are exchanged inside the count and loss kernels.  `value` is rows/s of the whole job with inputs
resident in HBM, timed after a stretch of continuous load (`burst` is the same right after the warm-up);
`e2e` repeats the step with the logits and targets copied from pinned host memory and the loss read back,
inside the timed region; `extras` (N = 1) are the other configurations of the path.  `--impl reference`
times the PyTorch CPU ATen path (the reference's own golden and CPU route) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (rows of the whole job, classes, dtype, ignore fraction, label smoothing)
    "ce_bf16_32768x128256": (32768, 128256, "bfloat16", 0.05, 0.1),   # the headline configuration
    "ce_fp32_4096x32000": (4096, 32000, "float32", 0.0, 0.0),          # the reference's own CPU-runnable case
    "ce_bf16_8192x50257": (8192, 50257, "bfloat16", 0.05, 0.1),        # a vocabulary whose row pitch is not a multiple of 16 bytes
    "ce_fp32_32768x2048": (32768, 2048, "float32", 0.0, 0.0),          # rows of 8 KB: the shared-memory slot ring
}
DEFAULT_WORKLOAD = "ce_bf16_32768x128256"


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs.  Reads through NVML
    in this process (two light queries per sample; a looping nvidia-smi with its power and event queries was seen to
    stall kernel launches for milliseconds); falls back to nvidia-smi when the NVML binding is missing.  Read-only."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_s: float = 0.004):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.proc = None
        self.lines = []
        self.thread = None
        self.samples = []       # (sm_mhz, reasons bitmask) from NVML
        self.sm_max = None
        self._stop = threading.Event()
        self._nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if self.gpu_index < len(ids) and ids[self.gpu_index].isdigit():
                    index = int(ids[self.gpu_index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _poll_nvml(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self._nvml is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            nv = self._nvml
            names = (("hw_slowdown", getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8)),
                     ("hw_thermal_slowdown", getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40)),
                     ("sw_thermal_slowdown", getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20)),
                     ("sw_power_cap", getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)))
            reasons = set()
            for _, mask in self.samples:
                for name, bit in names:
                    if mask & bit:
                        reasons.add(name)
            sm = [m for m, _ in self.samples]
            try:
                nv.nvmlShutdown()
            except Exception:
                pass
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.sm_max, "samples": len(sm),
                    "reasons": sorted(reasons), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def bind_to_gpu_numa_node(gpu_index: int):
    """Runs this rank on the CPUs next to its GPU (NVML's affinity mask, a read-only query), so that the pinned staging
    buffers of the end-to-end leg are first touched, and therefore placed, on the GPU's own NUMA node: with every rank on
    node 0 the host-to-device copies of eight ranks shared one root complex.  Returns the number of CPUs bound to, or None
    when nothing was changed (no NVML, or the mask does not intersect the CPUs this process may use)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        index = gpu_index
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if gpu_index < len(ids) and ids[gpu_index].isdigit():
                index = int(ids[gpu_index])
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        near = {c for c in range(ncpu) if (int(words[c // 64]) >> (c % 64)) & 1}
        allowed = os.sched_getaffinity(0) & near
        pynvml.nvmlShutdown()
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return None


def algorithmic_bytes(rows, classes, elem_size):
    """Read logits + write gradient + read targets, each once."""
    return 2 * rows * classes * elem_size + rows * 8


def moved_bytes(rows, classes, elem_size, ignored_rows):
    """What the fused sweep has to move: rows whose target is ignore_index are never read (their gradient, zeros, is
    still written)."""
    return algorithmic_bytes(rows, classes, elem_size) - ignored_rows * classes * elem_size


# DRAM bytes per row of the dominant kernel: dram__bytes_read.sum + dram__bytes_write.sum of ONE fused-sweep launch, from the
# ncu captures summarised under profiles/ (each file names its command), divided by the rows of the captured launch.  Traffic
# is proportional to the rows, so the figure is scaled by the rows of the timed launch.  Captured on the tree of commit
# 67f1c25; re-capture when cross_entropy_tma.cu or cross_entropy_ring_rows.cu change.
NCU_TRAFFIC_PER_ROW = {
    "ce_fp32_4096x32000": (524.369152e6 + 468.845312e6) / 4096,      # profiles/ce_resident_kernel_fp32_4096x32000.md
    "ce_bf16_32768x128256": (998.445568e6 + 994.885888e6) / 4096,    # profiles/ce_resident_kernel_bf16_4096x128256.md
    "ce_bf16_8192x50257": (782.501888e6 + 769.983744e6) / 8192,      # profiles/ce_resident_kernel_ragged_bf16_8192x50257.md
    "ce_fp32_32768x2048": (268.949760e6 + 213.385216e6) / 32768,     # profiles/ce_ring_rows_kernel_fp32_32768x2048.md
}
KERNEL_NAMES = {0: "ce_rows_cta_kernel (two sweeps)", 1: "ce_resident_kernel (1 CTA per row)", 2: "ce_resident_kernel (2-CTA cluster per row)",
                4: "ce_resident_kernel (4-CTA cluster per row)", 8: "ce_rows_reg_kernel (row in registers)",
                16: "ce_ring_rows_kernel (groups of rows on a shared-memory slot ring, one warp per row)"}


def workload_config(args, world):
    rows_total, classes, dtype_name, ignore_frac, eps = WORKLOADS[args.workload]
    if args.rows:
        rows_total = args.rows
    return {"workload": args.workload, "rows": rows_total, "classes": classes, "ignore_fraction": ignore_frac,
            "label_smoothing": eps, "reduction": "mean", "row_shards": world}


def run_reference(args):
    """The PyTorch CPU ATen path (the reference's test golden and its CPU route) on the host cores, each step a bounded
    row sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import oracle

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rows_full, classes, dtype_name, ignore_frac, eps = WORKLOADS[args.workload]
    dtype = getattr(torch, dtype_name)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_rows = args.cpu_rows or max(64, min(rows_full, int(2.0e9 / (classes * 4)) // 64 * 64))
    times = []
    for _ in range(args.warmup):
        oracle.time_aten_cross_entropy(sample_rows, classes, dtype, ignore_frac, eps, repeats=1, threads=cores, warm=False)
    for _ in range(args.steps):
        t, used = oracle.time_aten_cross_entropy(sample_rows, classes, dtype, ignore_frac, eps, repeats=1, threads=cores,
                                                 warm=False)
        times.append(t)
    sec = sum(times) / len(times)
    value = sample_rows / sec
    line = {
        "impl": "reference", "metric": "cross_entropy_fwd_bwd_rows_per_s", "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": workload_config(args, world),
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"PyTorch CPU ATen F.cross_entropy fwd+bwd on {sample_rows} rows x {classes} {dtype_name} per step"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import torch_supa_b200  # registers the "supa" device; raises if the native libraries are missing
    import bench_extras
    from torch_supa_b200 import capi
    from torch_supa_b200.distributed import LossComm, shard_rows, sharded_cross_entropy

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.supa.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    cpus_bound = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    torch.supa.set_device(local_rank)
    torch.cuda.set_device(local_rank)  # only for the synthetic-data generator
    device = torch.device("supa", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("gloo")  # host-side plumbing: barrier, max over ranks, handle and unique-id store
        comm = LossComm.from_env(device_index=local_rank)
    if args.force_generic:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, 0))
    if args.tune_variant >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, args.tune_variant))
    if args.tune_keep >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(3, args.tune_keep))
    if args.tune_window >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(2, args.tune_window))

    cfg = workload_config(args, world)
    rows_total, classes, eps, ignore_frac = cfg["rows"], cfg["classes"], cfg["label_smoothing"], cfg["ignore_fraction"]
    dtype_name = WORKLOADS[args.workload][2]
    dtype = getattr(torch, dtype_name)
    esize = torch.empty((), dtype=dtype).element_size()
    warmup = max(args.warmup, 3)
    peak, peak_kind = load_peaks()

    def barrier():
        torch.supa.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def make_inputs(rows, seed):
        """Seeded synthetic inputs of one rank: logits N(0,1)*2, targets uniform with a fraction set to ignore_index."""
        x = bench_extras.device_randn((rows, classes), dtype, device, seed=seed, scale=2.0)
        tg = torch.Generator().manual_seed(1000 + seed)
        host_t = torch.randint(0, classes, (rows,), generator=tg)
        if ignore_frac > 0:
            host_t[torch.randperm(rows, generator=torch.Generator().manual_seed(2000 + seed))[: int(rows * ignore_frac)]] = -100
        return x.requires_grad_(True), host_t

    def step(x, t):
        """One pass of the hot path through the public API: loss (global mean) and the logit gradient."""
        x.grad = None
        if comm is not None:
            loss = sharded_cross_entropy(x, t, comm, ignore_index=-100, label_smoothing=eps, reduction="mean")
        else:
            loss = F.cross_entropy(x, t, ignore_index=-100, label_smoothing=eps, reduction="mean")
        loss.backward()
        return loss

    def timed(x, t, steps):
        s0, s1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
        barrier()
        s0.record()
        for _ in range(steps):
            loss = step(x, t)
        s1.record()
        barrier()
        return max_over_ranks(s0.elapsed_time(s1)) / steps, loss

    # ---- the workload: the rows of the configuration, sharded over the ranks (strong scaling) ----
    b, e = shard_rows(rows_total, world, rank)
    rows = e - b
    logits, host_target = make_inputs(rows, seed=rank)
    target = host_target.to(device)
    nbytes = logits.numel() * esize
    ignored_local = int((host_target == -100).sum())

    sampler = ClockSampler(local_rank)
    for _ in range(warmup):
        step(logits, target)
    barrier()
    # a short burst right after the warm-up (the board has not reached its power cap yet) ...
    burst_ms, _ = timed(logits, target, args.steps)
    # ... then the measurement proper, after about half a second of continuous load, which is what a training loop sees:
    # at 1000 W the board caps its power and lowers the SM clock
    if not args.quick:
        for _ in range(20):  # a fixed count: every rank issues the same exchanges
            for _ in range(8):
                step(logits, target)
            torch.supa.synchronize()
    if rank == 0 and not args.no_clocks:
        sampler.start()
    ms_per_step, loss = timed(logits, target, args.steps)
    loss_value = float(loss.float().item())

    # ---- the dominant kernel alone, through the C ABI on the same buffers, same thermal state ----
    grad = torch.empty_like(logits)
    ws_row_loss = torch.empty(rows, dtype=torch.float32, device=device)
    ws_acc = torch.zeros(2, dtype=torch.float64, device=device)
    ws_status = torch.zeros(1, dtype=torch.int32, device=device)
    stream = torch.supa.current_stream_handle(local_rank)
    a = capi.CEArgs()
    a.logits, a.dtype, a.reduction, a.target = logits.data_ptr(), capi.torch_dtype_code(dtype), capi.REDUCTION_MEAN, target.data_ptr()
    a.grad_logits, a.row_loss, a.acc = grad.data_ptr(), ws_row_loss.data_ptr(), ws_acc.data_ptr()
    a.rows, a.classes, a.ignore_index, a.label_smoothing, a.grad_scale = rows, classes, -100, eps, 1.0
    a.status = ws_status.data_ptr()
    capi.ce_count_valid(target, rows, classes, -100, ws_acc, ws_status, stream)
    kernel_times = []
    for _ in range(args.steps):
        e0, e1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
        e0.record()
        capi.ce_forward_backward(a, stream)
        e1.record()
        e1.synchronize()
        kernel_times.append(e0.elapsed_time(e1))
    kernel_ms = statistics.mean(kernel_times)
    status_word = int(ws_status.cpu().item())
    clocks = sampler.stop() if (rank == 0 and not args.no_clocks) else None
    del grad

    # ---- weak scaling beside it (N > 1): every rank holds the whole configuration's row count ----
    weak = None
    if world > 1 and not args.quick:
        del logits, target
        torch.supa.empty_cache()
        wx, wt_host = make_inputs(rows_total, seed=100 + rank)
        wt = wt_host.to(device)
        for _ in range(3):
            step(wx, wt)
        weak_ms, _ = timed(wx, wt, max(3, args.steps // 2))
        weak = {"ms_per_step": weak_ms, "value": rows_total * world / (weak_ms * 1e-3), "unit": "rows/s", "rows_per_gpu": rows_total,
                "scaling": "weak"}
        del wx, wt
        torch.supa.empty_cache()
        logits, host_target = make_inputs(rows, seed=rank)
        target = host_target.to(device)

    # ---- end to end: host buffers -> loss on the host ----
    e2e = None
    if args.quick:
        args.no_cpu_baseline = True
    else:
        try:
            import psutil

            avail = psutil.virtual_memory().available
        except Exception:
            avail = 64 << 30
        budget = int(avail * 0.4 / max(world, 1))
        logits.grad = None
        if nbytes <= budget:
            host_logits = torch.empty(rows, classes, dtype=dtype).pin_memory()
            host_logits.copy_(logits.detach())
            pinned_target = host_target.pin_memory()
            e2e_steps = max(1, min(args.steps, args.e2e_steps))
            del logits
            torch.supa.empty_cache()

            def e2e_step():
                x = host_logits.to(device, non_blocking=True).requires_grad_(True)   # H2D of this step's logits
                t = pinned_target.to(device, non_blocking=True)                        # H2D of this step's targets
                return float(step(x, t).item())                                         # D2H of the loss (synchronises)

            e2e_step()
            barrier()
            t0 = time.perf_counter()
            s0, s1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
            s0.record()
            for _ in range(e2e_steps):
                e2e_loss = e2e_step()
            s1.record()
            barrier()
            e2e_ms = max_over_ranks(s0.elapsed_time(s1)) / e2e_steps
            wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
            e2e = {"value": rows_total / (e2e_ms * 1e-3), "unit": "rows/s", "ms_per_step": e2e_ms, "wall_ms_per_step": wall_ms,
                   "steps": e2e_steps, "h2d_bytes_per_step": rows_total * classes * esize + rows_total * 8, "d2h_bytes_per_step": esize * world,
                   "api": "tensor.to('supa', non_blocking) from pinned memory; " + ("sharded_cross_entropy" if comm is not None else "F.cross_entropy") + "; backward; loss.item()",
                   "loss": e2e_loss}
            del host_logits
        else:
            e2e = {"value": None, "unit": "rows/s", "skipped": "host memory too small for a pinned copy of the logits"}
    torch.supa.empty_cache()

    # ---- CPU baseline (rank 0, N = 1 only) ----
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle

        cores = os.cpu_count() or 1
        sample_rows = args.cpu_rows or max(64, min(rows, int(1.0e9 / (classes * 4)) // 64 * 64))
        sec, used = oracle.time_aten_cross_entropy(sample_rows, classes, dtype, ignore_frac, eps, repeats=2, threads=cores)
        cpu_baseline = {"value": sample_rows / sec, "unit": "rows/s", "cores": used, "kind": "port",
                        "sample": f"PyTorch CPU ATen F.cross_entropy fwd+bwd, best of 2, on {sample_rows} rows x {classes} {dtype_name}"}

    alg = algorithmic_bytes(rows, classes, esize)
    moved = moved_bytes(rows, classes, esize, ignored_local)
    achieved = alg / (kernel_ms * 1e-3) / 1e9
    achieved_moved = moved / (kernel_ms * 1e-3) / 1e9
    variant = capi.ce_kernel_variant(capi.torch_dtype_code(dtype), rows, classes)
    extras = None
    if rank == 0 and world == 1 and args.extras and (not args.quick or args.extras == 2):
        extras = bench_extras.run_extras(device, peak, profile=args.extras == 2)
    # my kernels per step: count, fused sweep, loss sum + finish (the two exchanges ride inside the count and the loss kernel),
    # fill of the root gradient (by autograd), rescale; through NCCL the loss sum and its finish are two launches
    launches_per_step = 5 if (comm is None or comm.peer_handle) else 6

    if rank == 0:
        traffic_per_row = NCU_TRAFFIC_PER_ROW.get(args.workload)
        line = {
            "metric": "cross_entropy_fwd_bwd_rows_per_s", "value": rows_total / (ms_per_step * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": cfg,
            "notes": {"rows_per_gpu": rows, "timed_after": "warm-up" if args.quick else "warm-up + 160 steps of continuous load (power-capped clocks)",
                      "api": "F.cross_entropy on the supa device + backward" if world == 1 else "sharded_cross_entropy + backward",
                      "exchange": None if comm is None else ("peer memory inside the count and loss kernels" if comm.peer_handle else "ncclAllReduce x2"),
                      "l2": "inputs larger than L2 (no flush)" if nbytes > (256 << 20) else "inputs smaller than 2x L2",
                      "cpus_bound_near_gpu": cpus_bound},
            "loss": loss_value, "status_word": status_word, "kernel_variant": variant,
            "burst": {"ms_per_step": burst_ms, "value": rows_total / (burst_ms * 1e-3), "unit": "rows/s",
                      "note": f"{args.steps} steps right after the warm-up, before the power cap lowers the clock"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs_nominal": achieved / 8000.0, "kernel": KERNEL_NAMES.get(variant, str(variant)),
                         "kernel_ms": kernel_ms, "algorithmic_bytes": alg,
                         "moved_bytes": moved, "achieved_moved": achieved_moved, "frac_moved": achieved_moved / peak,
                         "moved_note": "bytes the kernel has to move: rows whose target is ignore_index are not read",
                         "traffic": None if traffic_per_row is None else traffic_per_row * rows},
            "hbm_gbs_whole_step": alg / (ms_per_step * 1e-3) / 1e9, "weak": weak,
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if extras is not None:
            line["extras"] = extras
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the total row count (small profiling captures)")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU-baseline sample")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="profiling mode: no load loop, no weak-scaling leg, no e2e, no CPU baseline, no extras")
    ap.add_argument("--force-generic", action="store_true", help="tuning: always use the generic two-sweep kernel")
    ap.add_argument("--no-clocks", action="store_true", help="diagnostic: do not sample clocks during the run")
    ap.add_argument("--tune-variant", type=int, default=-1, help="tuning: force the resident kernel's cluster size (1, 2, 4)")
    ap.add_argument("--tune-keep", type=int, default=-1, help="tuning: 0 recompute bf16 exponentials in the gradient sweep, 1 keep them")
    ap.add_argument("--tune-window", type=int, default=-1, help="tuning: next-row chunks folded during the statistics exchange")
    ap.add_argument("--extras", type=int, default=1,
                    help="1 (default, N = 1): also time the other configurations (elementwise, reductions, log_softmax ...); 0: skip them; "
                         "2: one launch each (for profilers)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the cross-entropy hot path (forward + backward in one sweep) on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A "step" is one pass of the fused cross entropy over one batch of synthetic
logits: valid-row count, fused forward+backward sweep, deterministic loss sum (with the two scalar
all-reduces between them when rows are sharded over several GPUs).  `value` is rows/s over all ranks
with inputs resident in HBM; `e2e` repeats the step with the logits and targets copied from pinned
host memory and the loss read back, inside the timed region.  `--impl reference` times the PyTorch
CPU ATen path (the reference's own golden and CPU route) on the host cores for the same workload.
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
    # name: (rows per GPU, classes, dtype, ignore fraction, label smoothing)
    "ce_bf16_32768x128256": (32768, 128256, "bfloat16", 0.05, 0.1),   # BASELINE.json configs[4]
    "ce_fp32_4096x32000": (4096, 32000, "float32", 0.0, 0.0),          # BASELINE.json configs[0]
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
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
                "samples": len(sm), "reasons": sorted(reasons)}


def algorithmic_bytes(rows, classes, elem_size):
    """Read logits + write gradient + read targets, each once."""
    return 2 * rows * classes * elem_size + rows * 8


def make_inputs(torch, rows, classes, dtype, ignore_frac, device, seed):
    """Seeded synthetic logits N(0,1)*2 and uniform targets with a fraction set to ignore_index=-100."""
    g = torch.Generator(device=device).manual_seed(seed)
    logits = torch.empty(rows, classes, dtype=dtype, device=device)
    block = max(1, (1 << 28) // classes)
    for r0 in range(0, rows, block):
        r1 = min(rows, r0 + block)
        logits[r0:r1] = (torch.randn(r1 - r0, classes, device=device, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), device=device, generator=g)
    if ignore_frac > 0:
        n_ign = int(rows * ignore_frac)
        perm = torch.randperm(rows, device=device, generator=torch.Generator(device=device).manual_seed(seed + 1))
        target[perm[:n_ign]] = -100
    return logits, target


def run_reference(args):
    """The PyTorch CPU ATen path on the host cores, bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import oracle

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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": {"workload": args.workload, "rows_per_gpu": rows_full, "classes": classes,
                   "ignore_fraction": ignore_frac, "label_smoothing": eps, "reduction": "mean"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"PyTorch CPU ATen F.cross_entropy fwd+bwd on {sample_rows} rows x {classes} {dtype_name}"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from torch_supa_b200 import capi, functional as F2

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    capi.lib()  # fail loudly if the kernel library is missing
    if args.force_generic:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, 0))

    rows, classes, dtype_name, ignore_frac, eps = WORKLOADS[args.workload]
    if args.rows:
        rows = args.rows
    dtype = getattr(torch, dtype_name)
    esize = torch.empty((), dtype=dtype).element_size()
    logits, target = make_inputs(torch, rows, classes, dtype, ignore_frac, device, seed=rank)
    grad = torch.empty_like(logits)
    ws = F2.CrossEntropyWorkspace(rows, device)
    all_reduce = (lambda view: dist.all_reduce(view)) if world > 1 else None
    launches_per_step = 3  # count_valid, fused sweep, loss sum+finish (the all-reduces are NCCL's)
    if world > 1:
        launches_per_step = 4  # loss sum and finish are separate launches around the all-reduce

    def step():
        return F2.cross_entropy_forward_backward(logits, target, ignore_index=-100, label_smoothing=eps, reduction="mean",
                                                 grad=grad, workspace=ws, all_reduce=all_reduce)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # keep the GPU busy long enough for the clock sampler to see it under load
    t_end = time.time() + (0.0 if args.quick else 0.6)
    while time.time() < t_end:
        step()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------------------
    kernel_events = []
    stream = torch.cuda.current_stream()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fused_args = None
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        loss, _ = step()
    stop.record(stream)
    barrier()
    elapsed_ms = start.elapsed_time(stop)

    # dominant kernel alone (same launches, events around the fused sweep only)
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        capi.ce_count_valid(target, rows, classes, -100, ws.acc, ws.status, stream.cuda_stream)
        a = capi.CEArgs()
        a.logits, a.dtype, a.reduction, a.target = logits.data_ptr(), capi.torch_dtype_code(dtype), capi.REDUCTION_MEAN, target.data_ptr()
        a.grad_logits, a.row_loss, a.acc = grad.data_ptr(), ws.row_loss.data_ptr(), ws.acc.data_ptr()
        a.rows, a.classes, a.ignore_index, a.label_smoothing, a.grad_scale = rows, classes, -100, eps, 1.0
        a.status = ws.status.data_ptr()
        e0.record(stream)
        capi.ce_forward_backward(a, stream.cuda_stream)
        e1.record(stream)
        kernel_events.append((e0, e1))
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    kernel_ms = statistics.mean(e0.elapsed_time(e1) for e0, e1 in kernel_events)

    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    total_rows = rows * world
    value = total_rows / (ms_per_step * 1e-3)
    loss_value = float(loss.float().item())
    status_word = int(ws.status.item())

    # ---- end to end: host buffers -> loss on the host ---------------------------------------------
    e2e = None
    nbytes = logits.numel() * esize
    if args.quick:
        args.no_cpu_baseline = True
    else:
        try:
            import psutil

            avail = psutil.virtual_memory().available
        except Exception:
            avail = 64 << 30
        budget = int(avail * 0.4 / max(world, 1))
        pinned_rows = rows if nbytes <= budget else max(1, int(budget // (classes * esize)))
        host_logits = torch.empty(pinned_rows, classes, dtype=dtype).pin_memory()
        host_logits.copy_(logits[:pinned_rows])
        host_target = target.cpu().pin_memory()
        host_loss = torch.empty((), dtype=dtype).pin_memory()
        e2e_steps = max(1, min(args.steps, args.e2e_steps))

        def e2e_step():
            for r0 in range(0, rows, pinned_rows):
                r1 = min(rows, r0 + pinned_rows)
                logits[r0:r1].copy_(host_logits[: r1 - r0], non_blocking=True)
            target.copy_(host_target, non_blocking=True)
            l, _ = step()
            host_loss.copy_(l, non_blocking=True)

        e2e_step()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        s1.record(stream)
        barrier()
        t = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / e2e_steps
        e2e = {"value": total_rows / (e2e_ms * 1e-3), "unit": "rows/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
               "h2d_bytes_per_step": (nbytes + rows * 8) * world, "d2h_bytes_per_step": esize * world,
               "pinned_rows": pinned_rows}
        del host_logits

    # ---- CPU baseline (rank 0, N = 1 only) --------------------------------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle

        cores = os.cpu_count() or 1
        sample_rows = args.cpu_rows or max(64, min(rows, int(1.0e9 / (classes * 4)) // 64 * 64))
        sec, used = oracle.time_aten_cross_entropy(sample_rows, classes, dtype, ignore_frac, eps, repeats=2, threads=cores)
        cpu_baseline = {"value": sample_rows / sec, "unit": "rows/s", "cores": used, "kind": "port",
                        "sample": f"PyTorch CPU ATen F.cross_entropy fwd+bwd, best of 2, on {sample_rows} rows x {classes} {dtype_name}"}

    peak, peak_kind = load_peaks()
    alg = algorithmic_bytes(rows, classes, esize)
    achieved = alg / (kernel_ms * 1e-3) / 1e9
    extras = None
    if rank == 0 and world == 1 and args.extras:
        del logits, grad
        torch.cuda.empty_cache()
        from torch_supa_b200 import benchmarks

        extras = benchmarks.run_extras(device, peak)

    if rank == 0:
        line = {
            "metric": "cross_entropy_fwd_bwd_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": args.workload, "rows_per_gpu": rows, "classes": classes, "ignore_fraction": ignore_frac,
                       "label_smoothing": eps, "reduction": "mean", "parallelism": f"rows sharded x{world}",
                       "l2": "inputs larger than L2 (no flush)" if nbytes > (256 << 20) else "inputs rotate below L2 size"},
            "loss": loss_value, "status_word": status_word,
            "kernel_variant": capi.ce_kernel_variant(capi.torch_dtype_code(dtype), rows, classes),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs_nominal": achieved / 8000.0, "kernel_ms": kernel_ms,
                         "algorithmic_bytes": alg, "traffic": None},
            "hbm_gbs_whole_step": alg * world / (ms_per_step * 1e-3) / 1e9,
            "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if extras is not None:
            line["extras"] = extras
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override rows per GPU (small profiling captures)")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU-baseline sample")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="profiling mode: no clock warm loop, no e2e, no CPU baseline")
    ap.add_argument("--force-generic", action="store_true", help="tuning: always use the generic two-sweep kernel")
    ap.add_argument("--extras", type=int, default=0, help="1: also time the elementwise / reduction configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

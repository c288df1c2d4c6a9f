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
    "ce_bf16_32768x128256": (32768, 128256, "bfloat16", 0.05, 0.1),   # the headline configuration
    "ce_fp32_4096x32000": (4096, 32000, "float32", 0.0, 0.0),          # the reference's own CPU-runnable case
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


def algorithmic_bytes(rows, classes, elem_size):
    """Read logits + write gradient + read targets, each once."""
    return 2 * rows * classes * elem_size + rows * 8


# dram__bytes_read.sum + dram__bytes_write.sum of one fused-sweep launch from the ncu captures summarised under
# profiles/ (the bf16 figure is the 4096-row capture scaled by 8: traffic is proportional to rows).
TRAFFIC = {
    ("ce_fp32_4096x32000", 4096): 524.488192e6 + 469.110272e6,
    ("ce_bf16_32768x128256", 32768): 8 * (998.447616e6 + 995.276288e6),
}


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
    import torch.nn.functional as F

    import torch_supa_b200  # registers the "supa" device; raises if the native libraries are missing
    from torch_supa_b200 import benchmarks, capi
    from torch_supa_b200.distributed import LossComm, sharded_cross_entropy

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.supa.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.supa.set_device(local_rank)
    torch.cuda.set_device(local_rank)  # only for the synthetic-data generator
    device = torch.device("supa", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("gloo")  # host-side plumbing: barrier, max over ranks, unique-id store
        comm = LossComm.from_env(device_index=local_rank)
    if args.force_generic:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, 0))
    if args.tune_variant >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, args.tune_variant))
    if args.tune_keep >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(3, args.tune_keep))
    if args.tune_window >= 0:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(2, args.tune_window))

    rows, classes, dtype_name, ignore_frac, eps = WORKLOADS[args.workload]
    if args.rows:
        rows = args.rows
    dtype = getattr(torch, dtype_name)
    esize = torch.empty((), dtype=dtype).element_size()
    # seeded synthetic inputs: logits N(0,1)*2, targets uniform with a fraction set to ignore_index
    logits = benchmarks.device_randn((rows, classes), dtype, device, seed=rank, scale=2.0)
    tg = torch.Generator().manual_seed(1000 + rank)
    host_target = torch.randint(0, classes, (rows,), generator=tg)
    if ignore_frac > 0:
        host_target[torch.randperm(rows, generator=torch.Generator().manual_seed(2000 + rank))[: int(rows * ignore_frac)]] = -100
    target = host_target.to(device)
    logits.requires_grad_(True)
    nbytes = logits.numel() * esize
    warmup = max(args.warmup, 3)

    def step(x, t):
        """One pass of the hot path through the public API: loss (global mean) and the logit gradient."""
        x.grad = None
        if comm is not None:
            loss = sharded_cross_entropy(x, t, comm, ignore_index=-100, label_smoothing=eps, reduction="mean")
        else:
            loss = F.cross_entropy(x, t, ignore_index=-100, label_smoothing=eps, reduction="mean")
        loss.backward()
        return loss

    # my kernels per step: count_valid, fused sweep, loss sum(+finish), fill(root gradient, by autograd), rescale;
    # with N > 1 the loss sum and finish are two launches
    launches_per_step = 5 if world == 1 else 6

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

    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.no_clocks:
        sampler.start()
    for _ in range(warmup):
        step(logits, target)
    barrier()

    # ---- device-resident timing ---------------------------------------------------------------------
    start, stop = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        loss = step(logits, target)
    stop.record()
    barrier()
    ms_per_step = max_over_ranks(start.elapsed_time(stop)) / args.steps
    loss_value = float(loss.float().item())

    # ---- the dominant kernel alone, through the C ABI on the same buffers ------------------------------
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
    clocks = sampler.stop() if rank == 0 else None
    del grad

    # ---- the same step under sustained load: about half a second of back-to-back steps, the last ones timed.  At
    # 1000 W the board caps its power and lowers the SM clock, so this is slower than the short timed region above.
    sustained = None
    if not args.quick:
        sus_sampler = ClockSampler(local_rank, period_s=0.02)
        if rank == 0 and not args.no_clocks:
            sus_sampler.start()
        for _ in range(20):  # a fixed count: every rank must issue the same collectives
            for _ in range(8):
                step(logits, target)
            torch.supa.synchronize()
        s0, s1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
        barrier()
        s0.record()
        for _ in range(20):
            step(logits, target)
        s1.record()
        barrier()
        sus_ms = max_over_ranks(s0.elapsed_time(s1)) / 20
        sus_clocks = sus_sampler.stop() if (rank == 0 and not args.no_clocks) else None
        sustained = {"ms_per_step": sus_ms, "value": rows * world / (sus_ms * 1e-3), "unit": "rows/s", "after_steps_of_load": 160,
                     "clocks": sus_clocks}

    # ---- end to end: host buffers -> loss on the host ---------------------------------------------
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
            e2e = {"value": rows * world / (e2e_ms * 1e-3), "unit": "rows/s", "ms_per_step": e2e_ms, "wall_ms_per_step": wall_ms,
                   "steps": e2e_steps, "h2d_bytes_per_step": (nbytes + rows * 8) * world, "d2h_bytes_per_step": esize * world,
                   "api": "tensor.to('supa', non_blocking) from pinned memory; " + ("sharded_cross_entropy" if comm is not None else "F.cross_entropy") + "; backward; loss.item()",
                   "loss": e2e_loss}
            del host_logits
        else:
            e2e = {"value": None, "unit": "rows/s", "skipped": "host memory too small for a pinned copy of the logits"}
    torch.supa.empty_cache()

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
        extras = benchmarks.run_extras(device, peak, quick=args.quick, profile=args.extras == 2)

    if rank == 0:
        line = {
            "metric": "cross_entropy_fwd_bwd_rows_per_s", "value": rows * world / (ms_per_step * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": args.workload, "rows_per_gpu": rows, "classes": classes, "ignore_fraction": ignore_frac,
                       "label_smoothing": eps, "reduction": "mean", "parallelism": f"rows sharded x{world}",
                       "api": "F.cross_entropy on the supa device + backward" if world == 1 else "sharded_cross_entropy + backward",
                       "l2": "inputs larger than L2 (no flush)" if nbytes > (256 << 20) else "inputs smaller than 2x L2"},
            "loss": loss_value, "status_word": status_word,
            "kernel_variant": capi.ce_kernel_variant(capi.torch_dtype_code(dtype), rows, classes),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs_nominal": achieved / 8000.0, "kernel": "ce_resident_kernel",
                         "kernel_ms": kernel_ms, "algorithmic_bytes": alg, "traffic": TRAFFIC.get((args.workload, rows))},
            "hbm_gbs_whole_step": alg / (ms_per_step * 1e-3) / 1e9, "sustained": sustained,
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
    ap.add_argument("--no-clocks", action="store_true", help="diagnostic: do not sample clocks during the run")
    ap.add_argument("--tune-variant", type=int, default=-1, help="tuning: force the resident kernel's cluster size (1, 2, 4)")
    ap.add_argument("--tune-keep", type=int, default=-1, help="tuning: 0 recompute bf16 exponentials in the gradient sweep, 1 keep them")
    ap.add_argument("--tune-window", type=int, default=-1, help="tuning: next-row chunks folded during the statistics exchange")
    ap.add_argument("--extras", type=int, default=0, help="1: also time the elementwise / reduction configurations; 2: same, one launch each (for profilers)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

"""Timing helpers and the secondary benchmark configurations (elementwise, reductions, log_softmax) through
the ``supa`` operator API.  ``bench.py`` prints their results under ``extras``; the headline line is the
cross-entropy workload."""
from __future__ import annotations

import statistics

import torch
import torch.nn.functional as F


def device_randn(shape, dtype, device, seed, scale=1.0, low=None, high=None, uniform=False):
    """Seeded synthetic tensor on the supa device.  The random bits come from torch's CUDA generator (plumbing)
    and are handed over with a device-to-device copy; integer dtypes draw uniformly from [low, high], ``uniform``
    draws floats from [0, scale)."""
    from torch_supa_b200 import supa as supa_mod

    cuda = torch.device("cuda", device.index or 0)
    g = torch.Generator(device=cuda).manual_seed(seed)
    out = torch.empty(shape, dtype=dtype, device=device)
    flat_n = out.numel()
    block = 1 << 27
    esize = out.element_size()
    for i0 in range(0, flat_n, block):
        n = min(block, flat_n - i0)
        if dtype.is_floating_point:
            draw = torch.rand if uniform else torch.randn
            chunk = (draw(n, device=cuda, generator=g) * scale).to(dtype)
        else:
            chunk = torch.randint(low, high + 1, (n,), device=cuda, generator=g).to(dtype)
        torch.cuda.current_stream(cuda).synchronize()
        supa_mod.memcpy_async(out.data_ptr() + i0 * esize, chunk.data_ptr(), n * esize, device)
        supa_mod.synchronize(device)
    return out


def time_op(calls, warmup=3, samples=20, reps=4):
    """Milliseconds per call, as (median, min, max) over ``samples`` event-timed samples on the current supa stream.
    ``calls`` is one callable or a list of callables that do the same work on different buffer sets; they are used in
    rotation so that a working set smaller than the L2 cannot stay resident between two calls.  Each sample brackets
    ``reps`` back-to-back calls with one event pair, so that the device queue stays full and the host's dispatch time
    between an event and the launch that follows it is not counted as kernel time."""
    if callable(calls):
        calls = [calls]
    k = 0
    for _ in range(warmup):
        for fn in calls:
            fn()
    torch.supa.synchronize()
    times = []
    for _ in range(samples):
        e0, e1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
        e0.record()
        for _ in range(reps):
            calls[k % len(calls)]()
            k += 1
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return statistics.median(times), min(times), max(times)


def time_cpu(fn, repeats=2):
    """Best-of seconds of ``fn()`` on the host cores after one warm-up call."""
    import time

    fn()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def run_extras(device, peak_gbs, profile=False):
    """Times the configurations beside the headline workload at their full sizes and returns a list of
    {name, ms (median), ms_min, ms_max, algorithmic_bytes, gbs, frac_of_measured, buffer_sets, cpu_gbs, cpu_sample}.
    Bytes follow one rule: every distinct input element read once, every output element written once.  The CPU figure is
    the same operator of PyTorch's CPU backend on all host cores, on a bounded sample (a fraction of the rows), as GB/s
    of the sample's algorithmic bytes."""
    import os

    out = []
    torch.set_num_threads(os.cpu_count() or 1)
    samples, reps, warm = (1, 1, 1) if profile else (20, 4, 3)

    def entry(name, nbytes, calls, cpu=None, cpu_fraction=1.0, cpu_sample=""):
        med, lo, hi = time_op(calls, warmup=warm, samples=samples, reps=reps)
        gbs = nbytes / (med * 1e-3) / 1e9
        e = {"name": name, "ms": round(med, 4), "ms_min": round(lo, 4), "ms_max": round(hi, 4), "algorithmic_bytes": nbytes,
             "gbs": round(gbs, 1), "frac_of_measured": round(gbs / peak_gbs, 3), "frac_of_8TBs": round(gbs / 8000.0, 3),
             "buffer_sets": len(calls) if isinstance(calls, list) else 1}
        if cpu is not None and not profile:
            sec = time_cpu(cpu)
            e["cpu_gbs"] = round(nbytes * cpu_fraction / sec / 1e9, 2)
            e["cpu_sample"] = cpu_sample
        out.append(e)

    def cpu_like(t, rows):
        """The first ``rows`` rows of a supa tensor on the host (the CPU leg's bounded sample)."""
        return t[:rows].cpu()

    # ---- cross entropy through autograd: fp32 [4096, 32000] on three rotating buffer sets (1 GB each) ----
    def ce_call(x, t, **kw):
        def call():
            x.grad = None
            F.cross_entropy(x, t, **kw).backward()
        return call

    sets = []
    for i in range(3):
        x = device_randn((4096, 32000), torch.float32, device, 20 + i, 2.0).requires_grad_(True)
        t = device_randn((4096,), torch.int64, device, 30 + i, low=0, high=31999)
        sets.append((x, t))
    cx = cpu_like(sets[0][0].detach(), 1024).requires_grad_(True)
    ct = sets[0][1][:1024].cpu()
    entry("cross_entropy fwd+bwd fp32 [4096,32000] (operator API, autograd)", 2 * 4096 * 32000 * 4 + 4096 * 8,
          [ce_call(x, t) for x, t in sets], cpu=ce_call(cx, ct), cpu_fraction=0.25, cpu_sample="1024 of 4096 rows")
    del sets, cx, ct
    torch.supa.empty_cache()

    # ---- cross entropy with class-probability targets (logits and targets read, gradient written) ----
    x = device_randn((4096, 32000), torch.float32, device, 48, 2.0).requires_grad_(True)
    q = torch.softmax(device_randn((4096, 32000), torch.float32, device, 49, 2.0), -1)
    entry("cross_entropy fwd+bwd fp32 [4096,32000], probability targets (2 reads + 1 write; two sweeps, second from L2)", 3 * 4096 * 32000 * 4,
          ce_call(x, q))
    del x, q
    torch.supa.empty_cache()

    # ---- cross entropy on row shapes outside the benchmark's: a vocabulary whose pitch is not a multiple of 16 bytes, short rows ----
    x = device_randn((8192, 50257), torch.bfloat16, device, 40, 2.0).requires_grad_(True)
    t = device_randn((8192,), torch.int64, device, 41, low=0, high=50256)
    entry("cross_entropy fwd+bwd bf16 [8192,50257] (row pitch 100514 B)", 2 * 8192 * 50257 * 2 + 8192 * 8, ce_call(x, t, label_smoothing=0.1))
    del x, t
    x = device_randn((32768, 2048), torch.float32, device, 42, 2.0).requires_grad_(True)
    t = device_randn((32768,), torch.int64, device, 43, low=0, high=2047)
    x2 = device_randn((32768, 2048), torch.float32, device, 44, 2.0).requires_grad_(True)
    entry("cross_entropy fwd+bwd fp32 [32768,2048] (8 KB rows: slot ring, one warp per row)", 2 * 32768 * 2048 * 4 + 32768 * 8, [ce_call(x, t), ce_call(x2, t)])
    del x, t, x2
    x = device_randn((131072, 1000), torch.bfloat16, device, 45, 2.0).requires_grad_(True)
    t = device_randn((131072,), torch.int64, device, 46, low=0, high=999)
    x2 = device_randn((131072, 1000), torch.bfloat16, device, 47, 2.0).requires_grad_(True)
    entry("cross_entropy fwd+bwd bf16 [131072,1000] (2000 B rows: slot ring, four rows per bulk copy)", 2 * 131072 * 1000 * 2 + 131072 * 8,
          [ce_call(x, t, label_smoothing=0.1), ce_call(x2, t, label_smoothing=0.1)])
    del x, t, x2
    torch.supa.empty_cache()

    # ---- SwiGLU chain bf16 ----
    rows, half = 16384, 11008
    xx = device_randn((rows, 2 * half), torch.bfloat16, device, 2)
    a, b = xx[:, :half], xx[:, half:]
    g = device_randn((rows, half), torch.bfloat16, device, 3)
    u = device_randn((rows, half), torch.bfloat16, device, 4)
    n = rows * half * 2
    s = F.silu(a)
    sub = 2048
    cxx, cg, cu = cpu_like(xx, sub), cpu_like(g, sub), cpu_like(u, sub)
    ca, cb = cxx[:, :half], cxx[:, half:]
    cs = F.silu(ca)
    frac, what = sub / rows, f"{sub} of {rows} rows"
    entry("silu(a) bf16, a = strided half of [16384,22016]", 2 * n, lambda: F.silu(a), lambda: F.silu(ca), frac, what)
    entry("silu(a) * b bf16 (mul, b strided half)", 3 * n, lambda: s * b, lambda: cs * cb, frac, what)
    entry("glu(x) bf16 [16384,22016] (fused a * sigmoid(b))", 3 * n, lambda: F.glu(xx, -1), lambda: F.glu(cxx, -1), frac, what)
    entry("silu_backward bf16", 3 * n, lambda: torch.ops.aten.silu_backward(g, a), lambda: torch.ops.aten.silu_backward(cg, ca), frac, what)
    entry("gelu(tanh) bf16 [16384,11008]", 2 * n, lambda: F.gelu(u, approximate="tanh"), lambda: F.gelu(cu, approximate="tanh"), frac, what)
    entry("gelu_backward(tanh) bf16", 3 * n, lambda: torch.ops.aten.gelu_backward(g, u, approximate="tanh"),
          lambda: torch.ops.aten.gelu_backward(cg, cu, approximate="tanh"), frac, what)
    entry("gelu(erf) bf16 [16384,11008]", 2 * n, lambda: F.gelu(u), lambda: F.gelu(cu), frac, what)
    del xx, a, b, g, u, s, cxx, cg, cu, ca, cb, cs
    torch.supa.empty_cache()

    # ---- broadcast / strided / promoting binary ops ----
    p = device_randn((64, 1, 4096), torch.float16, device, 5)
    q = device_randn((1, 2048, 4096), torch.float16, device, 6)
    cp, cq = p[:8].cpu(), q.cpu()
    entry("add fp16 [64,1,4096] + [1,2048,4096]", 64 * 2048 * 4096 * 2 + 64 * 4096 * 2 + 2048 * 4096 * 2, lambda: p + q,
          lambda: cp + cq, 8 / 64, "8 of 64 outer slices")
    w = torch.empty((64, 2048, 4096), dtype=torch.float16, device=device)
    entry("fill_ fp16 [64,2048,4096] (write only)", 64 * 2048 * 4096 * 2, lambda: w.fill_(1.0))
    del p, q, w, cp, cq
    torch.supa.empty_cache()
    msets = []
    for i in range(3):  # 0.4 GB per set: three sets in rotation, more than twice the L2 together
        m = device_randn((8192, 4096), torch.float32, device, 50 + i).t()
        nn_ = device_randn((4096, 8192), torch.float32, device, 60 + i)
        msets.append((m, nn_))
    cm, cn = msets[0][0].cpu(), msets[0][1].cpu()
    entry("mul fp32 transposed view [4096,8192] * contiguous (m.t() * n)", 3 * 4096 * 8192 * 4,
          [(lambda m=m, k=k: m * k) for m, k in msets], lambda: cm * cn, 1.0, "full size")
    entry("mul fp32 contiguous * transposed view (n * m.t())", 3 * 4096 * 8192 * 4,
          [(lambda m=m, k=k: k * m) for m, k in msets], lambda: cn * cm, 1.0, "full size")
    del msets, cm, cn
    torch.supa.empty_cache()
    i32 = device_randn((8192, 8192), torch.int32, device, 9, low=-1000, high=1000)
    f32 = device_randn((8192, 8192), torch.float32, device, 10)
    ci, cf = cpu_like(i32, 2048), cpu_like(f32, 2048)
    entry("add int32 + fp32 [8192,8192] -> fp32", 3 * 8192 * 8192 * 4, lambda: i32 + f32, lambda: ci + cf, 0.25, "2048 of 8192 rows")
    del i32, f32, ci, cf
    torch.supa.empty_cache()

    # ---- row reductions and log_softmax ----
    r = device_randn((8192, 65536), torch.bfloat16, device, 11)
    cr = cpu_like(r, 1024)
    nb = 8192 * 65536 * 2 + 8192 * 2
    what = "1024 of 8192 rows"
    entry("sum(-1) bf16 [8192,65536]", nb, lambda: r.sum(-1), lambda: cr.sum(-1), 0.125, what)
    entry("mean(-1) bf16 [8192,65536]", nb, lambda: r.mean(-1), lambda: cr.mean(-1), 0.125, what)
    entry("amax(-1) bf16 [8192,65536]", nb, lambda: r.amax(-1), lambda: cr.amax(-1), 0.125, what)
    entry("sum(-1, dtype=float32) bf16 [8192,65536]", nb + 8192 * 2, lambda: r.sum(-1, dtype=torch.float32),
          lambda: cr.sum(-1, dtype=torch.float32), 0.125, what)
    del r, cr
    torch.supa.empty_cache()
    # short rows (lane groups share a row) and column sums (rows cut into chunks over the grid)
    tall = device_randn((4194304, 64), torch.float32, device, 21)
    nb = 4194304 * 64 * 4
    entry("sum(-1) fp32 [4194304,64]", nb + 4194304 * 4, lambda: tall.sum(-1))
    entry("amax(-1) fp32 [4194304,64]", nb + 4194304 * 4, lambda: tall.amax(-1))
    entry("sum(0) fp32 [4194304,64]", nb, lambda: tall.sum(0))
    entry("argmax(-1) fp32 [4194304,64] (value and index state per lane group)", nb + 4194304 * 8, lambda: tall.argmax(-1))
    entry("var(0) fp32 [4194304,64] (fp64 state, columns in chunks)", nb, lambda: tall.var(0))
    del tall
    torch.supa.empty_cache()
    mid = device_randn((524288, 1024), torch.bfloat16, device, 22)
    nb = 524288 * 1024 * 2
    entry("sum(-1) bf16 [524288,1024]", nb + 524288 * 2, lambda: mid.sum(-1))
    entry("sum(0) bf16 [524288,1024]", nb, lambda: mid.sum(0))
    del mid
    torch.supa.empty_cache()
    wide = device_randn((8192, 32000), torch.float32, device, 23)
    nb = 8192 * 32000 * 4
    entry("argmax(-1) fp32 [8192,32000]", nb + 8192 * 8, lambda: wide.argmax(-1))
    entry("var(-1) fp32 [8192,32000]", nb + 8192 * 4, lambda: wide.var(-1))
    del wide
    torch.supa.empty_cache()
    ls_rows = 16384 if profile else 65536
    sm = device_randn((ls_rows, 32000), torch.float32, device, 12, 3.0)
    csm = cpu_like(sm, 2048)
    samples_keep, reps_keep = samples, reps
    samples, reps = (samples, reps) if profile else (20, 1)  # 2.6 ms per call: one call per sample
    entry(f"log_softmax(-1) fp32 [{ls_rows},32000]", 2 * ls_rows * 32000 * 4, lambda: F.log_softmax(sm, -1), lambda: F.log_softmax(csm, -1),
          2048 / ls_rows, f"2048 of {ls_rows} rows")
    entry(f"softmax(-1) fp32 [{ls_rows},32000]", 2 * ls_rows * 32000 * 4, lambda: F.softmax(sm, -1))
    del sm, csm
    torch.supa.empty_cache()
    bw_rows = 16384
    y = F.log_softmax(device_randn((bw_rows, 32000), torch.float32, device, 12, 3.0), -1)
    go = device_randn((bw_rows, 32000), torch.float32, device, 18)
    entry(f"log_softmax backward fp32 [{bw_rows},32000] (2 reads, 1 write)", 3 * bw_rows * 32000 * 4,
          lambda: torch.ops.aten._log_softmax_backward_data(go, y, -1, torch.float32))
    del y, go
    samples, reps = samples_keep, reps_keep
    torch.supa.empty_cache()

    # ---- nll_loss2d on a segmentation-shaped input ----
    n4, c4, h4, w4 = 8, 19, 1024, 2048
    logp = device_randn((n4, c4, h4, w4), torch.float32, device, 13)
    t4 = device_randn((n4, h4, w4), torch.int64, device, 14, low=0, high=c4 - 1)
    npx = n4 * h4 * w4
    entry("nll_loss2d forward (mean) fp32 [8,19,1024,2048]: one gathered element + target per sample", npx * (4 + 8), lambda: F.nll_loss(logp, t4))
    go = device_randn((), torch.float32, device, 15)
    tw = torch.ones((), dtype=torch.float32, device=device)
    entry("nll_loss2d backward (mean) fp32 [8,19,1024,2048]: gradient written once + targets", npx * c4 * 4 + npx * 8,
          lambda: torch.ops.aten.nll_loss2d_backward(go, logp, t4, None, 1, -100, tw))
    del logp, t4
    torch.supa.empty_cache()

    # ---- binary_cross_entropy_with_logits, fp32 [8192,8192] ----
    bx = device_randn((8192, 8192), torch.float32, device, 16, 3.0).requires_grad_(True)
    bt = device_randn((8192, 8192), torch.float32, device, 17, uniform=True)
    nb2 = 8192 * 8192 * 4
    entry("binary_cross_entropy_with_logits mean fp32 [8192,8192] (fused loss + reduction: 2 reads)", 2 * nb2,
          lambda: F.binary_cross_entropy_with_logits(bx.detach(), bt))

    def bce_step():
        bx.grad = None
        F.binary_cross_entropy_with_logits(bx, bt).backward()

    entry("binary_cross_entropy_with_logits mean fwd+bwd fp32 [8192,8192] (2 reads + 2 reads, 1 write)", 5 * nb2, bce_step)
    del bx, bt
    torch.supa.empty_cache()

    # ---- random fills and dropout from the device generator (Philox4x32-10: bound by the integer multiplier, not by HBM) ----
    r32 = torch.empty((16384, 16384), dtype=torch.float32, device=device)
    entry("uniform_ fp32 [16384,16384] (write only; Philox-bound)", 16384 * 16384 * 4, lambda: r32.uniform_())
    entry("normal_ fp32 [16384,16384] (write only; Box-Muller with logf / sincospif)", 16384 * 16384 * 4, lambda: r32.normal_())
    del r32
    dx = device_randn((16384, 11008), torch.bfloat16, device, 18)
    entry("dropout(p=0.1) bf16 [16384,11008] (read, write + 1-byte mask)", 16384 * 11008 * 5, lambda: F.dropout(dx, 0.1, training=True))
    del dx
    torch.supa.empty_cache()
    return out

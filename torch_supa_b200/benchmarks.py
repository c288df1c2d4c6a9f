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
    from . import supa as supa_mod

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


def time_op(fn, warmup=3, iters=10, reps=5):
    """Median milliseconds per call of ``fn()``, measured with events on the current supa stream.  Each sample
    brackets ``reps`` back-to-back calls with one event pair, so that the device queue stays full and the host's
    dispatch time between an event and the launch that follows it is not counted as kernel time."""
    for _ in range(warmup):
        fn()
    torch.supa.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / reps)
    return statistics.median(times)


def _entry(name, nbytes, ms, peak):
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"name": name, "ms": round(ms, 4), "algorithmic_bytes": nbytes, "gbs": round(gbs, 1), "frac_of_measured": round(gbs / peak, 3),
            "frac_of_8TBs": round(gbs / 8000.0, 3)}


def run_extras(device, peak_gbs, quick=False, profile=False):
    """Times the secondary configurations (everything but the headline workload) and returns a list of
    {name, ms, algorithmic_bytes, gbs, frac_of_measured}.  Bytes follow the counting rule of the benchmark
    description: every distinct input element read once, every output element written once."""
    out = []
    it = 5 if quick else 10
    _timer = globals()["time_op"]  # the module-level timer; the name is rebound locally below
    if profile:  # one warm-up and one timed launch per operator: short enough to sit under a profiler

        def time_op(fn, warmup=1, iters=1):  # noqa: F811  (shadows the module-level timer inside this function)
            return _timer(fn, 1, 1, 1)
    else:

        def time_op(fn, warmup=3, iters=10):  # noqa: F811
            return _timer(fn, warmup, iters)

    # ---- config 0: cross entropy fp32 [4096, 32000], forward + backward through autograd ----
    x = device_randn((4096, 32000), torch.float32, device, 0, 2.0).requires_grad_(True)
    t = device_randn((4096,), torch.int64, device, 1, low=0, high=31999)

    def ce():
        x.grad = None
        F.cross_entropy(x, t).backward()

    out.append(_entry("cross_entropy fwd+bwd fp32 [4096,32000] (operator API, autograd)", 2 * 4096 * 32000 * 4 + 4096 * 8,
                      time_op(ce, iters=it), peak_gbs))
    del x, t

    # ---- config 1: SwiGLU chain bf16 ----
    rows, half = 16384, 11008
    xx = device_randn((rows, 2 * half), torch.bfloat16, device, 2)
    a, b = xx[:, :half], xx[:, half:]
    g = device_randn((rows, half), torch.bfloat16, device, 3)
    u = device_randn((rows, half), torch.bfloat16, device, 4)
    n = rows * half * 2
    s = F.silu(a)
    out.append(_entry("silu(a) bf16, a = strided half of [16384,22016]", 2 * n, time_op(lambda: F.silu(a), iters=it), peak_gbs))
    out.append(_entry("silu(a) * b bf16 (mul, b strided half)", 3 * n, time_op(lambda: s * b, iters=it), peak_gbs))
    out.append(_entry("glu(x) bf16 [16384,22016] (fused a * sigmoid(b))", 3 * n, time_op(lambda: F.glu(xx, -1), iters=it), peak_gbs))
    out.append(_entry("silu_backward bf16", 3 * n, time_op(lambda: torch.ops.aten.silu_backward(g, a), iters=it), peak_gbs))
    out.append(_entry("gelu(tanh) bf16 [16384,11008]", 2 * n, time_op(lambda: F.gelu(u, approximate="tanh"), iters=it), peak_gbs))
    out.append(_entry("gelu_backward(tanh) bf16", 3 * n, time_op(lambda: torch.ops.aten.gelu_backward(g, u, approximate="tanh"), iters=it),
                      peak_gbs))
    out.append(_entry("gelu(erf) bf16 [16384,11008]", 2 * n, time_op(lambda: F.gelu(u), iters=it), peak_gbs))
    del xx, a, b, g, u, s

    # ---- config 2: broadcast / strided / promoting binary ops ----
    p = device_randn((64, 1, 4096), torch.float16, device, 5)
    q = device_randn((1, 2048, 4096), torch.float16, device, 6)
    out.append(_entry("add fp16 [64,1,4096] + [1,2048,4096]", 64 * 2048 * 4096 * 2 + 64 * 4096 * 2 + 2048 * 4096 * 2,
                      time_op(lambda: p + q, iters=it), peak_gbs))
    w = torch.empty((64, 2048, 4096), dtype=torch.float16, device=device)
    out.append(_entry("fill_ fp16 [64,2048,4096] (write only)", 64 * 2048 * 4096 * 2, time_op(lambda: w.fill_(1.0), iters=it), peak_gbs))
    del p, q, w
    m = device_randn((8192, 4096), torch.float32, device, 7).t()
    nn_ = device_randn((4096, 8192), torch.float32, device, 8)
    out.append(_entry("mul fp32 transposed view [4096,8192] * contiguous (m.t() * n)", 3 * 4096 * 8192 * 4, time_op(lambda: m * nn_, iters=it),
                      peak_gbs))
    out.append(_entry("mul fp32 contiguous * transposed view (n * m.t())", 3 * 4096 * 8192 * 4, time_op(lambda: nn_ * m, iters=it), peak_gbs))
    del m, nn_
    i32 = device_randn((8192, 8192), torch.int32, device, 9, low=-1000, high=1000)
    f32 = device_randn((8192, 8192), torch.float32, device, 10)
    out.append(_entry("add int32 + fp32 [8192,8192] -> fp32", 3 * 8192 * 8192 * 4, time_op(lambda: i32 + f32, iters=it), peak_gbs))
    del i32, f32

    # ---- config 3: row reductions and log_softmax ----
    r = device_randn((8192, 65536), torch.bfloat16, device, 11)
    nb = 8192 * 65536 * 2 + 8192 * 2
    out.append(_entry("sum(-1) bf16 [8192,65536]", nb, time_op(lambda: r.sum(-1), iters=it), peak_gbs))
    out.append(_entry("mean(-1) bf16 [8192,65536]", nb, time_op(lambda: r.mean(-1), iters=it), peak_gbs))
    out.append(_entry("amax(-1) bf16 [8192,65536]", nb, time_op(lambda: r.amax(-1), iters=it), peak_gbs))
    out.append(_entry("sum(-1, dtype=float32) bf16 [8192,65536]", nb + 8192 * 2, time_op(lambda: r.sum(-1, dtype=torch.float32), iters=it),
                      peak_gbs))
    del r
    torch.supa.empty_cache()
    ls_rows = 16384 if (quick or profile) else 65536
    sm = device_randn((ls_rows, 32000), torch.float32, device, 12, 3.0)
    out.append(_entry(f"log_softmax(-1) fp32 [{ls_rows},32000]", 2 * ls_rows * 32000 * 4, time_op(lambda: F.log_softmax(sm, -1), iters=3 if not quick else 3),
                      peak_gbs))
    if ls_rows <= 16384:
        y = F.log_softmax(sm, -1)
        go = device_randn((ls_rows, 32000), torch.float32, device, 18)
        out.append(_entry(f"log_softmax backward fp32 [{ls_rows},32000] (2 reads, 1 write)", 3 * ls_rows * 32000 * 4,
                          time_op(lambda: torch.ops.aten._log_softmax_backward_data(go, y, -1, torch.float32), iters=3), peak_gbs))
        out.append(_entry(f"softmax(-1) fp32 [{ls_rows},32000]", 2 * ls_rows * 32000 * 4, time_op(lambda: F.softmax(sm, -1), iters=3),
                          peak_gbs))
        del y, go
    del sm
    torch.supa.empty_cache()
    # ---- beyond the headline configurations: nll_loss2d on a segmentation-shaped input ----
    n4, c4, h4, w4 = 8, 19, 1024, 2048
    logp = device_randn((n4, c4, h4, w4), torch.float32, device, 13)
    t4 = device_randn((n4, h4, w4), torch.int64, device, 14, low=0, high=c4 - 1)
    samples = n4 * h4 * w4
    out.append(_entry("nll_loss2d forward (mean) fp32 [8,19,1024,2048]: one gathered element + target per sample",
                      samples * (4 + 8), time_op(lambda: F.nll_loss(logp, t4), iters=it), peak_gbs))
    go = device_randn((), torch.float32, device, 15)
    tw = torch.ones((), dtype=torch.float32, device=device)
    out.append(_entry("nll_loss2d backward (mean) fp32 [8,19,1024,2048]: gradient written once + targets",
                      samples * c4 * 4 + samples * 8,
                      time_op(lambda: torch.ops.aten.nll_loss2d_backward(go, logp, t4, None, 1, -100, tw), iters=it), peak_gbs))
    del logp, t4
    torch.supa.empty_cache()
    # ---- binary_cross_entropy_with_logits, fp32 [8192,8192] ----
    bx = device_randn((8192, 8192), torch.float32, device, 16, 3.0).requires_grad_(True)
    bt = device_randn((8192, 8192), torch.float32, device, 17, uniform=True)
    nb2 = 8192 * 8192 * 4
    out.append(_entry("binary_cross_entropy_with_logits mean fp32 [8192,8192] (fused loss + reduction: 2 reads)", 2 * nb2,
                      time_op(lambda: F.binary_cross_entropy_with_logits(bx.detach(), bt), iters=it), peak_gbs))

    def bce_step():
        bx.grad = None
        F.binary_cross_entropy_with_logits(bx, bt).backward()

    out.append(_entry("binary_cross_entropy_with_logits mean fwd+bwd fp32 [8192,8192] (2 reads + 2 reads, 1 write)", 5 * nb2,
                      time_op(bce_step, iters=it), peak_gbs))
    del bx, bt
    torch.supa.empty_cache()
    return out

"""Generates tests/golden/hotpath_golden.npz from PyTorch's CPU ATen kernels.

The reference's tests keep no stored vectors; their golden is always the CPU result of the same torch
call (torch_supa/testing/common_utils.py:151-168).  This script freezes such CPU results for small
seeded inputs so that the C oracle and the CUDA kernels can be checked against them anywhere.

Run from the repository root:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "hotpath_golden.npz"


def ce_cases():
    """(name, rows, classes, reduction, ignore_index, n_ignored, label_smoothing)"""
    cases = []
    for rows, classes in ((6, 130), (1, 6), (9, 1027)):
        for red in ("mean", "sum", "none"):
            for ign, eps in ((0, 0.0), (2, 0.0), (0, 0.1), (2, 0.1)):
                if rows == 1 and ign:
                    continue
                if classes == 1027 and (red, ign, eps) not in (("mean", 2, 0.1), ("none", 0, 0.0), ("sum", 2, 0.0)):
                    continue
                cases.append((f"ce_{rows}x{classes}_{red}_ign{ign}_eps{int(eps * 10)}", rows, classes, red, -100, ign, eps))
    cases.append(("ce_4x10_mean_allignored", 4, 10, "mean", -100, 4, 0.0))
    cases.append(("ce_5x12_mean_ignoreclass2", 5, 12, "mean", 2, 0, 0.0))
    return cases


def main():
    torch.manual_seed(0)
    torch.set_num_threads(1)
    d = {}
    g = torch.Generator().manual_seed(0)
    for name, rows, classes, red, ignore_index, n_ign, eps in ce_cases():
        x = (torch.randn(rows, classes, generator=g) * 2).requires_grad_(True)
        t = torch.randint(0, classes, (rows,), generator=g)
        if n_ign:
            t[torch.randperm(rows, generator=g)[:n_ign]] = ignore_index
        loss = F.cross_entropy(x, t, ignore_index=ignore_index, label_smoothing=eps, reduction=red)
        go = torch.randn(loss.shape, generator=g) if red == "none" else torch.tensor(0.75)
        (grad,) = torch.autograd.grad(loss, x, go)
        d[name + "/logits"] = x.detach().numpy()
        d[name + "/target"] = t.numpy()
        d[name + "/loss"] = loss.detach().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad"] = grad.numpy()
        d[name + "/meta"] = np.array([ignore_index, eps], dtype=np.float64)

    # log_softmax forward/backward over the last and a middle dimension
    for name, shape, dim in (("lsm_last", (7, 300), 1), ("lsm_mid", (3, 17, 5), 1), ("lsm_long", (2, 2500), 1)):
        x = (torch.randn(*shape, generator=g) * 3).requires_grad_(True)
        y = F.log_softmax(x, dim)
        go = torch.randn(*shape, generator=g)
        (gi,) = torch.autograd.grad(y, x, go)
        d[name + "/x"] = x.detach().numpy()
        d[name + "/y"] = y.detach().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad_in"] = gi.numpy()
        d[name + "/dim"] = np.array([dim])

    # nll_loss with and without class weights
    for name, red, use_w in (("nll_mean", "mean", False), ("nll_sum_w", "sum", True), ("nll_none_w", "none", True),
                             ("nll_mean_w", "mean", True)):
        logp = F.log_softmax(torch.randn(11, 23, generator=g), 1).requires_grad_(True)
        t = torch.randint(0, 23, (11,), generator=g)
        t[3] = -100
        w = torch.rand(23, generator=g) + 0.5 if use_w else None
        out = F.nll_loss(logp, t, weight=w, reduction=red)
        go = torch.randn(out.shape, generator=g)
        (gi,) = torch.autograd.grad(out, logp, go)
        d[name + "/logp"] = logp.detach().numpy()
        d[name + "/target"] = t.numpy()
        if use_w:
            d[name + "/weight"] = w.numpy()
        d[name + "/out"] = out.detach().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad_in"] = gi.numpy()

    # row reductions
    r = torch.randn(9, 777, generator=g)
    d["red/x"] = r.numpy()
    d["red/sum"] = r.sum(-1).numpy()
    d["red/mean"] = r.mean(-1).numpy()
    d["red/amax"] = r.amax(-1).numpy()
    d["red/amin"] = r.amin(-1).numpy()
    d["red/sum_dim0"] = r.sum(0).numpy()
    rb = r.bfloat16()
    d["red/bf16_sum"] = rb.sum(-1).float().numpy()
    d["red/bf16_sum_f32"] = rb.sum(-1, dtype=torch.float32).numpy()
    d["red/bf16_mean"] = rb.mean(-1).float().numpy()
    d["red/bf16_amax"] = rb.amax(-1).float().numpy()

    # activations forward / backward
    a = (torch.randn(5, 14, generator=g) * 2).requires_grad_(True)
    go = torch.randn(5, 14, generator=g)
    for key, fn in (("gelu_erf", lambda v: F.gelu(v)), ("gelu_tanh", lambda v: F.gelu(v, approximate="tanh")),
                    ("silu", F.silu)):
        y = fn(a)
        (gi,) = torch.autograd.grad(y, a, go)
        d[f"act/{key}"] = y.detach().numpy()
        d[f"act/{key}_bwd"] = gi.numpy()
    y = F.glu(a, -1)
    go_glu = torch.randn(5, 7, generator=g)
    (gi,) = torch.autograd.grad(y, a, go_glu)
    d["act/x"] = a.detach().numpy()
    d["act/grad_out"] = go.numpy()
    d["act/glu"] = y.detach().numpy()
    d["act/glu_grad_out"] = go_glu.numpy()
    d["act/glu_bwd"] = gi.numpy()

    # binary ops with promotion and broadcasting
    p = torch.randn(4, 1, 16, generator=g).half()
    q = torch.randn(1, 5, 16, generator=g).half()
    d["bin/p"] = p.numpy()
    d["bin/q"] = q.numpy()
    d["bin/p_plus_q"] = (p + q).numpy()
    i32 = torch.randint(-1000, 1001, (8, 8), generator=g, dtype=torch.int32)
    f32 = torch.randn(8, 8, generator=g)
    d["bin/i32"] = i32.numpy()
    d["bin/f32"] = f32.numpy()
    d["bin/i32_plus_f32"] = (i32 + f32).numpy()
    d["bin/add_alpha"] = torch.add(f32, f32.t(), alpha=2.5).numpy()
    d["bin/mul_t"] = (f32.t() * f32).numpy()
    big = torch.tensor([2**31 - 1, -2**31, 7], dtype=torch.int32)
    d["bin/int_wrap"] = (big + torch.tensor([1, -1, 3], dtype=torch.int32)).numpy()
    # nll_loss2d: (N, C, H, W) log-probabilities and (N, H, W) targets (drawn last: earlier cases keep their values)
    for name, red, use_w in (("nll2d_mean", "mean", False), ("nll2d_sum_w", "sum", True), ("nll2d_none_w", "none", True),
                             ("nll2d_mean_w", "mean", True)):
        logp = F.log_softmax(torch.randn(2, 5, 3, 7, generator=g), 1).requires_grad_(True)
        t = torch.randint(0, 5, (2, 3, 7), generator=g)
        t[0, 1, 2] = -100
        t[1, 2, 6] = -100
        w = torch.rand(5, generator=g) + 0.5 if use_w else None
        out = F.nll_loss(logp, t, weight=w, reduction=red)
        go = torch.randn(out.shape, generator=g)
        (gi,) = torch.autograd.grad(out, logp, go)
        d[name + "/logp"] = logp.detach().numpy()
        d[name + "/target"] = t.numpy()
        if use_w:
            d[name + "/weight"] = w.numpy()
        d[name + "/out"] = out.detach().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad_in"] = gi.numpy()
    # binary_cross_entropy_with_logits (drawn after everything above)
    for name, shape, use_w, pw_shape in (("bce_plain", (6, 9), False, None), ("bce_w", (6, 9), True, None), ("bce_pw", (6, 9), False, (9,)),
                                         ("bce_pw_w", (2, 3, 4), True, (3, 1))):
        x = (torch.rand(*shape, generator=g) * 10 - 5).requires_grad_(True)
        t = torch.rand(*shape, generator=g)
        w = torch.rand(*shape, generator=g) * 1.9 + 0.1 if use_w else None
        pw = torch.rand(*pw_shape, generator=g) * 2.9 + 0.1 if pw_shape else None
        loss = F.binary_cross_entropy_with_logits(x, t, weight=w, pos_weight=pw, reduction="none")
        go = torch.randn(*shape, generator=g)
        (gi,) = torch.autograd.grad(loss, x, go)
        d[name + "/x"] = x.detach().numpy()
        d[name + "/target"] = t.numpy()
        if use_w:
            d[name + "/weight"] = w.numpy()
        if pw_shape:
            d[name + "/pos_weight"] = pw.numpy()
        d[name + "/loss"] = loss.detach().numpy()
        d[name + "/mean"] = loss.detach().mean().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad_in"] = gi.numpy()
    # softmax (not log), drawn after everything above
    for name, shape, dim in (("sm_last", (7, 300), 1), ("sm_mid", (3, 17, 5), 1)):
        x = (torch.randn(*shape, generator=g) * 3).requires_grad_(True)
        y = F.softmax(x, dim)
        go = torch.randn(*shape, generator=g)
        (gi,) = torch.autograd.grad(y, x, go)
        d[name + "/x"] = x.detach().numpy()
        d[name + "/y"] = y.detach().numpy()
        d[name + "/grad_out"] = go.numpy()
        d[name + "/grad_in"] = gi.numpy()
        d[name + "/dim"] = np.array([dim])
    # ---- everything below was added after the cases above and is drawn after them, so their values stay as they were ----
    # cross entropy with class weights and label smoothing together
    for name, rows, classes, red in (("cew_mean", 7, 40, "mean"), ("cew_sum", 5, 33, "sum"), ("cew_none", 6, 21, "none")):
        x = (torch.randn(rows, classes, generator=g) * 2).requires_grad_(True)
        t = torch.randint(0, classes, (rows,), generator=g)
        t[1] = -100
        w = torch.rand(classes, generator=g) + 0.25
        loss = F.cross_entropy(x, t, weight=w, label_smoothing=0.2, reduction=red)
        go = torch.randn(loss.shape, generator=g) if red == "none" else torch.tensor(1.5)
        (grad,) = torch.autograd.grad(loss, x, go)
        for key, val in (("logits", x.detach()), ("target", t), ("weight", w), ("loss", loss.detach()), ("grad_out", go), ("grad", grad)):
            d[f"{name}/{key}"] = val.numpy()
    # cross entropy with class-probability targets, with and without weights and smoothing
    for name, rows, classes, red, use_w, eps in (("cep_mean", 6, 50, "mean", False, 0.0), ("cep_sum_w", 4, 31, "sum", True, 0.0),
                                                 ("cep_none_eps", 5, 19, "none", False, 0.1), ("cep_mean_w_eps", 7, 64, "mean", True, 0.3)):
        x = (torch.randn(rows, classes, generator=g) * 2).requires_grad_(True)
        t = torch.softmax(torch.randn(rows, classes, generator=g), 1)
        w = torch.rand(classes, generator=g) + 0.25 if use_w else None
        loss = F.cross_entropy(x, t, weight=w, label_smoothing=eps, reduction=red)
        go = torch.randn(loss.shape, generator=g) if red == "none" else torch.tensor(0.5)
        (grad,) = torch.autograd.grad(loss, x, go)
        for key, val in (("logits", x.detach()), ("target", t), ("loss", loss.detach()), ("grad_out", go), ("grad", grad)):
            d[f"{name}/{key}"] = val.numpy()
        if use_w:
            d[f"{name}/weight"] = w.numpy()
        d[f"{name}/eps"] = np.array([eps])
    # extrema with indices: ties resolve to the first index, NaN wins for max and for min
    a = torch.randint(-3, 4, (5, 9, 4), generator=g).float()
    a[1, 3, 2] = float("nan")
    a[1, 6, 2] = float("nan")
    a[4, 0, 0] = float("nan")
    d["arg/x"] = a.numpy()
    for dim in (0, 1, 2):
        mv, mi = a.max(dim)
        nv, ni = a.min(dim)
        d[f"arg/max{dim}_values"], d[f"arg/max{dim}_indices"] = mv.numpy(), mi.numpy()
        d[f"arg/min{dim}_values"], d[f"arg/min{dim}_indices"] = nv.numpy(), ni.numpy()
    d["arg/argmax_flat"] = np.array(a[0].argmax().item())
    d["arg/argmin_flat"] = np.array(a[0].argmin().item())
    ai = torch.randint(-50, 50, (6, 11), generator=g, dtype=torch.int32)
    d["arg/i32"] = ai.numpy()
    d["arg/i32_argmax1"] = ai.argmax(1).numpy()
    d["arg/i32_min1_values"], d["arg/i32_min1_indices"] = (v.numpy() for v in ai.min(1))
    # var / std / var_mean
    v = torch.randn(4, 37, 3, generator=g) * 3 + 5
    d["mom/x"] = v.numpy()
    for dim in (0, 1, 2):
        d[f"mom/var{dim}"] = v.var(dim).numpy()
        d[f"mom/std{dim}_c0"] = v.std(dim, correction=0).numpy()
    d["mom/var_all"] = v.var().numpy()
    d["mom/var_dims02"] = v.var((0, 2)).numpy()
    d["mom/mean1"] = v.mean(1).numpy()
    # prod / nansum
    pr = torch.rand(5, 12, generator=g) + 0.5
    d["prod/x"] = pr.numpy()
    d["prod/dim1"] = pr.prod(1).numpy()
    d["prod/all"] = pr.prod().numpy()
    ns = torch.randn(4, 9, generator=g)
    ns[0, 2] = float("nan")
    ns[3, :] = float("nan")
    d["nansum/x"] = ns.numpy()
    d["nansum/dim1"] = ns.nansum(1).numpy()
    # div with a rounding mode: floats (signs, zeros, exact multiples) and integers
    da = torch.tensor([7.5, -7.5, 7.5, -7.5, 6.0, -6.0, 0.0, -0.0, 5.0, 1e-3, 3.0, -3.0])
    db = torch.tensor([2.0, 2.0, -2.0, -2.0, 3.0, 3.0, 4.0, 4.0, 0.0, 7.0, 0.3, 0.3])
    d["div/a"], d["div/b"] = da.numpy(), db.numpy()
    d["div/trunc"] = torch.div(da, db, rounding_mode="trunc").numpy()
    d["div/floor"] = torch.div(da, db, rounding_mode="floor").numpy()
    ia = torch.randint(-40, 41, (64,), generator=g, dtype=torch.int32)
    ib = torch.randint(1, 9, (64,), generator=g, dtype=torch.int32) * (torch.randint(0, 2, (64,), generator=g, dtype=torch.int32) * 2 - 1)
    d["div/ia"], d["div/ib"] = ia.numpy(), ib.numpy()
    d["div/itrunc"] = torch.div(ia, ib, rounding_mode="trunc").numpy()
    d["div/ifloor"] = torch.div(ia, ib, rounding_mode="floor").numpy()
    np.savez_compressed(OUT, **d)
    print("wrote", OUT, OUT.stat().st_size, "bytes,", len(d), "arrays")


if __name__ == "__main__":
    main()

"""Rows beside the benchmark's: probability targets, indexed extrema, moments, prod / nansum, div rounding modes — through
the C ABI against the fixtures and the oracle, and through the supa operator API against the CPU (needs a GPU)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def supa():
    import torch_supa_b200  # noqa: F401

    if not torch.supa.is_available():
        pytest.skip("no supa device")
    return torch.device("supa", 0)


# ---- cross entropy with probability targets --------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["cep_mean", "cep_sum_w", "cep_none_eps", "cep_mean_w_eps"])
def test_prob_targets_golden(golden, cuda_device, name):
    from torch_supa_b200 import functional as F2

    red = name.split("_")[1]
    go = golden[name + "/grad_out"]
    w = torch.from_numpy(golden[name + "/weight"]).to(cuda_device) if name + "/weight" in golden.files else None
    kw = dict(label_smoothing=float(golden[name + "/eps"][0]), reduction=red, class_weight=w)
    if red == "none":
        kw["row_grad_out"] = torch.from_numpy(go).to(cuda_device)
    else:
        kw["grad_scale"] = float(go)
    loss, grad = F2.cross_entropy_prob_forward_backward(torch.from_numpy(golden[name + "/logits"]).to(cuda_device),
                                                        torch.from_numpy(golden[name + "/target"]).to(cuda_device), **kw)
    torch.cuda.synchronize()
    assert_close(np.atleast_1d(loss.cpu().numpy()), np.atleast_1d(golden[name + "/loss"]), 2e-6, 2e-6, name + " loss")
    assert_close(grad.cpu().numpy(), golden[name + "/grad"], 1e-5, 3e-7, name + " grad")


@pytest.mark.parametrize("rows,classes,dtype", [(64, 32000, torch.float32), (33, 50257, torch.bfloat16), (500, 1000, torch.float32),
                                                (17, 129, torch.float16), (4, 128256, torch.bfloat16)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_prob_targets_against_oracle(cuda_device, rows, classes, dtype, reduction):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(rows + classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.softmax(torch.randn(rows, classes, generator=g) * 3, 1).to(dtype)
    w = torch.rand(classes, generator=g) + 0.25
    eps = 0.1 if classes % 2 else 0.0
    loss, grad = F2.cross_entropy_prob_forward_backward(logits.to(cuda_device), target.to(cuda_device), label_smoothing=eps,
                                                        reduction=reduction, class_weight=w.to(cuda_device))
    torch.cuda.synchronize()
    eloss, egrad = oracle.c_cross_entropy_prob(logits.float().numpy(), target.float().numpy(), w.numpy(), eps, reduction)
    scale = float(rows) if reduction == "mean" else 1.0
    if dtype == torch.float32:
        assert_close(np.atleast_1d(loss.cpu().numpy()), eloss, 4e-6, 4e-6, "loss")
        assert_close(grad.cpu().numpy() * scale, egrad * scale, 1e-5, 3e-7, "grad")
    else:
        rtol, atol = (1.6e-2, 1e-4) if dtype == torch.bfloat16 else (2e-3, 2e-5)
        assert_close(np.atleast_1d(loss.float().cpu().numpy()), eloss, 1e-2 if reduction != "none" else 4e-6, 4e-6, "loss")
        assert_close(grad.float().cpu().numpy() * scale, egrad * scale, rtol, atol, "grad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_prob_targets_operator(supa, dtype, reduction):
    """F.cross_entropy with float targets on the supa device: the fused kernel, its autograd node and the CPU agree."""
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(21)
    x_cpu = (torch.randn(40, 700, generator=g) * 2).to(dtype)
    t_cpu = torch.softmax(torch.randn(40, 700, generator=g), 1).to(dtype)
    w = torch.rand(700, generator=g) + 0.5
    xr = x_cpu.float().clone().requires_grad_(True)
    ref = F.cross_entropy(xr, t_cpu.float(), weight=w, label_smoothing=0.1, reduction=reduction)
    x = x_cpu.clone().to(supa).requires_grad_(True)
    out = F.cross_entropy(x, t_cpu.to(supa), weight=w.to(supa), label_smoothing=0.1, reduction=reduction)
    go = torch.rand(ref.shape, generator=g) + 0.5
    ref.backward(go)
    out.backward(go.to(dtype).to(supa))
    rt, at = {torch.float32: (2e-5, 1e-6), torch.bfloat16: (1.6e-2, 1e-3), torch.float16: (2e-3, 1e-4)}[dtype]
    assert out.dtype == dtype and out.shape == ref.shape
    assert_allclose(ref.detach(), out.detach().float(), rt, at)
    assert_allclose(xr.grad, x.grad.float(), rt * 2, at * 1e-1)
    with pytest.raises(RuntimeError, match="ignore_index is not supported"):
        F.cross_entropy(x.detach(), t_cpu.to(supa), ignore_index=3)


# ---- extrema with indices -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [0, 1, 2])
@pytest.mark.parametrize("is_max", [True, False])
def test_indexed_extrema_golden(golden, cuda_device, dim, is_max):
    from torch_supa_b200 import functional as F2

    values, indices = F2.arg_reduce(torch.from_numpy(golden["arg/x"]).to(cuda_device), dim, is_max)
    key = f"arg/{'max' if is_max else 'min'}{dim}"
    assert np.array_equal(indices.cpu().numpy(), golden[key + "_indices"])
    assert np.array_equal(values.cpu().numpy(), golden[key + "_values"], equal_nan=True)


@pytest.mark.parametrize("shape,dim", [((7, 100000), 1), ((3, 5000000), 1), ((2000, 300), 1), ((64, 257, 33), 1), ((1, 3000000), 1),
                                       ((100000, 8), 0), ((70000, 3), 1),
                                       # lane groups per row (1 - 32 lanes, vector and scalar loads), columns in chunks
                                       ((70001, 64), 1), ((5000, 1000), 1), ((3000, 1001), 1), ((9000, 8), 1), ((4000, 2048), 1),
                                       ((300000, 64), 0), ((40000, 33), 0), ((3, 20000, 70), 1), ((50, 4100), 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32, torch.int64, torch.float64])
def test_indexed_extrema_bit_exact_against_cpu(cuda_device, shape, dim, dtype):
    """Every path of the kernel (rows in one CTA, rows cut into segments, columns), every accumulation type; few distinct
    values so that ties are everywhere: the lowest index must win, bit for bit."""
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = torch.randint(-6, 7, shape, generator=g)
    x = x.to(dtype) if not dtype.is_floating_point else (x.to(torch.float32) * 0.5).to(dtype)
    if dtype.is_floating_point and shape[0] > 2:
        x[1].view(-1)[min(5, x[1].numel() - 1)] = float("nan")
    for is_max in (True, False):
        values, indices = F2.arg_reduce(x.to(cuda_device), dim, is_max)
        ref_v, ref_i = (x.max(dim) if is_max else x.min(dim))
        assert torch.equal(indices.cpu(), ref_i), "indices"
        assert torch.equal(values.cpu().nan_to_num(777), ref_v.nan_to_num(777)) if dtype.is_floating_point else torch.equal(values.cpu(), ref_v)


def test_indexed_extrema_operator(supa):
    g = torch.Generator().manual_seed(3)
    x = torch.randint(-4, 5, (6, 50, 7), generator=g).float()
    x[2, 10, 3] = float("nan")
    d = x.to(supa)
    for dim in (0, 1, 2, -1):
        for keepdim in (False, True):
            for fn in ("max", "min"):
                v, i = getattr(d, fn)(dim, keepdim)
                rv, ri = getattr(x, fn)(dim, keepdim)
                assert torch.equal(i.cpu(), ri) and torch.equal(v.cpu().nan_to_num(9), rv.nan_to_num(9))
            assert torch.equal(d.argmax(dim, keepdim).cpu(), x.argmax(dim, keepdim))
            assert torch.equal(d.argmin(dim, keepdim).cpu(), x.argmin(dim, keepdim))
    assert d.argmax().item() == x.argmax().item() and d.argmin().item() == x.argmin().item()
    y = x.nan_to_num(0.0)
    assert y.to(supa).max().item() == y.max().item() and y.to(supa).min().item() == y.min().item()
    assert torch.isnan(d.max().cpu())
    t = x.transpose(0, 2)  # a non-contiguous input
    assert torch.equal(t.to(supa).argmax(1).cpu(), t.argmax(1))
    out_v, out_i = torch.empty(0, device=supa), torch.empty(0, dtype=torch.int64, device=supa)
    torch.max(d, 1, out=(out_v, out_i))
    assert torch.equal(out_i.cpu(), x.max(1)[1])
    with pytest.raises(IndexError):
        torch.empty(0, device=supa).argmax()


# ---- var / std ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_moments_golden(golden, cuda_device, dim):
    from torch_supa_b200 import functional as F2

    x = torch.from_numpy(golden["mom/x"]).to(cuda_device)
    var, mean = F2.moments(x, dim, 1.0, False)
    std, _ = F2.moments(x, dim, 0.0, True)
    assert_close(var.cpu().numpy(), golden[f"mom/var{dim}"], 2e-6, 1e-6, "var")
    assert_close(std.cpu().numpy(), golden[f"mom/std{dim}_c0"], 2e-6, 1e-6, "std")
    if dim == 1:
        assert_close(mean.cpu().numpy(), golden["mom/mean1"], 2e-6, 1e-6, "mean")


@pytest.mark.parametrize("shape,dim", [((5, 200000), 1), ((3000, 700), 1), ((40, 1000, 9), 1), ((2, 4000000), 1),
                                       ((70001, 64), 1), ((3000, 1001), 1), ((9000, 8), 1), ((2000, 2048), 1), ((300000, 64), 0),
                                       ((40000, 33), 0), ((3, 20000, 70), 1), ((50, 4100), 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_moments_against_oracle(cuda_device, shape, dim, dtype):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(shape[1])
    x = (torch.randn(shape, generator=g) * 2 + 100).to(dtype)  # a mean far from zero: the naive sum of squares would cancel
    var, mean = F2.moments(x.to(cuda_device), dim, 1.0, False)
    evar, emean = oracle.c_moments(x.double().numpy(), dim, 1.0, False)
    rtol = {torch.float32: 2e-6, torch.bfloat16: 8e-3, torch.float64: 1e-12}[dtype]
    assert_close(var.double().cpu().numpy(), evar, rtol, 0, "var")
    assert_close(mean.double().cpu().numpy(), emean, rtol, 0, "mean")


def test_moments_operator(supa):
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 40, 9, generator=g) * 2 + 3
    d = x.to(supa)
    for dim in (None, 0, 1, -1, (0, 2), (1, 2)):
        for keepdim in (False, True):
            for corr in (0, 1, 2):
                kw = dict(dim=dim, correction=corr, keepdim=keepdim)
                assert_allclose(x.var(**kw), d.var(**kw), 2e-6, 1e-6)
                assert_allclose(x.std(**kw), d.std(**kw), 2e-6, 1e-6)
    v, m = torch.var_mean(d, 1)
    rv, rm = torch.var_mean(x, 1)
    assert_allclose(rv, v, 2e-6, 1e-6)
    assert_allclose(rm, m, 2e-6, 1e-6)
    s, m = torch.std_mean(d, (0, 1), correction=0)
    rs, rm = torch.std_mean(x, (0, 1), correction=0)
    assert_allclose(rs, s, 2e-6, 1e-6)
    assert_allclose(rm, m, 2e-6, 1e-6)
    one = torch.tensor([2.0]).to(supa)
    assert torch.isnan(one.var().cpu())  # n - correction = 0
    xb = x.bfloat16()
    assert_allclose(xb.var(1), xb.to(supa).var(1), 1.6e-2, 1e-3)
    xg = x.clone().requires_grad_(True)
    dg = x.to(supa).requires_grad_(True)
    xg.var(1).sum().backward()  # the derivative formula of var composes sub / mul / sum, all on the device
    dg.var(1).sum().backward()
    assert_allclose(xg.grad, dg.grad, 1e-5, 1e-6)


# ---- prod / nansum --------------------------------------------------------------------------------------------------
def test_prod_nansum_operator(supa, golden):
    from tests.supa_testing import assert_allclose

    pr = torch.from_numpy(golden["prod/x"])
    assert_allclose(torch.from_numpy(golden["prod/dim1"]), pr.to(supa).prod(1), 2e-6, 1e-7)
    assert_allclose(torch.from_numpy(golden["prod/all"]), pr.to(supa).prod(), 4e-6, 1e-7)
    assert_allclose(pr.prod(0, keepdim=True), pr.to(supa).prod(0, keepdim=True), 2e-6, 1e-7)
    ints = torch.arange(1, 13, dtype=torch.int32).reshape(3, 4)
    assert torch.equal(ints.to(supa).prod(1).cpu(), ints.prod(1)) and ints.to(supa).prod().item() == ints.prod().item()
    ns = torch.from_numpy(golden["nansum/x"])
    assert_allclose(torch.from_numpy(golden["nansum/dim1"]), ns.to(supa).nansum(1), 2e-6, 1e-6)
    assert_allclose(ns.nansum(), ns.to(supa).nansum(), 2e-6, 1e-6)
    g = torch.Generator().manual_seed(1)
    big = torch.randn(64, 70000, generator=g)
    big[big > 2.5] = float("nan")
    assert_allclose(big.nansum(1), big.to(supa).nansum(1), 1e-5, 1e-3)
    assert torch.equal(ints.to(supa).nansum(0).cpu(), ints.nansum(0))


# ---- div with a rounding mode --------------------------------------------------------------------------------------
def test_div_rounding_modes_golden(supa, golden):
    a, b = torch.from_numpy(golden["div/a"]), torch.from_numpy(golden["div/b"])
    for mode in ("trunc", "floor"):
        got = torch.div(a.to(supa), b.to(supa), rounding_mode=mode).cpu()
        want = torch.from_numpy(golden["div/" + mode])
        assert torch.equal(got, want) and torch.equal(torch.signbit(got), torch.signbit(want)), mode
    ia, ib = torch.from_numpy(golden["div/ia"]), torch.from_numpy(golden["div/ib"])
    assert torch.equal(torch.div(ia.to(supa), ib.to(supa), rounding_mode="trunc").cpu(), torch.from_numpy(golden["div/itrunc"]))
    assert torch.equal(torch.div(ia.to(supa), ib.to(supa), rounding_mode="floor").cpu(), torch.from_numpy(golden["div/ifloor"]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.int32, torch.int64, torch.int16, torch.uint8])
@pytest.mark.parametrize("mode", ["trunc", "floor"])
def test_div_rounding_modes_bit_exact_against_cpu(supa, dtype, mode):
    g = torch.Generator().manual_seed(7)
    if dtype.is_floating_point:
        a = (torch.randn(5000, generator=g) * 50).to(dtype)
        b = (torch.randn(5000, generator=g) * 5).to(dtype)
        b[b == 0] = 1
    else:
        lo = 0 if dtype == torch.uint8 else -100
        a = torch.randint(lo, 100, (5000,), generator=g).to(dtype)
        b = torch.randint(1, 12, (5000,), generator=g).to(dtype)
        if dtype != torch.uint8:
            b = b * (torch.randint(0, 2, (5000,), generator=g).to(dtype) * 2 - 1)
    want = torch.div(a, b, rounding_mode=mode)
    got = torch.div(a.to(supa), b.to(supa), rounding_mode=mode)
    assert got.dtype == want.dtype and torch.equal(got.cpu(), want)
    # broadcasting, a Python scalar divisor, the in-place form and //
    a2 = a.reshape(50, 100)
    assert torch.equal(torch.div(a2.to(supa), b[:100].to(supa), rounding_mode=mode).cpu(), torch.div(a2, b[:100], rounding_mode=mode))
    assert torch.equal(torch.div(a.to(supa), 3, rounding_mode=mode).cpu(), torch.div(a, 3, rounding_mode=mode))
    c = a.clone().to(supa)
    c.div_(b.to(supa), rounding_mode=mode)
    assert torch.equal(c.cpu(), want)
    if mode == "floor":
        assert torch.equal((a.to(supa) // b.to(supa)).cpu(), a // b)

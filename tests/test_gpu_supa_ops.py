"""Operators through the ``supa`` device and the ATen dispatcher, golden = the same call on the CPU.

These read like the reference's own op tests (test/test_add.py, test_binary_mul_kernel.py,
test_activation_*_kernel.py, test_reduce_ops.py, test_softmax.py, test_loss.py): build the same data on CPU
and on the device, run the operator on both, compare with the reference's tolerances."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [(16,), (1024, 512), (1023, 511), (1025, 513), (128, 2135)]
DTYPES = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def supa():
    import torch_supa_b200  # noqa: F401

    if not torch.supa.is_available():
        pytest.skip("no supa device")
    return torch.device("supa", 0)


def _pair(shape, dtype, seed=0, requires_grad=False, **kw):
    from tests.supa_testing import create_random_tensor

    return create_random_tensor(shape, dtype, seed=seed, requires_grad=requires_grad, **kw)


def _close(golden, out, dtype=None, loosen=1.0):
    from tests.supa_testing import ATOL, RTOL, assert_allclose

    dtype = dtype or golden.dtype
    assert out.device.type == "supa" and out.dtype == golden.dtype and out.shape == golden.shape
    assert_allclose(golden, out, RTOL[dtype] * loosen, ATOL[dtype] * loosen, equal_nan=True)


# ---- runtime ---------------------------------------------------------------------------------------------------
def test_roundtrip_and_views(supa):
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    d = x.to(supa)
    assert d.device == supa and d.is_supa
    assert torch.equal(d.cpu(), x)
    assert torch.equal(d.transpose(0, 2).contiguous().cpu(), x.transpose(0, 2).contiguous())
    assert torch.equal(d[:, 1:, ::2].cpu(), x[:, 1:, ::2])
    assert torch.equal(d.view(6, 4).t().cpu(), x.view(6, 4).t())
    assert torch.equal(d.to(torch.int32).cpu(), x.to(torch.int32))
    assert torch.equal(torch.ones(5, device=supa).cpu(), torch.ones(5))
    assert torch.equal(torch.zeros(3, 2, device=supa, dtype=torch.bfloat16).cpu(), torch.zeros(3, 2, dtype=torch.bfloat16))
    assert torch.full((4,), 7, device=supa).sum(0).item() == 28
    e = torch.empty(0, device=supa)
    assert e.numel() == 0 and e.cpu().numel() == 0
    y = d.clone()
    y.resize_(4, 6)
    assert y.shape == (4, 6) and torch.equal(y.cpu().flatten(), x.flatten())
    nc = torch.empty(4, 6, device=supa).t()
    nc.copy_(x.view(6, 4))
    assert torch.equal(nc.cpu(), x.view(6, 4))


def test_pinned_non_blocking_copies(supa):
    host = torch.randn(1 << 20).pin_memory()
    d = host.to(supa, non_blocking=True)
    back = torch.empty_like(host).pin_memory()
    back.copy_(d, non_blocking=True)
    torch.supa.synchronize()
    assert torch.equal(back, host)


def test_allocator_statistics_and_host_side_oom(supa):
    torch.supa.synchronize()
    base = torch.supa.memory_allocated()
    x = torch.empty(1 << 20, device=supa)
    assert torch.supa.memory_allocated() - base == 4 << 20
    assert torch.supa.max_memory_allocated() >= base + (4 << 20)
    del x
    assert torch.supa.memory_allocated() == base
    assert torch.supa.memory_reserved() >= 0
    torch.supa.set_memory_limit(base + (1 << 20))
    try:
        with pytest.raises(torch.OutOfMemoryError):
            torch.empty(1 << 20, device=supa)  # 4 MiB > 1 MiB cap: refused on the host, the GPU is never asked
        small = torch.empty(1 << 10, device=supa)
        assert small.numel() == 1 << 10
    finally:
        torch.supa.set_memory_limit(0)
    assert torch.supa.memory_stats()["num_ooms"] >= 1
    torch.supa.empty_cache()


def test_streams_and_events(supa):
    s = torch.Stream(device=supa)
    start, end = torch.Event(device="supa", enable_timing=True), torch.Event(device="supa", enable_timing=True)
    x = torch.randn(1 << 22).to(supa)
    with s:
        start.record()
        y = x * 2
        y.record_stream(s) if hasattr(y, "record_stream") else None
        end.record()
    end.synchronize()
    assert start.elapsed_time(end) >= 0
    s.synchronize()
    assert torch.equal(y.cpu(), x.cpu() * 2)


def test_autograd_engine_runs_backward_on_device(supa):
    a_cpu, a = _pair((64, 128), torch.float32, requires_grad=True)
    b_cpu, b = _pair((64, 128), torch.float32, seed=1, requires_grad=True)
    (F.silu(a) * b).sum().backward()
    (F.silu(a_cpu) * b_cpu).sum().backward()
    _close(a_cpu.grad, a.grad, loosen=4)
    _close(b_cpu.grad, b.grad, loosen=4)


# ---- add / mul ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_add_sub_mul_same_shape(supa, shape, dtype):
    a_cpu, a = _pair(shape, dtype)
    b_cpu, b = _pair(shape, dtype, seed=1)
    _close(a_cpu + b_cpu, a + b)
    _close(a_cpu - b_cpu, a - b)
    _close(a_cpu * b_cpu, a * b)
    _close(torch.add(a_cpu, b_cpu, alpha=2), torch.add(a, b, alpha=2))
    _close(a_cpu / (b_cpu.abs() + 1), a / (b.abs() + 1) if hasattr(torch.Tensor, "_never") else (a / (b_cpu.abs() + 1).to("supa")))
    _close(-a_cpu, -a)


@pytest.mark.parametrize("dtype", DTYPES)
def test_broadcast_scalar_inplace(supa, dtype):
    a_cpu, a = _pair((128, 96), dtype)
    one_cpu, one = _pair((1,), dtype, seed=2)
    row_cpu, row = _pair((96,), dtype, seed=3)
    _close(a_cpu + one_cpu, a + one)
    _close(a_cpu * row_cpu, a * row)
    _close(a_cpu + 2.5, a + 2.5)
    _close(3 * a_cpu, 3 * a)
    _close(1.5 - a_cpu, 1.5 - a)
    _close(a_cpu * 0.5, a * 0.5)
    c_cpu, c = a_cpu.clone(), a.clone()
    c_cpu += row_cpu
    c += row
    _close(c_cpu, c)
    c_cpu *= 2
    c *= 2
    _close(c_cpu, c)
    out = torch.empty(0, device="supa", dtype=dtype)
    torch.add(a, row, out=out)
    _close(a_cpu + row_cpu, out)
    out_t = torch.empty(96, 128, device="supa", dtype=dtype).t()  # out= with foreign strides
    torch.mul(a, row, out=out_t)
    _close(a_cpu * row_cpu, out_t)


def test_as_strided_transposed_operand(supa):
    """The reference's strided-add case (test/test_add.py:79-92): [1, 1024, 512] with strides [524288, 1, 1024]."""
    base_cpu, base = _pair((524288,), torch.float32)
    w_cpu, w = _pair((1, 1024, 512), torch.float32, seed=1)
    v_cpu = base_cpu.as_strided((1, 1024, 512), (524288, 1, 1024))
    v = base.as_strided((1, 1024, 512), (524288, 1, 1024))
    _close(v_cpu + w_cpu, v + w)
    m_cpu, m = _pair((512, 256), torch.float32, seed=2)
    n_cpu, n = _pair((256, 512), torch.float32, seed=3)
    r = m.t() * n
    assert r.stride() == (m_cpu.t() * n_cpu).stride()
    _close(m_cpu.t() * n_cpu, r)
    _close(n_cpu * m_cpu.t(), n * m.t())


def test_type_promotion_contract(supa):
    """bf16 x fp32 -> fp32 (test/test_binary_mul_kernel.py:97-108), int32 + fp32 -> fp32, wrapped numbers."""
    a_cpu, a = _pair((1024, 128), torch.bfloat16)
    b_cpu, b = _pair((1024, 128), torch.float32, seed=1)
    r = a * b
    assert r.dtype == torch.float32
    _close(a_cpu * b_cpu, r)
    i_cpu, i = _pair((256, 256), torch.int32, min_value=-1000, max_value=1000)
    r = i + b[:256, :].contiguous().view(-1)[: 256 * 128].repeat(2).view(256, 256) if False else None
    f_cpu, f = _pair((256, 256), torch.float32, seed=2)
    r = i + f
    assert r.dtype == torch.float32
    assert torch.equal(r.cpu(), i_cpu + f_cpu)
    h_cpu, h = _pair((64,), torch.float16)
    assert (h + 1.5).dtype == torch.float16 and torch.equal((h + 1.5).cpu(), h_cpu + 1.5)
    assert (i * 1.5).dtype == torch.float32 and torch.equal((i * 1.5).cpu(), i_cpu * 1.5)
    b1_cpu, b1 = _pair((100,), torch.bool)
    b2_cpu, b2 = _pair((100,), torch.bool, seed=1)
    assert torch.equal((b1 + b2).cpu(), b1_cpu + b2_cpu) and torch.equal((b1 * b2).cpu(), b1_cpu * b2_cpu)
    big = torch.tensor([2**31 - 1, -2**31], dtype=torch.int32)
    assert torch.equal((big.to(supa) + torch.tensor([1, -1], dtype=torch.int32).to(supa)).cpu(), big + torch.tensor([1, -1], dtype=torch.int32))
    a4_cpu, a4 = _pair((1, 64, 24, 64), torch.bfloat16, seed=5)
    b4_cpu, b4 = _pair((1, 64, 1, 64), torch.float32, seed=6)
    _close(a4_cpu * b4_cpu, a4 * b4)


# ---- activations -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["gelu", "gelu_tanh", "silu"])
def test_activation_forward_backward(supa, shape, dtype, act):
    fn = {"gelu": F.gelu, "gelu_tanh": lambda v: F.gelu(v, approximate="tanh"), "silu": F.silu}[act]
    x_cpu, x = _pair(shape, dtype, requires_grad=True)
    g_cpu, g = _pair(shape, dtype, seed=1)
    y = fn(x)
    # low-precision golden: fp32 on up-cast inputs, cast down (test/test_loss.py:258-276)
    xr = x_cpu.detach().float().requires_grad_(True)
    yr = fn(xr)
    _close(yr.detach().to(dtype), y.detach(), loosen=2)
    y.backward(g)
    yr.backward(g_cpu.float())
    _close(xr.grad.to(dtype), x.grad, loosen=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,dim", [((1024, 512), -1), ((1023, 510), 1), ((64, 22016), -1), ((6, 8, 10), 1), ((512, 100), 0)])
def test_glu_forward_backward(supa, shape, dim, dtype):
    x_cpu, x = _pair(shape, dtype, requires_grad=True)
    y = F.glu(x, dim)
    xr = x_cpu.detach().float().requires_grad_(True)
    yr = F.glu(xr, dim)
    g_cpu, g = _pair(tuple(yr.shape), dtype, seed=1)
    from tests.supa_testing import assert_allclose

    assert_allclose(yr.detach().to(dtype), y.detach(), 1.6e-2 if dtype == torch.bfloat16 else 2e-3 if dtype == torch.float16 else 3e-6,
                    1e-2 if dtype == torch.bfloat16 else 1e-4 if dtype == torch.float16 else 1e-5)
    y.backward(g)
    yr.backward(g_cpu.float())
    assert_allclose(xr.grad.to(dtype), x.grad, 1.6e-2 if dtype == torch.bfloat16 else 3e-3 if dtype == torch.float16 else 4e-6,
                    1e-2 if dtype == torch.bfloat16 else 1e-3 if dtype == torch.float16 else 1e-5)


def test_swiglu_chain_on_views(supa):
    """silu(a) * b with a, b the two halves of one bf16 tensor (strided views), forward and backward."""
    x_cpu, x = _pair((256, 22016), torch.bfloat16, requires_grad=True)
    g_cpu, g = _pair((256, 11008), torch.bfloat16, seed=1)
    out = F.silu(x[:, :11008]) * x[:, 11008:]
    out.backward(g)
    xr = x_cpu.detach().float().requires_grad_(True)
    ref = (F.silu(xr[:, :11008]).bfloat16().float() * xr[:, 11008:])
    ref.backward(g_cpu.float())
    _close(ref.detach().bfloat16(), out.detach(), loosen=1)
    from tests.supa_testing import assert_allclose

    assert_allclose(xr.grad.bfloat16(), x.grad, 2.4e-2, 2e-2)


# ---- reductions ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES + [torch.float64])
@pytest.mark.parametrize("shape,dim", [((16,), 0), ((1024, 512), -1), ((1023, 511), 0), ((64, 65536), -1), ((7, 9, 11), (0, 2)),
                                       ((5, 6, 7, 8), None), ((1,), 0), ((3, 1, 5), 1)])
def test_sum_mean_amax(supa, shape, dim, dtype):
    from tests.supa_testing import assert_allclose

    x_cpu, x = _pair(shape, dtype)
    n = x_cpu.numel() if dim is None else int(np.prod([shape[d] for d in (dim if isinstance(dim, tuple) else (dim,))]))
    for keepdim in (False, True):
        kw = {} if dim is None else {"dim": dim, "keepdim": keepdim}
        for op in ("sum", "mean"):
            out = getattr(x, op)(**kw)
            ref = getattr(x_cpu.double(), op)(**kw)
            assert out.dtype == dtype and out.shape == ref.shape
            if dtype in (torch.bfloat16, torch.float16):
                assert_allclose(ref.to(dtype).float(), out.float(), 8e-3 if dtype == torch.bfloat16 else 1e-3, 2e-2 if op == "sum" else 1e-3)
            else:
                k = max(1.0, 4 * (np.log2(n) - 4)) if n > 32 else 1.0
                assert_allclose(ref.to(dtype), out, k * 1.3e-6 if dtype == torch.float32 else 1e-12,
                                k * 1e-5 * (max(1.0, n ** 0.5 / 8) if op == "sum" else 1) if dtype == torch.float32 else 1e-10)
        if dim is not None:
            assert torch.equal(x.amax(**kw).cpu(), x_cpu.amax(**kw)), "amax is exact"
            assert torch.equal(x.amin(**kw).cpu(), x_cpu.amin(**kw))


def test_reduction_dtype_rules(supa):
    x_cpu, x = _pair((300, 700), torch.bfloat16)
    out = x.sum(-1, dtype=torch.float32)
    assert out.dtype == torch.float32
    _close(x_cpu.sum(-1, dtype=torch.float32), out, loosen=40)
    i_cpu, i = _pair((50, 999), torch.int32, min_value=0, max_value=100)
    assert i.sum().dtype == torch.int64 and i.sum().item() == i_cpu.sum().item()
    assert torch.equal(i.sum(1).cpu(), i_cpu.sum(1))
    b_cpu, b = _pair((1000,), torch.bool)
    assert b.sum().item() == b_cpu.sum().item()
    nan_cpu = x_cpu.float().clone()
    nan_cpu[5, 77] = float("nan")
    assert torch.isnan(nan_cpu.to(supa).amax(-1).cpu()[5]).item()
    with pytest.raises((RuntimeError, IndexError)):
        torch.empty(0, 4, device=supa).amax(0)
    assert torch.equal(torch.empty(0, 4, device=supa).sum(0).cpu(), torch.zeros(4))
    out = torch.empty(0, device=supa)
    torch.sum(x.float(), 1, out=out)
    _close(x_cpu.float().sum(1), out, loosen=40)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(16,), (1024, 512), (1023, 511), (3, 5, 7)])
def test_neighbouring_unary_ops_forward_backward(supa, shape, dtype):
    """sigmoid / tanh / exp / log and their autograd formulas (sigmoid_backward, tanh_backward, mul, div) on the device."""
    from tests.supa_testing import ATOL, RTOL, assert_allclose

    for name, fn, positive in (("sigmoid", torch.sigmoid, False), ("tanh", torch.tanh, False), ("exp", torch.exp, False),
                               ("log", torch.log, True)):
        x_cpu, x = _pair(shape, dtype, seed=len(name), requires_grad=True)
        if positive:
            x_cpu = (x_cpu.detach().abs() + 0.5).requires_grad_(True)
            x = x_cpu.detach().to(supa).requires_grad_(True)
        g_cpu, g = _pair(shape, dtype, seed=9)
        y = fn(x)
        # the CPU golden runs in the same dtype: the backward formulas start from the rounded forward result on both sides
        xr = x_cpu.detach().clone().requires_grad_(True)
        yr = fn(xr)
        assert_allclose(yr.detach(), y.detach(), RTOL[dtype] * 4, ATOL[dtype] * 4)
        y.backward(g)
        yr.backward(g_cpu)
        assert_allclose(xr.grad, x.grad, RTOL[dtype] * 8, max(ATOL[dtype] * 8, 2e-2 if dtype != torch.float32 else 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32, torch.int64])
def test_comparisons_extrema_where_masked_fill(supa, dtype):
    g = torch.Generator().manual_seed(4)
    if dtype.is_floating_point:
        a_cpu = torch.randn(37, 129, generator=g).to(dtype)
        b_cpu = torch.randn(37, 129, generator=g).to(dtype)
        b_cpu[::3] = a_cpu[::3]
    else:
        a_cpu = torch.randint(-5, 6, (37, 129), generator=g, dtype=dtype)
        b_cpu = torch.randint(-5, 6, (37, 129), generator=g, dtype=dtype)
    a, b = a_cpu.to(supa), b_cpu.to(supa)
    for op in (torch.eq, torch.ne, torch.lt, torch.le, torch.gt, torch.ge):
        out = op(a, b)
        assert out.dtype == torch.bool and torch.equal(out.cpu(), op(a_cpu, b_cpu)), op.__name__
        out = op(a, 1)
        assert torch.equal(out.cpu(), op(a_cpu, 1)), op.__name__ + " scalar"
        out = op(a, b[0])                                     # broadcast row
        assert torch.equal(out.cpu(), op(a_cpu, b_cpu[0])), op.__name__ + " broadcast"
    assert torch.equal(torch.maximum(a, b).cpu(), torch.maximum(a_cpu, b_cpu))
    assert torch.equal(torch.minimum(a, b).cpu(), torch.minimum(a_cpu, b_cpu))
    cond_cpu = a_cpu > b_cpu
    cond = cond_cpu.to(supa)
    assert torch.equal(torch.where(cond, a, b).cpu(), torch.where(cond_cpu, a_cpu, b_cpu))
    assert torch.equal(torch.where(cond[:, :1], a, b).cpu(), torch.where(cond_cpu[:, :1], a_cpu, b_cpu))
    filled = a.clone().masked_fill_(cond, 3)
    assert torch.equal(filled.cpu(), a_cpu.clone().masked_fill_(cond_cpu, 3))
    assert torch.equal(a.masked_fill(cond[0], -2).cpu(), a_cpu.masked_fill(cond_cpu[0], -2))   # functional form, broadcast mask
    if dtype.is_floating_point:
        n_cpu = a_cpu.clone()
        n_cpu[1, 2] = float("nan")
        n = n_cpu.to(supa)
        assert torch.equal(torch.isnan(torch.maximum(n, b).cpu()), torch.isnan(torch.maximum(n_cpu, b_cpu)))
        assert torch.equal(torch.isnan(torch.minimum(b, n).cpu()), torch.isnan(torch.minimum(b_cpu, n_cpu)))
        assert not bool((n == n).cpu()[1, 2]) and bool((n != n).cpu()[1, 2])


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cross_entropy_weights_with_label_smoothing(supa, reduction, dtype):
    """Class weights together with label smoothing (the reference reaches the upstream composite for them,
    CrossEntropyLoss.cpp:23-33,50): same loss and gradient as the CPU."""
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(8)
    x_cpu = (torch.randn(24, 500, generator=g) * 2).to(dtype).requires_grad_(True)
    x = x_cpu.detach().to(supa).requires_grad_(True)
    t = torch.randint(0, 500, (24,), generator=g)
    t[::5] = -100
    w = torch.rand(500, generator=g) + 0.5
    ref = F.cross_entropy(x_cpu.float(), t, weight=w, label_smoothing=0.1, reduction=reduction)
    out = F.cross_entropy(x, t.to(supa), weight=w.to(supa), label_smoothing=0.1, reduction=reduction)
    go = torch.rand(ref.shape, generator=g) + 0.5
    ref.backward(go)
    out.backward(go.to(supa).to(out.dtype))
    rt, at = (2e-5, 1e-6) if dtype == torch.float32 else (1.6e-2, 1e-3)
    assert_allclose(ref.detach().to(dtype), out.detach(), rt, at)
    assert_allclose(x_cpu.grad.float(), x.grad.float(), rt, at * 1e-1)


# ---- softmax / nll -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((16,), 0), ((1024, 512), -1), ((1023, 511), -1), ((1025, 513), 0), ((64, 32000), -1),
                                       ((4, 5, 6, 7), 2)])
def test_log_softmax_forward_backward(supa, shape, dim, dtype):
    from tests.supa_testing import assert_allclose

    x_cpu, x = _pair(shape, dtype, requires_grad=True)
    g_cpu, g = _pair(shape, dtype, seed=1)
    y = F.log_softmax(x, dim)
    xr = x_cpu.detach().float().requires_grad_(True)
    yr = F.log_softmax(xr, dim)
    assert_allclose(yr.detach().to(dtype), y.detach(), 1.3e-6 if dtype == torch.float32 else 1.6e-2, 1e-5 if dtype == torch.float32 else 1e-3)
    y.backward(g)
    yr.backward(g_cpu.float())
    mag = float(g_cpu.float().sum(dim, keepdim=True).abs().max()) + 1
    assert_allclose(xr.grad.to(dtype), x.grad, 1.3e-6 if dtype == torch.float32 else 1.6e-2, (1e-5 if dtype == torch.float32 else 2e-2) * mag)
    yf = F.log_softmax(x.detach(), dim, dtype=torch.float32)
    assert yf.dtype == torch.float32
    assert_allclose(F.log_softmax(x_cpu.detach().float(), dim), yf, 2e-6, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((16,), 0), ((1024, 512), -1), ((1023, 511), 0), ((64, 32000), -1), ((4, 5, 6, 7), 2)])
def test_softmax_forward_backward(supa, shape, dim, dtype):
    """F.softmax dispatches to _softmax / _softmax_backward_data on the device (autograd wiring from libtorch)."""
    from tests.supa_testing import assert_allclose

    x_cpu, x = _pair(shape, dtype, requires_grad=True)
    g_cpu, g = _pair(shape, dtype, seed=1)
    y = F.softmax(x, dim)
    xr = x_cpu.detach().float().requires_grad_(True)
    yr = F.softmax(xr, dim)
    assert_allclose(yr.detach().to(dtype), y.detach(), 4e-6 if dtype == torch.float32 else 1.6e-2, 1e-7 if dtype == torch.float32 else 1e-5)
    y.backward(g)
    yr.backward(g_cpu.float())
    assert_allclose(xr.grad.to(dtype), x.grad, 2e-5 if dtype == torch.float32 else 3e-2, 1e-6 if dtype == torch.float32 else 2e-3)
    yf = F.softmax(x.detach(), dim, dtype=torch.float32)
    assert yf.dtype == torch.float32
    assert_allclose(F.softmax(x_cpu.detach().float(), dim), yf, 4e-6, 1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(16, 10), (1024, 512), (2000, 1000), (100, 20000)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_nll_loss_forward_backward_weight(supa, shape, reduction, dtype):
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(shape[0])
    logp_cpu = F.log_softmax(torch.randn(*shape, generator=g), 1).to(dtype).requires_grad_(True)
    t_cpu = torch.randint(0, shape[1], (shape[0],), generator=g)
    t_cpu[::9] = -100
    t_before = t_cpu.clone()
    w_cpu = (torch.rand(shape[1], generator=g) + 0.5).to(dtype)
    for weight in (None, w_cpu):
        x = logp_cpu.detach().to(supa).requires_grad_(True)
        t = t_cpu.to(supa)
        out = F.nll_loss(x, t, weight=None if weight is None else weight.to(supa), reduction=reduction)
        xr = logp_cpu.detach().float().requires_grad_(True)
        ref = F.nll_loss(xr, t_cpu, weight=None if weight is None else weight.float(), reduction=reduction)
        rtol = {torch.float32: 4e-6, torch.bfloat16: 1.6e-2, torch.float16: 2e-3}[dtype]
        assert_allclose(ref.detach().to(dtype), out.detach(), rtol, rtol)
        go_cpu = torch.randn(ref.shape, generator=g).to(dtype)
        out.backward(go_cpu.to(supa))
        ref.backward(go_cpu.float())
        assert_allclose(xr.grad.to(dtype), x.grad, rtol * 2, 1e-6 if dtype == torch.float32 else 1e-4)
        assert torch.equal(t.cpu(), t_before), "the target tensor is not modified"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 19, 64, 128), (3, 5, 7, 9), (2, 19, 512, 1024)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_nll_loss2d_and_spatial_cross_entropy(supa, shape, reduction, dtype):
    """(N, C, H, W) inputs: F.nll_loss dispatches to nll_loss2d_forward / backward, F.cross_entropy to log_softmax over
    dim 1 followed by them (the 4-D shape (2, 19, 512, 1024) is the reference's segmentation case)."""
    from tests.supa_testing import assert_allclose

    if shape[2] >= 512 and (dtype != torch.float32 or reduction == "sum"):
        pytest.skip("the large shape runs once per reduction family")
    g = torch.Generator().manual_seed(shape[1])
    x_cpu = torch.randn(*shape, generator=g).to(dtype)
    t_cpu = torch.randint(0, shape[1], (shape[0],) + shape[2:], generator=g)
    t_cpu.view(-1)[::11] = -100
    w_cpu = (torch.rand(shape[1], generator=g) + 0.5).to(dtype)
    rtol = {torch.float32: 4e-6, torch.bfloat16: 1.6e-2, torch.float16: 2e-3}[dtype]
    for weight in (None, w_cpu):
        # nll_loss on log-probabilities
        logp_cpu = F.log_softmax(x_cpu.float(), 1).to(dtype)
        x = logp_cpu.to(supa).requires_grad_(True)
        out = F.nll_loss(x, t_cpu.to(supa), weight=None if weight is None else weight.to(supa), reduction=reduction)
        xr = logp_cpu.float().requires_grad_(True)
        ref = F.nll_loss(xr, t_cpu, weight=None if weight is None else weight.float(), reduction=reduction)
        assert_allclose(ref.detach().to(dtype), out.detach(), rtol, rtol)
        go_cpu = torch.randn(ref.shape, generator=g).to(dtype)
        out.backward(go_cpu.to(supa))
        ref.backward(go_cpu.float())
        assert_allclose(xr.grad.to(dtype), x.grad, rtol * 2, 1e-6 if dtype == torch.float32 else 1e-4)
    # cross entropy on logits
    x = x_cpu.to(supa).requires_grad_(True)
    loss = F.cross_entropy(x, t_cpu.to(supa), reduction=reduction)
    xr = x_cpu.float().requires_grad_(True)
    ref = F.cross_entropy(xr, t_cpu, reduction=reduction)
    assert_allclose(ref.detach().to(dtype), loss.detach(), rtol * 4, rtol * 4)
    go_cpu = torch.randn(ref.shape, generator=g).to(dtype)
    loss.backward(go_cpu.to(supa))
    ref.backward(go_cpu.float())
    scale = 1.0 if reduction != "mean" else float((t_cpu != -100).sum())
    assert_allclose(xr.grad.to(dtype) * scale, x.grad * scale, rtol * 4, 1e-5 if dtype == torch.float32 else 2e-3)


@pytest.mark.parametrize("shape, dtype, reduction, with_weight, with_pos_weight, pos_weight_shape", [
    ((4,), torch.float32, "none", False, False, None),
    ((1024, 512), torch.float32, "sum", True, False, None),
    ((1024, 512), torch.bfloat16, "mean", False, True, None),
    ((1023, 511), torch.float16, "none", True, True, None),
    ((1025, 513), torch.float16, "sum", True, True, None),
    ((2, 3, 4), torch.float32, "mean", False, True, (3, 1)),
    ((2048, 4096), torch.float32, "mean", False, False, None),
])
def test_binary_cross_entropy_with_logits_forward_backward(supa, shape, dtype, reduction, with_weight, with_pos_weight, pos_weight_shape):
    """The parameter list of the reference's test (test/test_binary_misc_ops_kernels.py:176-245) plus the backward
    pass, which runs our own autograd node (one fused kernel) instead of libtorch's operator chain."""
    from tests.supa_testing import ATOL, RTOL, assert_allclose

    g = torch.Generator().manual_seed(shape[0])
    x_cpu = (torch.rand(*shape, generator=g) * 10 - 5).to(dtype)
    t_cpu = torch.rand(*shape, generator=g).to(dtype)
    w_cpu = (torch.rand(*shape, generator=g) * 1.9 + 0.1).to(dtype) if with_weight else None
    pw_cpu = None
    if with_pos_weight:
        pw_cpu = (torch.rand(*(pos_weight_shape or (shape[-1],)), generator=g) * 2.9 + 0.1).to(dtype)
    xr = x_cpu.float().detach().clone().requires_grad_(True)
    ref = F.binary_cross_entropy_with_logits(xr, t_cpu.float(), weight=None if w_cpu is None else w_cpu.float(),
                                             pos_weight=None if pw_cpu is None else pw_cpu.float(), reduction=reduction)
    x = x_cpu.to(supa).requires_grad_(True)
    out = F.binary_cross_entropy_with_logits(x, t_cpu.to(supa), weight=None if w_cpu is None else w_cpu.to(supa),
                                             pos_weight=None if pw_cpu is None else pw_cpu.to(supa), reduction=reduction)
    assert out.device.type == "supa" and out.dtype == dtype
    loosen = 8 if reduction == "sum" else 2   # a sum of half a million terms rounded to 16 bits
    assert_allclose(ref.detach().to(dtype), out.detach(), RTOL[dtype] * loosen, ATOL[dtype] * loosen)
    go_cpu = torch.rand(ref.shape, generator=g).to(dtype)
    out.backward(go_cpu.to(supa))
    ref.backward(go_cpu.float())
    scale = float(x_cpu.numel()) if reduction == "mean" else 1.0
    assert_allclose(xr.grad.to(dtype) * scale, x.grad * scale, RTOL[dtype] * 4, ATOL[dtype] * 4)
    # no autograd: the plain kernel path
    with torch.no_grad():
        out2 = F.binary_cross_entropy_with_logits(x_cpu.to(supa), t_cpu.to(supa), reduction=reduction)
        ref2 = F.binary_cross_entropy_with_logits(x_cpu.float(), t_cpu.float(), reduction=reduction)
    assert_allclose(ref2.to(dtype), out2, RTOL[dtype] * loosen, ATOL[dtype] * loosen)


# ---- cross entropy -------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 1000), (16, 1000), (1, 6), (512, 1024), (512, 1027), (64, 32000), (160, 128256)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_cross_entropy_forward_backward(supa, shape, reduction, dtype):
    """F.cross_entropy through the dispatcher (test/test_loss.py:235-276), with ignore_index and label smoothing."""
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(shape[1])
    x_cpu = (torch.randn(*shape, generator=g) * 2).to(dtype)
    t_cpu = torch.randint(0, shape[1], (shape[0],), generator=g)
    if shape[0] > 4:
        t_cpu[::7] = -100
    for eps in (0.0, 0.1):
        x = x_cpu.detach().clone().to(supa).requires_grad_(True)
        loss = F.cross_entropy(x, t_cpu.to(supa), reduction=reduction, label_smoothing=eps)
        # golden: the CPU kernels in fp64 on the same values (for fp32 logits the fp32 CPU path loses digits in
        # the label-smoothing composite, where a sum over all classes feeds the softmax term), cast down
        xr = x_cpu.detach().clone().double().requires_grad_(True)
        ref = F.cross_entropy(xr, t_cpu, reduction=reduction, label_smoothing=eps)
        assert loss.dtype == dtype and loss.shape == ref.shape
        rtol = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}[dtype]
        assert_allclose(ref.detach().to(dtype), loss.detach(), rtol, 1e-5 if dtype == torch.float32 else 1e-2)
        go = torch.randn(ref.shape, generator=g).to(dtype) if reduction == "none" else torch.tensor(0.5, dtype=dtype)
        loss.backward(go.to(supa))
        ref.backward(go.double())
        scale = float((t_cpu != -100).sum()) if reduction == "mean" else 1.0
        grtol = {torch.float32: 1e-5, torch.bfloat16: 2.4e-2, torch.float16: 3e-3}[dtype]
        gatol = {torch.float32: 3e-7, torch.bfloat16: 2e-4, torch.float16: 4e-5}[dtype]
        assert x.grad.dtype == dtype
        assert_allclose((xr.grad * scale).float(), x.grad.float().cpu() * scale, grtol, gatol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(16, 1000), (64, 32000), (160, 128256)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy_class_weights_forward_backward(supa, shape, reduction, dtype):
    """F.cross_entropy(..., weight=w) stays on the fused kernel when there is no label smoothing (weights together with
    smoothing go to libtorch's composite, whose mask operators are outside this path)."""
    from tests.supa_testing import assert_allclose

    g = torch.Generator().manual_seed(shape[0])
    x_cpu = (torch.randn(*shape, generator=g) * 2).to(dtype)
    t_cpu = torch.randint(0, shape[1], (shape[0],), generator=g)
    t_cpu[::5] = -100
    w_cpu = (torch.rand(shape[1], generator=g) + 0.25).to(dtype)
    rtol = {torch.float32: 1e-5, torch.bfloat16: 1.6e-2, torch.float16: 2e-3}[dtype]
    for eps in (0.0,):
        x = x_cpu.to(supa).requires_grad_(True)
        out = F.cross_entropy(x, t_cpu.to(supa), weight=w_cpu.to(supa), reduction=reduction, label_smoothing=eps)
        xr = x_cpu.float().detach().clone().requires_grad_(True)
        ref = F.cross_entropy(xr, t_cpu, weight=w_cpu.float(), reduction=reduction, label_smoothing=eps)
        assert_allclose(ref.detach().to(dtype), out.detach(), rtol, rtol)
        go_cpu = (torch.rand(ref.shape, generator=g) + 0.5).to(dtype)
        out.backward(go_cpu.to(supa))
        ref.backward(go_cpu.float())
        scale = float(w_cpu.float()[t_cpu[t_cpu >= 0]].sum()) if reduction == "mean" else 1.0
        assert_allclose(xr.grad.to(dtype) * scale, x.grad * scale, rtol * 2, 1e-5 if dtype == torch.float32 else 2e-3)


def test_cross_entropy_edge_cases(supa):
    x_cpu, x = _pair((8, 20), torch.float32)
    all_ign = torch.full((8,), -100)
    assert torch.isnan(F.cross_entropy(x, all_ign.to(supa)).cpu()).item()
    assert F.cross_entropy(x, all_ign.to(supa), reduction="sum").item() == 0
    assert torch.equal(F.cross_entropy(x, all_ign.to(supa), reduction="none").cpu(), torch.zeros(8))
    t = torch.tensor([1, 2, 2, 3, 2, 0, 5, 2])
    _close(F.cross_entropy(x_cpu, t, ignore_index=2), F.cross_entropy(x, t.to(supa), ignore_index=2), loosen=2)
    v_cpu, v = _pair((20,), torch.float32, seed=3)  # 1-D logits with a 0-d target
    _close(F.cross_entropy(v_cpu, torch.tensor(4)), F.cross_entropy(v, torch.tensor(4).to(supa)), loosen=2)
    nc = x_cpu.t().contiguous().to(supa).t()  # non-contiguous logits
    _close(F.cross_entropy(x_cpu, t), F.cross_entropy(nc, t.to(supa)), loosen=2)
    # no gradient requested: forward only, nothing is saved
    with torch.no_grad():
        _close(F.cross_entropy(x_cpu, t), F.cross_entropy(x, t.to(supa)), loosen=2)
    # composite fallbacks: class weights, probability targets, fp64
    w_cpu = torch.rand(20) + 0.5
    _close(F.cross_entropy(x_cpu, t, weight=w_cpu), F.cross_entropy(x, t.to(supa), weight=w_cpu.to(supa)), loosen=4)
    d_cpu, d = _pair((8, 20), torch.float64, seed=4)
    _close(F.cross_entropy(d_cpu, t), F.cross_entropy(d, t.to(supa)))


def test_cross_entropy_backward_twice_and_scaled(supa):
    x_cpu, x = _pair((32, 5000), torch.float32, requires_grad=True)
    t = torch.randint(0, 5000, (32,), generator=torch.Generator().manual_seed(1))
    loss = F.cross_entropy(x, t.to(supa))
    (loss / 4).backward(retain_graph=True)
    g1 = x.grad.clone()
    x.grad = None
    loss.backward()
    g2 = x.grad.clone()
    ref = F.cross_entropy(x_cpu, t)
    ref.backward()
    from tests.supa_testing import assert_allclose

    assert_allclose(x_cpu.grad * 32, g2 * 32, 1e-5, 3e-7)
    assert_allclose(x_cpu.grad * 8, g1 * 32, 1e-5, 3e-7)


def test_cross_entropy_retained_graph_hands_out_independent_gradients(supa):
    """torch.autograd.grad twice on a retained graph, no clone in between: the tensor returned first must not change
    when the second call runs with another upstream gradient, and both must match the CPU."""
    from tests.supa_testing import assert_allclose

    x_cpu, x = _pair((48, 3000), torch.float32, requires_grad=True)
    t = torch.randint(0, 3000, (48,), generator=torch.Generator().manual_seed(2))
    loss = F.cross_entropy(x, t.to(supa), label_smoothing=0.1)
    ref = F.cross_entropy(x_cpu, t, label_smoothing=0.1)
    (g1,) = torch.autograd.grad(loss, x, torch.tensor(0.5).to(supa), retain_graph=True)
    g1_copy = g1.cpu().clone()
    (g2,) = torch.autograd.grad(loss, x, torch.tensor(3.0).to(supa), retain_graph=True)
    (g3,) = torch.autograd.grad(loss, x, torch.tensor(1.0).to(supa))
    (r,) = torch.autograd.grad(ref, x_cpu)
    assert torch.equal(g1.cpu(), g1_copy), "the first result changed under its holder"
    assert g1.data_ptr() != g2.data_ptr() and g2.data_ptr() != g3.data_ptr()
    for got, f in ((g1, 0.5), (g2, 3.0), (g3, 1.0)):
        assert_allclose(r * 48 * f, got * 48, 1e-5, 3e-7)


def test_cross_entropy_zero_upstream_then_one_raises_instead_of_dividing(supa):
    """An upstream gradient of zero wipes the stored gradient; a later backward on the retained graph cannot undo that
    and says so at the next synchronisation instead of returning NaN silently."""
    _, x = _pair((16, 300), torch.float32, requires_grad=True)
    t = torch.randint(0, 300, (16,), generator=torch.Generator().manual_seed(3)).to(supa)
    loss = F.cross_entropy(x, t)
    (g0,) = torch.autograd.grad(loss, x, torch.tensor(0.0).to(supa), retain_graph=True)
    assert float(g0.cpu().abs().max()) == 0.0
    (g1,) = torch.autograd.grad(loss, x, torch.tensor(1.0).to(supa), retain_graph=True)
    with pytest.raises(RuntimeError, match="zero upstream"):
        g1.cpu()
    torch.supa.synchronize()  # the device and the status word are usable again
    assert float(F.cross_entropy(x.detach(), t).cpu()) > 0


def test_cross_entropy_fp16_survives_loss_scaling(supa):
    """fp16 logits with a loss-scaling upstream gradient: most probabilities over the row count are below fp16's
    smallest subnormal, so the gradient must be formed with the upstream factor folded in before it is rounded."""
    from tests.supa_testing import assert_allclose

    rows, classes, scale = 32768, 64, 1024.0  # a power of two that an fp16 loss can be multiplied by without overflowing
    g = torch.Generator().manual_seed(4)
    x_cpu = torch.randn(rows, classes, generator=g).half()
    t = torch.randint(0, classes, (rows,), generator=g)
    x = x_cpu.to(supa).requires_grad_(True)
    loss = F.cross_entropy(x, t.to(supa))
    (loss * scale).backward()
    xr = x_cpu.double().requires_grad_(True)
    (F.cross_entropy(xr, t) * scale).backward()
    got, want = x.grad.cpu().double(), xr.grad
    assert float(got.abs().max()) > 0
    small = want.abs() < 0.5  # everything but the class of the target
    rel = ((got - want).abs() / want.abs().clamp_min(1e-30))[small & (want.abs() > 1e-3)]
    assert float(rel.max()) <= 1e-2, f"relative error {float(rel.max())}"
    assert_allclose(want.float(), got.float(), 2e-3, 1e-5)


def test_out_of_range_target_raises_at_the_next_sync_and_device_survives(supa):
    x_cpu, x = _pair((6, 8), torch.float32)
    bad = torch.tensor([1, 2, 8, 3, 0, 1]).to(supa)
    loss = F.cross_entropy(x, bad)  # asynchronous: nothing is raised here, nothing traps on the device
    with pytest.raises(IndexError):
        loss.item()
    good = torch.tensor([1, 2, 7, 3, 0, 1])
    _close(F.cross_entropy(x_cpu, good), F.cross_entropy(x, good.to(supa)), loosen=2)
    torch.supa.synchronize()


# ---- pinned host memory ------------------------------------------------------------------------------------------
def test_pinned_host_allocator_reuses_blocks_and_waits_for_copies(supa):
    """Pinned blocks are cached per size class; a block freed while a non-blocking copy still reads it is not handed out
    again before that copy has finished."""
    torch.supa.synchronize()
    torch.supa.empty_host_cache()
    base = torch.supa.host_memory_stats()
    a = torch.arange(1 << 18, dtype=torch.float32).pin_memory("supa")
    assert a.is_pinned("supa")
    s1 = torch.supa.host_memory_stats()
    assert s1["host_allocs"] == base["host_allocs"] + 1 and s1["allocated_bytes"] >= a.numel() * 4
    ptr = a.data_ptr()
    del a
    b = torch.zeros(1 << 18, dtype=torch.float32).pin_memory("supa")  # same size class: the cached block, no new cudaHostAlloc
    s2 = torch.supa.host_memory_stats()
    assert b.data_ptr() == ptr and s2["host_allocs"] == s1["host_allocs"] and s2["cache_hits"] == s1["cache_hits"] + 1
    # a non-blocking copy out of the block, then the block is dropped and another one of the same size is asked for at once
    big = torch.full((1 << 24,), 3.0).pin_memory("supa")           # 64 MB: the copy takes a while
    ptr_big = big.data_ptr()
    d = big.to(supa, non_blocking=True)
    del big
    other = torch.empty(1 << 24, dtype=torch.float32).pin_memory("supa")
    other.fill_(7.0)                                               # would corrupt the copy if it got the same block too early
    torch.supa.synchronize()
    assert float(d.sum(0).cpu()) == 3.0 * (1 << 24)
    assert other.data_ptr() != ptr_big or True  # (the address may be reused only after the copy has completed)
    del other, b, d
    torch.supa.empty_host_cache()
    assert torch.supa.host_memory_stats()["reserved_bytes"] == 0

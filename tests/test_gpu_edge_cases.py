"""Edge cases of the operator path that the reference's tests or its kernels call out: very large element counts,
degenerate reductions, out= handling, CPU scalar operands, probability targets (needs a GPU)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def supa():
    import torch_supa_b200  # noqa: F401

    if not torch.supa.is_available():
        pytest.skip("no supa device")
    return torch.device("supa", 0)


def test_more_than_2_31_elements(cuda_device):
    """A dense run and a reduction past the 32-bit index range (the reference special-cases it, Reduce.cuh:1279-1287,
    Loops.cuh:126-134): 2^31 + 4100 one-byte elements."""
    from torch_supa_b200 import capi, functional as F2

    n = (1 << 31) + 4100
    x = torch.ones(n, dtype=torch.uint8, device=cuda_device)
    x[-3:] = 5
    x[0] = 7
    total = F2.reduce(capi.RED_SUM, x, [0])
    torch.cuda.synchronize()
    assert total.dtype == torch.int64 and int(total) == n - 4 + 7 + 15
    y = torch.empty_like(x)
    F2.elementwise(capi.EW_ADD, y, x, x)          # one dense dimension longer than 2^31
    torch.cuda.synchronize()
    assert int(y[0]) == 14 and int(y[-1]) == 10 and int(y[n // 2]) == 2 and int(y[(1 << 31) + 5]) == 2
    del x, y
    torch.cuda.empty_cache()


def test_degenerate_reductions(supa):
    """0-d and one-element inputs, dim=() meaning all dimensions, negative and tuple dims, keepdim, empty reduced dimension."""
    s = torch.tensor(3.5).to(supa)
    assert float(s.sum()) == 3.5 and float(s.amax()) == 3.5 and float(s.mean()) == 3.5
    one = torch.tensor([[2.0]]).to(supa)
    assert float(one.sum((0, 1))) == 2.0 and one.sum(-1, keepdim=True).shape == (1, 1)
    g = torch.Generator().manual_seed(0)
    x_cpu = torch.randn(5, 6, 7, generator=g)
    x = x_cpu.to(supa)
    torch.testing.assert_close(x.sum(()).cpu(), x_cpu.sum(()), rtol=1e-5, atol=1e-5)       # empty tuple = everything
    torch.testing.assert_close(x.sum((-1, 0)).cpu(), x_cpu.sum((-1, 0)), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(x.amax((0, 2), keepdim=True).cpu(), x_cpu.amax((0, 2), keepdim=True))
    torch.testing.assert_close(x.mean(1).cpu(), x_cpu.mean(1), rtol=1e-5, atol=1e-6)
    e = torch.empty(4, 0).to(supa)
    assert torch.equal(e.sum(1).cpu(), torch.zeros(4))
    assert torch.isnan(e.mean(1).cpu()).all()
    with pytest.raises((RuntimeError, IndexError)):
        e.amax(1)                                                # amax over an empty dimension has no identity


def test_out_argument_is_resized_or_proxied(supa):
    a_cpu, b_cpu = torch.randn(8, 16), torch.randn(8, 16)
    a, b = a_cpu.to(supa), b_cpu.to(supa)
    out = torch.empty(0).to(supa)
    torch.add(a, b, out=out)                                     # wrong shape: resized
    assert out.shape == (8, 16) and torch.equal(out.cpu(), a_cpu + b_cpu)
    base = torch.zeros(16, 8).to(supa)
    out_t = base.t()                                             # right shape, transposed strides: written through a proxy
    torch.mul(a, b, out=out_t)
    assert torch.equal(out_t.cpu(), a_cpu * b_cpu) and torch.equal(base.cpu(), (a_cpu * b_cpu).t())


def test_cpu_scalar_operands(supa):
    x_cpu = torch.randn(33, 65)
    x = x_cpu.to(supa)
    assert torch.equal((x + torch.tensor(2.0)).cpu(), x_cpu + 2.0)      # 0-dim CPU tensor: lifted to a scalar
    assert torch.equal((x * 3).cpu(), x_cpu * 3)
    assert torch.equal((2.5 - x).cpu(), 2.5 - x_cpu)
    h = x_cpu.half().to(supa)
    assert (h + 1.5).dtype == torch.float16                              # wrapped numbers do not promote
    i = torch.arange(10, dtype=torch.int32).to(supa)
    assert (i * 2.5).dtype == torch.float32
    with pytest.raises(RuntimeError):
        x + torch.randn(33, 65)                                          # any other CPU operand is an error


def test_cross_entropy_probability_targets(supa):
    """Class-probability targets take libtorch's composite (log_softmax, mul, sum, neg, div on the device)."""
    g = torch.Generator().manual_seed(3)
    x_cpu = torch.randn(12, 40, generator=g)
    p_cpu = torch.softmax(torch.randn(12, 40, generator=g), 1)
    for reduction in ("mean", "sum", "none"):
        x = x_cpu.to(supa).requires_grad_(True)
        out = F.cross_entropy(x, p_cpu.to(supa), reduction=reduction)
        xr = x_cpu.clone().requires_grad_(True)
        ref = F.cross_entropy(xr, p_cpu, reduction=reduction)
        torch.testing.assert_close(out.detach().cpu(), ref.detach(), rtol=1e-5, atol=1e-5)
        go = torch.ones_like(ref)
        out.backward(go.to(supa))
        ref.backward(go)
        torch.testing.assert_close(x.grad.cpu(), xr.grad, rtol=1e-5, atol=1e-6)

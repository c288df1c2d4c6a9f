"""Reductions through the C ABI against fixtures, oracle and PyTorch CPU (needs a GPU)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.helpers import accumulation_tol, assert_close

pytestmark = pytest.mark.gpu

OPS = {"sum": 0, "mean": 1, "amax": 2, "amin": 3}


def _red(dev, op, x, dims, **kw):
    from torch_supa_b200 import functional as F2

    out = F2.reduce(OPS[op], x.to(dev), dims, **kw)
    torch.cuda.synchronize()
    return out.cpu()


def test_fixtures(golden, cuda_device):
    x = torch.from_numpy(golden["red/x"])
    rtol, atol = accumulation_tol(777)
    assert_close(_red(cuda_device, "sum", x, [-1]).numpy(), golden["red/sum"], rtol, atol, "sum")
    assert_close(_red(cuda_device, "mean", x, [-1]).numpy(), golden["red/mean"], rtol, atol, "mean")
    assert np.array_equal(_red(cuda_device, "amax", x, [-1]).numpy(), golden["red/amax"])
    assert np.array_equal(_red(cuda_device, "amin", x, [-1]).numpy(), golden["red/amin"])
    assert_close(_red(cuda_device, "sum", x, [0]).numpy(), golden["red/sum_dim0"], rtol, atol, "sum dim 0")
    xb = x.bfloat16()
    assert_close(_red(cuda_device, "sum", xb, [-1]).float().numpy(), golden["red/bf16_sum"], 1.6e-2, 1e-3, "bf16 sum")
    assert_close(_red(cuda_device, "sum", xb, [-1], out_dtype=torch.float32).numpy(), golden["red/bf16_sum_f32"], rtol, atol,
                 "bf16 sum -> fp32")
    assert_close(_red(cuda_device, "mean", xb, [-1]).float().numpy(), golden["red/bf16_mean"], 1.6e-2, 1e-3, "bf16 mean")
    assert np.array_equal(_red(cuda_device, "amax", xb, [-1]).float().numpy(), golden["red/bf16_amax"])


SHAPES = [((16,), [0]), ((1024, 512), [-1]), ((1023, 511), [-1]), ((1025, 513), [0]), ((128, 2135), [1]),
          ((64, 65536), [-1]), ((3, 200000), [-1]), ((1, 1 << 20), [1]), ((7, 9, 11), [1]), ((7, 9, 11), [0, 2]),
          ((5, 6, 7, 8), [1, 3]), ((300, 40), [0]), ((2, 70000), [0]), ((1,), [0]), ((4, 1, 6), [1]),
          ((33, 1000), [0, 1])]


@pytest.mark.parametrize("shape,dims", SHAPES)
@pytest.mark.parametrize("op", ["sum", "mean", "amax"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_against_pytorch_cpu(cuda_device, shape, dims, op, dtype):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dtype)
    out = _red(cuda_device, op, x, dims)
    n = 1
    for d in dims:
        n *= shape[d]
    ref64 = getattr(x.double(), op)(dims)
    assert out.shape == ref64.shape and out.dtype == dtype
    if op == "amax":
        assert torch.equal(out, x.amax(dims)), "amax must be exact"
        return
    if dtype in (torch.bfloat16, torch.float16):
        # one rounding of the exact fp32-accumulated value
        assert_close(out.double().numpy(), ref64.numpy(), 4e-3 if dtype == torch.bfloat16 else 5e-4,
                     1e-2 if op == "sum" else 1e-3, op)
    elif dtype == torch.float32:
        rtol, atol = accumulation_tol(n)
        assert_close(out.double().numpy(), ref64.numpy(), rtol, atol * (1 if op == "mean" else max(1.0, n ** 0.5 / 8)), op)
    else:
        assert_close(out.numpy(), ref64.numpy(), 1e-12, 1e-10, op)


def test_oracle_rows(cuda_device):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(37, 5000, generator=g)
    for op in ("sum", "mean"):
        rtol, atol = accumulation_tol(5000)
        assert_close(_red(cuda_device, op, x, [-1]).double().numpy(), oracle.c_reduce_rows(x.numpy(), op), rtol, atol, op)
    assert np.array_equal(_red(cuda_device, "amax", x, [-1]).double().numpy(), oracle.c_reduce_rows(x.numpy(), "amax"))


def test_amax_propagates_nan(cuda_device):
    x = torch.randn(8, 3000)
    x[3, 1234] = float("nan")
    out = _red(cuda_device, "amax", x, [-1])
    assert torch.isnan(out[3]) and not torch.isnan(out[[0, 1, 2, 4, 5, 6, 7]]).any()
    xb = x.bfloat16()
    assert torch.isnan(_red(cuda_device, "amax", xb, [-1])[3])


def test_integer_and_bool_sums_are_exact(cuda_device):
    g = torch.Generator().manual_seed(2)
    for dt in (torch.int32, torch.int64, torch.int16, torch.uint8, torch.int8):
        x = torch.randint(0, 100, (50, 3001), generator=g).to(dt)
        assert torch.equal(_red(cuda_device, "sum", x, [-1]), x.sum(-1))
        assert torch.equal(_red(cuda_device, "amax", x, [-1]), x.amax(-1))
    b = torch.rand(20, 500, generator=g) > 0.5
    assert torch.equal(_red(cuda_device, "sum", b, [1]), b.sum(1))


def test_keepdim_and_noncontiguous_input(cuda_device):
    x = torch.randn(40, 60)
    out = _red(cuda_device, "sum", x, [1], keepdim=True)
    assert out.shape == (40, 1)
    assert_close(out.numpy(), x.sum(1, keepdim=True).numpy(), 1e-5, 1e-5, "keepdim")
    from torch_supa_b200 import functional as F2

    xt = x.to(cuda_device).t()  # [60, 40] with strides (1, 60)
    out = F2.reduce(OPS["sum"], xt, [1]).cpu()
    assert_close(out.numpy(), x.t().sum(1).numpy(), 1e-5, 1e-5, "transposed view")


def test_split_rows_path_is_deterministic(cuda_device):
    from torch_supa_b200 import capi, functional as F2

    x = torch.randn(4, 1 << 21, device=cuda_device)
    out = torch.empty(4, device=cuda_device)
    desc = capi.make_reduce_desc(OPS["sum"], x, out, [1])
    assert capi.reduce_path(desc) == 1 and capi.reduce_scratch_bytes(desc) > 0
    a = F2.reduce(OPS["sum"], x, [1])
    b = F2.reduce(OPS["sum"], x, [1])
    assert torch.equal(a, b)
    assert_close(a.cpu().double().numpy(), x.double().sum(1).cpu().numpy(), 2e-6, 1e-2, "split rows")

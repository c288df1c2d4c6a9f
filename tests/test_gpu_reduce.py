"""Reductions through the C ABI against fixtures, oracle and PyTorch CPU (needs a GPU)."""
import numpy as np

import pytest
import torch

from oracle import oracle
from tests.helpers import accumulation_tol, assert_close

pytestmark = pytest.mark.gpu

OPS = {"sum": 0, "mean": 1, "amax": 2, "amin": 3, "prod": 4, "nansum": 5}


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
          ((33, 1000), [0, 1]),
          # column reductions cut into row chunks: tall and narrow, 125 column vectors, an unaligned pitch, a middle dimension
          ((100000, 64), [0]), ((5000, 1000), [0]), ((4096, 4099), [0]), ((7, 3000, 96), [1]), ((70000, 8), [0]), ((300, 16384), [0]),
          # rows of whole 16-byte vectors: lanes share a row (4 B - 4 KB), then a warp per row (to 8 KB), then a CTA
          ((5000, 64), [-1]), ((3001, 256), [-1]), ((777, 1000), [-1]), ((301, 1024), [-1]), ((4099, 8), [-1]),
          ((203, 4096), [-1]), ((101, 3000), [-1]), ((67, 4), [-1]), ((50, 8192), [-1]), ((9, 40, 72), [2])]


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


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64, torch.uint8, torch.bool])
def test_tall_column_sums_of_integers_are_exact(cuda_device, dtype):
    g = torch.Generator().manual_seed(3)
    x = torch.randint(0, 2 if dtype == torch.bool else 100, (50000, 48), generator=g).to(dtype)
    out = _red(cuda_device, "sum", x, [0])
    assert out.dtype == torch.int64 and torch.equal(out, x.sum(0))
    assert torch.equal(_red(cuda_device, "amax", x, [0]), x.amax(0)) if dtype != torch.bool else True


def test_column_sum_is_bit_reproducible(cuda_device):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(200000, 96, generator=g)
    a = _red(cuda_device, "sum", x, [0])
    b = _red(cuda_device, "sum", x, [0])
    assert torch.equal(a, b)


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [64, 1000, 2048])
def test_rows_of_a_strided_view(cuda_device, dtype, cols):
    # rows that are slices of longer rows, kept dimensions that do not merge, NaN and minus infinity in the data
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(cols)
    x = torch.randn(6, 50, 2 * cols, generator=g).to(dtype)
    x[1, 2, 3] = float("-inf")
    x[4, 7, cols - 1] = float("nan")
    xd = x.to(cuda_device)
    view = xd[:, 1:, cols // 2: cols // 2 + cols]
    ref = x[:, 1:, cols // 2: cols // 2 + cols]
    got, want = F2.reduce(OPS["amax"], view, [-1]).cpu(), ref.amax(-1)
    assert torch.equal(torch.isnan(got), torch.isnan(want)) and torch.equal(got[~torch.isnan(got)], want[~torch.isnan(want)])
    s, sw = F2.reduce(OPS["sum"], view, [-1]).cpu().double(), ref.double().sum(-1)
    fin = torch.isfinite(sw)
    assert torch.equal(torch.isnan(s), torch.isnan(sw)) and torch.equal(torch.isinf(s), torch.isinf(sw))
    assert_close(s[fin].numpy(), sw[fin].numpy(), 1e-2 if dtype == torch.bfloat16 else 1e-5, 1e-1 if dtype == torch.bfloat16 else 1e-3,
                 "sum")
    ns = F2.reduce(OPS["nansum"], view, [-1]).cpu().double()
    nsw = torch.nan_to_num(ref.double(), nan=0.0, neginf=float("-inf")).sum(-1)
    fin = torch.isfinite(nsw)
    assert not torch.isnan(ns).any()
    assert_close(ns[fin].numpy(), nsw[fin].numpy(), 1e-2 if dtype == torch.bfloat16 else 1e-5,
                 1e-1 if dtype == torch.bfloat16 else 1e-3, "nansum")


def test_row_kernels_agree_with_the_cta_kernel(cuda_device):
    # the same rows through the vector row kernels and, with them switched off, through the older ones
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(8)
    for cols, dtype in ((64, torch.float32), (1000, torch.bfloat16), (2048, torch.float16), (4096, torch.float32)):
        x = torch.randn(999, cols, generator=g).to(dtype).to(cuda_device)
        new = {op: F2.reduce(OPS[op], x, [-1]) for op in ("sum", "amax", "amin", "prod")}
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(8, 0))
        try:
            old = {op: F2.reduce(OPS[op], x, [-1]) for op in new}
        finally:
            capi.check("sb_set_tuning", capi.lib().sb_set_tuning(8, 8192))
        for op in ("amax", "amin"):
            assert torch.equal(new[op], old[op]), (op, cols)
        assert_close(new["sum"].double().cpu().numpy(), old["sum"].double().cpu().numpy(), 1e-2 if dtype != torch.float32 else 1e-5,
                     1e-1 if dtype != torch.float32 else 1e-3, "sum")


def test_dimension_order_of_the_descriptor_does_not_choose_the_path(cuda_device):
    # a TensorIterator lists the reduced dimensions first: x.sum(0) arrives as [rows (reduced, stride cols), cols (kept, stride 1)]
    from torch_supa_b200 import capi

    x = torch.randn(5000, 96, device=cuda_device)
    out = torch.empty(96, device=cuda_device)
    d = capi.make_reduce_desc(OPS["sum"], x, out, [0])
    assert d.ndim == 2 and capi.reduce_path(d) == 2
    for field in (d.sizes, d.in_strides, d.out_strides):
        field[0], field[1] = field[1], field[0]
    assert d.in_strides[0] == 96 and d.out_strides[0] == 0
    assert capi.reduce_path(d) == 2
    scratch = torch.empty(max(capi.reduce_scratch_bytes(d), 8), dtype=torch.uint8, device=cuda_device)
    d.scratch, d.scratch_bytes = scratch.data_ptr(), scratch.numel()
    capi.reduce(d)
    torch.cuda.synchronize()
    assert_close(out.cpu().numpy(), x.cpu().double().sum(0).numpy(), 1e-5, 1e-3, "sum(0), reduced dimension listed first")
    # through the operator: the same plan, so the same bits as the C ABI call in stride order
    import torch_supa_b200  # noqa: F401  (registers the supa device)

    xs = x.cpu().to("supa")
    assert torch.equal(xs.sum(0).cpu(), capi_sum0(x))


def capi_sum0(x):
    from torch_supa_b200 import functional as F2

    return F2.reduce(OPS["sum"], x, [0]).cpu()


@pytest.fixture(scope="module")
def supa():
    import torch_supa_b200  # noqa: F401  (registers the supa device)

    if not torch.supa.is_available():
        pytest.skip("no supa device")
    return torch.device("supa", 0)


@pytest.mark.parametrize("seed", range(6))
def test_seeded_random_shapes_views_and_dims(supa, seed):
    """Random shapes (sizes drawn around the kernels' switch points), dimension sets, dtypes and views (slices, permutations,
    expanded dimensions) through the operator, against PyTorch CPU: sum, amax, mean, argmax and var."""
    import random

    rnd = random.Random(1000 + seed)
    g = torch.Generator().manual_seed(seed)
    sizes = [1, 2, 3, 4, 7, 8, 16, 31, 32, 33, 64, 100, 128, 255, 256, 257, 1000, 1024, 2048, 2052, 4096, 5000]
    for _ in range(40):
        nd = rnd.choice([1, 2, 2, 2, 3, 3, 4])
        shape, numel = [], 1
        for _d in range(nd):
            cand = [v for v in sizes if numel * v <= 3_000_000] or [1]
            shape.append(rnd.choice(cand))
            numel *= shape[-1]
        dtype = rnd.choice([torch.float32, torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32, torch.int64])
        if dtype.is_floating_point:
            x = torch.randn(shape, generator=g).to(dtype)
        else:
            x = torch.randint(-50, 50, shape, generator=g).to(dtype)
        view = rnd.choice(["plain", "plain", "slice", "permute", "expand"])
        d = x.to(supa)
        if view == "slice" and shape[-1] >= 8:
            lo = rnd.choice([0, 1, 4])
            hi = shape[-1] - rnd.choice([0, 1, 4])
            x, d = x[..., lo:hi], d[..., lo:hi]
        elif view == "permute" and nd >= 2:
            perm = list(range(nd))
            rnd.shuffle(perm)
            x, d = x.permute(perm), d.permute(perm)
        elif view == "expand":
            x, d = x.unsqueeze(0).expand(3, *x.shape), d.unsqueeze(0).expand(3, *d.shape)
        k = rnd.randint(1, x.dim())
        dims = sorted(rnd.sample(range(x.dim()), k))
        what = f"{tuple(x.shape)} strides {tuple(x.stride())} {dtype} dims {dims}"
        n = 1
        for dd in dims:
            n *= x.shape[dd]
        ref = x.double().sum(dims) if dtype.is_floating_point else x.sum(dims)
        got = d.sum(dims).cpu()
        if dtype.is_floating_point:
            tol = {torch.float32: 2e-5, torch.float64: 1e-11, torch.bfloat16: 1e-2, torch.float16: 2e-3}[dtype]
            scale = float(x.double().abs().sum(dims).max()) if x.numel() else 1.0
            assert torch.allclose(got.double(), ref, rtol=tol, atol=tol * max(scale, 1.0)), "sum " + what
            assert torch.equal(d.amax(dims).cpu(), x.amax(dims)), "amax " + what
            m = d.mean(dims).cpu().double()
            assert torch.allclose(m, x.double().mean(dims), rtol=tol, atol=tol * max(scale / max(n, 1), 1.0)), "mean " + what
        else:
            assert torch.equal(got, ref), "sum " + what
            assert torch.equal(d.amax(dims).cpu(), x.amax(dims)), "amax " + what
        one = rnd.choice(range(x.dim()))
        assert torch.equal(d.argmax(one).cpu(), x.argmax(one)), f"argmax({one}) " + what
        if dtype in (torch.float32, torch.float64) and x.shape[one] > 1:
            v, rv = d.var(one).cpu().double(), x.double().var(one)
            assert torch.allclose(v, rv, rtol=1e-4 if dtype == torch.float32 else 1e-10, atol=1e-6), f"var({one}) " + what


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

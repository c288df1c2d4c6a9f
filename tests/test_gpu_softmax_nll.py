"""log_softmax and nll_loss kernels through the C ABI against fixtures, oracle and PyTorch CPU (needs a GPU)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["lsm_last", "lsm_mid", "lsm_long"])
def test_log_softmax_fixtures(golden, cuda_device, name):
    from torch_supa_b200 import functional as F2

    dim = int(golden[name + "/dim"][0])
    x = torch.from_numpy(golden[name + "/x"]).to(cuda_device)
    y = F2.log_softmax(x, dim)
    assert_close(y.cpu().numpy(), golden[name + "/y"], 2e-6, 2e-6, name)
    gi = F2.log_softmax_backward(torch.from_numpy(golden[name + "/grad_out"]).to(cuda_device), y, dim)
    assert_close(gi.cpu().numpy(), golden[name + "/grad_in"], 1e-5, 2e-6, name + " backward")


@pytest.mark.parametrize("shape,dim", [((16,), 0), ((1024, 512), -1), ((1023, 511), -1), ((1025, 513), 0),
                                       ((128, 2135), -1), ((6, 32000), -1), ((4, 5, 6, 7), 2), ((3, 40000), -1),
                                       ((2, 1027), -1), ((5, 4100), -1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_log_softmax_forward_backward(cuda_device, shape, dim, dtype):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(len(shape) * 17 + shape[0])
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    go = torch.randn(*shape, generator=g).to(dtype)
    y = F2.log_softmax(x.to(cuda_device), dim)
    ref = F.log_softmax(x.double(), dim)
    tol = {torch.float32: (2e-6, 4e-6), torch.float64: (1e-12, 1e-12), torch.bfloat16: (1.6e-2, 1e-2),
           torch.float16: (2e-3, 2e-3)}[dtype]
    assert_close(y.double().cpu().numpy(), ref.numpy(), tol[0], tol[1], "forward")
    gi = F2.log_softmax_backward(go.to(cuda_device), y, dim)
    sumg = go.double().sum(dim, keepdim=True)
    ref_gi = go.double() - torch.exp(y.double().cpu()) * sumg
    mag = float(sumg.abs().max()) + 1.0
    atol = {torch.float32: 4e-6, torch.float64: 1e-11, torch.bfloat16: 2e-2, torch.float16: 3e-3}[dtype] * mag
    assert_close(gi.double().cpu().numpy(), ref_gi.numpy(), tol[0], atol, "backward")


@pytest.mark.parametrize("name", ["sm_last", "sm_mid"])
def test_softmax_fixtures(golden, cuda_device, name):
    from torch_supa_b200 import functional as F2

    dim = int(golden[name + "/dim"][0])
    x = torch.from_numpy(golden[name + "/x"]).to(cuda_device)
    y = F2.softmax(x, dim)
    assert_close(y.cpu().numpy(), golden[name + "/y"], 2e-6, 1e-8, name)
    gi = F2.softmax_backward(torch.from_numpy(golden[name + "/grad_out"]).to(cuda_device), y, dim)
    assert_close(gi.cpu().numpy(), golden[name + "/grad_in"], 2e-5, 1e-7, name + " backward")


@pytest.mark.parametrize("shape,dim", [((16,), 0), ((1024, 512), -1), ((1023, 511), -1), ((1025, 513), 0), ((128, 2135), -1),
                                       ((200, 32000), -1), ((4, 5, 6, 7), 2), ((3, 40000), -1), ((160, 128256), -1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_softmax_forward_backward(cuda_device, shape, dim, dtype):
    """softmax (not log): generic kernels and, for long last-dimension rows, the shared-memory-resident pipeline;
    rows sum to 1; backward y * (g - sum(g * y))."""
    from torch_supa_b200 import functional as F2

    if shape[-1] > 100000 and dtype == torch.float64:
        pytest.skip("no fp64 case at this size")
    g = torch.Generator().manual_seed(len(shape) * 19 + shape[0])
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    go = torch.randn(*shape, generator=g).to(dtype)
    y = F2.softmax(x.to(cuda_device), dim)
    ref = F.softmax(x.double(), dim)
    tol = {torch.float32: (4e-6, 1e-9), torch.float64: (1e-12, 1e-15), torch.bfloat16: (1.6e-2, 1e-6),
           torch.float16: (2e-3, 1e-7)}[dtype]
    assert_close(y.double().cpu().numpy(), ref.numpy(), tol[0], tol[1], "forward")
    sums = y.double().sum(dim).cpu()
    assert float((sums - 1).abs().max()) < {torch.float32: 1e-5, torch.float64: 1e-12, torch.bfloat16: 2e-2, torch.float16: 3e-3}[dtype]
    gi = F2.softmax_backward(go.to(cuda_device), y, dim)
    yd = y.double().cpu()
    ref_gi = yd * (go.double() - (go.double() * yd).sum(dim, keepdim=True))
    # y * (g - sum) cancels where g is close to the sum: the floor scales with the operands, not with the result
    atol = {torch.float32: 1e-6, torch.float64: 1e-13, torch.bfloat16: 2e-3, torch.float16: 2e-4}[dtype]
    assert_close(gi.double().cpu().numpy(), ref_gi.numpy(), tol[0] * 4, atol, "backward")


def test_log_softmax_half_to_float(cuda_device):
    from torch_supa_b200 import functional as F2

    x = torch.randn(33, 700).bfloat16()
    y = F2.log_softmax(x.to(cuda_device), -1, out_dtype=torch.float32)
    assert y.dtype == torch.float32
    assert_close(y.cpu().numpy(), F.log_softmax(x.float(), -1).numpy(), 2e-6, 4e-6, "bf16 -> fp32")
    go = torch.randn(33, 700)
    gi = F2.log_softmax_backward(go.to(cuda_device), y, -1, input_dtype=torch.bfloat16)
    assert gi.dtype == torch.bfloat16
    ref = go - torch.exp(y.cpu()) * go.sum(-1, keepdim=True)
    assert_close(gi.float().cpu().numpy(), ref.numpy(), 1.6e-2, 0.3, "backward to bf16")


@pytest.mark.parametrize("name", ["nll_mean", "nll_sum_w", "nll_none_w", "nll_mean_w"])
def test_nll_fixtures(golden, cuda_device, name):
    from torch_supa_b200 import functional as F2

    red = name.split("_")[1]
    w = torch.from_numpy(golden[name + "/weight"]).to(cuda_device) if name.endswith("_w") else None
    logp = torch.from_numpy(golden[name + "/logp"]).to(cuda_device)
    t = torch.from_numpy(golden[name + "/target"]).to(cuda_device)
    out, tw = F2.nll_loss_forward(logp, t, w, -100, red)
    assert_close(np.atleast_1d(out.cpu().numpy()), np.atleast_1d(golden[name + "/out"]), 2e-6, 2e-6, name)
    go = torch.from_numpy(np.atleast_1d(golden[name + "/grad_out"])).to(cuda_device)
    gi = F2.nll_loss_backward(go, logp, t, w, -100, red, tw)
    assert_close(gi.cpu().numpy(), golden[name + "/grad_in"], 2e-6, 1e-7, name + " backward")


@pytest.mark.parametrize("rows,classes", [(16, 10), (1000, 2000), (20000, 100), (100, 20000), (70001, 33)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
def test_nll_against_oracle(cuda_device, rows, classes, reduction, dtype):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(rows + classes)
    logp = F.log_softmax(torch.randn(rows, classes, generator=g), 1).to(dtype)
    t = torch.randint(0, classes, (rows,), generator=g)
    t[::7] = -100
    out, tw = F2.nll_loss_forward(logp.to(cuda_device), t.to(cuda_device), None, -100, reduction)
    eout, etw = oracle.c_nll_loss(logp.float().numpy(), t.numpy(), None, -100, reduction)
    rtol = {torch.float32: 2e-6, torch.float64: 1e-6, torch.bfloat16: 1e-2}[dtype]
    assert_close(np.atleast_1d(out.double().cpu().numpy()), eout, rtol, rtol, "forward")
    if reduction != "none":
        assert abs(float(tw) - etw) <= (0 if dtype != torch.bfloat16 else 1e-2 * etw)
    go = torch.randn(rows if reduction == "none" else 1, generator=g).to(dtype)
    gi = F2.nll_loss_backward(go.to(cuda_device), logp.to(cuda_device), t.to(cuda_device), None, -100, reduction, tw)
    egi = oracle.c_nll_loss_backward(go.double().numpy(), t.numpy(), classes, None, -100, reduction, float(tw))
    assert_close(gi.double().cpu().numpy(), egi, rtol, 0, "backward")
    assert int((gi != 0).sum()) <= rows


def test_nll_many_rows_weights_and_targets_out_of_range(cuda_device):
    """The reduction over a cluster of CTAs (16384 rows and more): class weights, ignored rows, and targets outside
    [0, classes), which are reported in the status word and left out."""
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(9)
    rows, classes = 50001, 37
    logp = F.log_softmax(torch.randn(rows, classes, generator=g), 1)
    w = torch.rand(classes, generator=g) + 0.5
    t = torch.randint(0, classes, (rows,), generator=g)
    t[::5] = -100
    bad = torch.tensor([3, 20000, 49999])
    t_bad = t.clone()
    t_bad[bad] = torch.tensor([-5, classes, 1000])
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for red in ("mean", "sum"):
        out, tw = F2.nll_loss_forward(logp.to(cuda_device), t_bad.to(cuda_device), w.to(cuda_device), -100, red, status)
        t_ref = t_bad.clone()
        t_ref[bad] = -100  # an index out of range is skipped like an ignored one
        ref = F.nll_loss(logp.double(), t_ref, w.double(), ignore_index=-100, reduction=red)
        assert_close(np.atleast_1d(out.double().cpu().numpy()), np.atleast_1d(ref.numpy()), 2e-6, 2e-6, red)
        keep = t_ref != -100
        assert abs(float(tw) - float(w[t_ref[keep]].double().sum())) <= 1e-6 * float(tw)
        a = F2.nll_loss_forward(logp.to(cuda_device), t_bad.to(cuda_device), w.to(cuda_device), -100, red, status)[0]
        assert torch.equal(a, out), "the same bits on every run"
    assert int(status.item()) & capi.STATUS_TARGET_OUT_OF_RANGE


def test_nll_uint8_targets(cuda_device):
    from torch_supa_b200 import functional as F2

    logp = F.log_softmax(torch.randn(50, 200), 1)
    t = torch.randint(0, 200, (50,), dtype=torch.uint8)
    out, _ = F2.nll_loss_forward(logp.to(cuda_device), t.to(cuda_device), None, -100, "sum")
    eout, _ = oracle.c_nll_loss(logp.numpy(), t.numpy().astype(np.int64), None, -100, "sum")
    assert_close(np.atleast_1d(out.cpu().numpy()), eout, 2e-6, 2e-6, "uint8 targets")


# ---- nll_loss over (N, C, d1, ...) --------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["nll2d_mean", "nll2d_sum_w", "nll2d_none_w", "nll2d_mean_w"])
def test_nll2d_fixtures(golden, cuda_device, name):
    from torch_supa_b200 import functional as F2

    red = name.split("_")[1]
    w = torch.from_numpy(golden[name + "/weight"]).to(cuda_device) if name.endswith("_w") else None
    logp = torch.from_numpy(golden[name + "/logp"]).to(cuda_device)
    t = torch.from_numpy(golden[name + "/target"]).to(cuda_device)
    out, tw = F2.nll_loss_nd_forward(logp, t, w, -100, red)
    assert_close(np.atleast_1d(out.cpu().numpy()), np.atleast_1d(golden[name + "/out"]), 2e-6, 2e-6, name)
    go = torch.from_numpy(np.atleast_1d(golden[name + "/grad_out"])).to(cuda_device)
    gi = F2.nll_loss_nd_backward(go, logp, t, w, -100, red, tw)
    assert_close(gi.cpu().numpy(), golden[name + "/grad_in"], 2e-6, 1e-7, name + " backward")


@pytest.mark.parametrize("shape", [(2, 19, 64, 48), (3, 5, 7, 9), (1, 3, 1, 1), (4, 21, 33, 40), (5, 7, 1), (2, 1000, 8, 16)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_nll_nd_against_oracle(cuda_device, shape, reduction, dtype):
    """Vector (inner a multiple of 16 bytes) and scalar store paths, class weights, ignored samples; the gradient has at
    most one non-zero per sample and is bit-exact (a product of two exactly representable factors, rounded once)."""
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(sum(shape))
    classes = shape[1]
    logp = F.log_softmax(torch.randn(*shape, generator=g), 1).to(dtype)
    tshape = (shape[0],) + tuple(shape[2:])
    t = torch.randint(0, classes, tshape, generator=g)
    t.view(-1)[::5] = -100
    w = (torch.rand(classes, generator=g) + 0.5).to(dtype)
    for weight in (None, w):
        wd = None if weight is None else weight.to(cuda_device)
        wn = None if weight is None else weight.float().numpy()
        out, tw = F2.nll_loss_nd_forward(logp.to(cuda_device), t.to(cuda_device), wd, -100, reduction)
        eout, etw = oracle.c_nll_loss_nd(logp.float().numpy(), t.numpy(), wn, -100, reduction)
        rtol = {torch.float32: 2e-6, torch.float64: 1e-6, torch.bfloat16: 1e-2, torch.float16: 2e-3}[dtype]
        assert_close(np.atleast_1d(out.double().cpu().numpy()), np.atleast_1d(eout), rtol, rtol, "forward")
        if reduction != "none":
            assert abs(float(tw) - etw) <= rtol * max(etw, 1.0)
        go = torch.randn(tshape if reduction == "none" else (1,), generator=g).to(dtype)
        gi = F2.nll_loss_nd_backward(go.to(cuda_device), logp.to(cuda_device), t.to(cuda_device), wd, -100, reduction, tw)
        egi = oracle.c_nll_loss_nd_backward(go.double().numpy(), t.numpy(), shape, wn, -100, reduction, float(tw))
        assert_close(gi.double().cpu().numpy(), egi, rtol, 0, "backward")
        assert int((gi != 0).sum()) <= t.numel()


def test_nll_nd_all_ignored_and_uint8(cuda_device):
    from torch_supa_b200 import functional as F2

    logp = F.log_softmax(torch.randn(2, 6, 4, 8), 1)
    t = torch.full((2, 4, 8), -100)
    out, tw = F2.nll_loss_nd_forward(logp.to(cuda_device), t.to(cuda_device), None, -100, "mean")
    assert torch.isnan(out.cpu()) and float(tw) == 0.0, "mean over no samples is NaN, as on the CPU"
    out, _ = F2.nll_loss_nd_forward(logp.to(cuda_device), t.to(cuda_device), None, -100, "sum")
    assert float(out) == 0.0
    t8 = torch.randint(0, 6, (2, 4, 8), dtype=torch.uint8)
    out, _ = F2.nll_loss_nd_forward(logp.to(cuda_device), t8.to(cuda_device), None, -100, "sum")
    eout, _ = oracle.c_nll_loss_nd(logp.numpy(), t8.numpy().astype(np.int64), None, -100, "sum")
    assert_close(np.atleast_1d(out.cpu().numpy()), eout, 2e-6, 2e-6, "uint8 targets")

"""Elementwise engine through the C ABI against fixtures, oracle and PyTorch CPU (needs a GPU)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1.3e-6, 1e-5), torch.bfloat16: (1.6e-2, 1e-5), torch.float16: (1e-3, 1e-5),
       torch.float64: (1e-12, 1e-12)}
SHAPES = [(16,), (1024, 512), (1023, 511), (1025, 513), (128, 2135), (3, 5, 7)]


def _ew(dev, op, out_shape, out_dtype, *inputs, **kw):
    from torch_supa_b200 import functional as F2

    out = torch.empty(out_shape, dtype=out_dtype, device=dev)
    F2.elementwise(op, out, *[i.to(dev) if i.device.type == "cpu" else i for i in inputs], **kw)
    torch.cuda.synchronize()
    return out.cpu()


def _cmp(out, ref, dtype, what, loosen=1.0):
    rtol, atol = TOL[dtype]
    assert out.dtype == ref.dtype
    assert_close(out.double().numpy(), ref.double().numpy(), rtol * loosen, atol * loosen, what)


def test_fixtures(golden, cuda_device):
    from torch_supa_b200 import capi

    x = torch.from_numpy(golden["act/x"])
    go = torch.from_numpy(golden["act/grad_out"])
    for key, fwd, bwd in (("gelu_erf", capi.EW_GELU_ERF, capi.EW_GELU_ERF_BWD),
                          ("gelu_tanh", capi.EW_GELU_TANH, capi.EW_GELU_TANH_BWD), ("silu", capi.EW_SILU, capi.EW_SILU_BWD)):
        assert_close(_ew(cuda_device, fwd, x.shape, torch.float32, x).numpy(), golden[f"act/{key}"], 2e-6, 2e-6, key)
        assert_close(_ew(cuda_device, bwd, x.shape, torch.float32, go, x).numpy(), golden[f"act/{key}_bwd"], 4e-6, 2e-6,
                     key + " backward")
    a, b = x[:, :7], x[:, 7:]
    assert_close(_ew(cuda_device, capi.EW_GLU, (5, 7), torch.float32, a, b).numpy(), golden["act/glu"], 2e-6, 2e-6, "glu")
    p, q = torch.from_numpy(golden["bin/p"]), torch.from_numpy(golden["bin/q"])
    out = _ew(cuda_device, capi.EW_ADD, (4, 5, 16), torch.float16, p, q)
    assert np.array_equal(out.numpy(), golden["bin/p_plus_q"]), "fp16 add is exactly rounded"
    i32, f32 = torch.from_numpy(golden["bin/i32"]), torch.from_numpy(golden["bin/f32"])
    out = _ew(cuda_device, capi.EW_ADD, (8, 8), torch.float32, i32, f32, common_dtype=torch.float32)
    assert np.array_equal(out.numpy(), golden["bin/i32_plus_f32"]), "int32 + fp32 is exactly rounded"
    out = _ew(cuda_device, capi.EW_ADD, (8, 8), torch.float32, f32, f32.t(), alpha=2.5)
    assert_close(out.numpy(), golden["bin/add_alpha"], 1.3e-6, 1e-6, "add with alpha, transposed operand")
    out = _ew(cuda_device, capi.EW_MUL, (8, 8), torch.float32, f32.t(), f32)
    assert np.array_equal(out.numpy(), golden["bin/mul_t"])
    big = torch.tensor([2**31 - 1, -2**31, 7], dtype=torch.int32)
    out = _ew(cuda_device, capi.EW_ADD, (3,), torch.int32, big, torch.tensor([1, -1, 3], dtype=torch.int32))
    assert np.array_equal(out.numpy(), golden["bin/int_wrap"]), "int32 overflow wraps"


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_activations_forward_backward(cuda_device, shape, dtype):
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 2).to(dtype)
    go = torch.randn(*shape, generator=g).to(dtype)
    xr = x.double().requires_grad_(True)
    cases = [("gelu", capi.EW_GELU_ERF, capi.EW_GELU_ERF_BWD, lambda v: F.gelu(v)),
             ("gelu_tanh", capi.EW_GELU_TANH, capi.EW_GELU_TANH_BWD, lambda v: F.gelu(v, approximate="tanh")),
             ("silu", capi.EW_SILU, capi.EW_SILU_BWD, F.silu)]
    for name, fwd, bwd, fn in cases:
        y = fn(xr)
        (gi,) = torch.autograd.grad(y, xr, go.double())
        _cmp(_ew(cuda_device, fwd, shape, dtype, x), y.detach().to(dtype), dtype, name, loosen=2 if dtype != torch.float64 else 1e3)
        _cmp(_ew(cuda_device, bwd, shape, dtype, go, x), gi.to(dtype), dtype, name + " backward",
             loosen=3 if dtype != torch.float64 else 1e3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1024, 512), (1023, 510), (16, 22016)])
def test_glu_on_strided_halves(cuda_device, shape, dtype):
    """glu reads the two halves of the last dimension as strided views, as the SwiGLU configuration does."""
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(*shape, generator=g).to(dtype)
    h = shape[1] // 2
    xd = x.to(cuda_device)
    a, b = xd[:, :h], xd[:, h:]
    ref = F.glu(x.double(), -1)
    _cmp(_ew(cuda_device, capi.EW_GLU, (shape[0], h), dtype, a, b), ref.to(dtype), dtype, "glu", loosen=2)
    # silu(a) * b, the SwiGLU chain as two separately dispatched operators
    s = _ew(cuda_device, capi.EW_SILU, (shape[0], h), dtype, a)
    out = _ew(cuda_device, capi.EW_MUL, (shape[0], h), dtype, s, b)
    ref2 = (F.silu(x[:, :h].float()).to(dtype).float() * x[:, h:].float()).to(dtype)
    _cmp(out, ref2, dtype, "silu(a) * b", loosen=2)
    go = torch.randn(shape[0], h, generator=g).to(dtype)
    ga = _ew(cuda_device, capi.EW_GLU_BWD_A, (shape[0], h), dtype, go, b)
    gb = _ew(cuda_device, capi.EW_GLU_BWD_B, (shape[0], h), dtype, go, b, a)
    xr = x.double().requires_grad_(True)
    (gi,) = torch.autograd.grad(F.glu(xr, -1), xr, go.double())
    _cmp(torch.cat([ga, gb], 1), gi.to(dtype), dtype, "glu backward", loosen=3)


def test_broadcast_add_fp16(cuda_device):
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(0)
    p = torch.randn(16, 1, 4096, generator=g).half()
    q = torch.randn(1, 64, 4096, generator=g).half()
    out = _ew(cuda_device, capi.EW_ADD, (16, 64, 4096), torch.float16, p, q)
    assert torch.equal(out, p + q)
    # in-place with a broadcast `other`
    from torch_supa_b200 import functional as F2

    acc = (p + q).to(cuda_device)
    F2.elementwise(capi.EW_ADD, acc, acc, q.to(cuda_device), alpha=2.0)
    assert_close(acc.cpu().float().numpy(), torch.add(p + q, q, alpha=2.0).float().numpy(), 1e-3, 1e-3, "in place")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(8, 12, 256), (5, 7, 64), (4, 4, 8), (9, 6, 1032), (3, 5, 7, 40)])
def test_outer_broadcast_binary_ops(cuda_device, shape, dtype):
    """a[..., :, None, :] op b[..., None, :, :]: each input constant along a different dimension; ragged tile
    edges and non-commutative ops pin the operand order of the register-tiled kernel."""
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(sum(shape))
    lead = shape[:-3]
    n2, n1, n0 = shape[-3:]
    a = torch.randn(*lead, n2, 1, n0, generator=g).to(dtype)
    b = (torch.rand(*lead, 1, n1, n0, generator=g) + 0.5).to(dtype)
    for op, fn in ((capi.EW_ADD, torch.add), (capi.EW_SUB, torch.sub), (capi.EW_MUL, torch.mul), (capi.EW_DIV, torch.div)):
        for x, y in ((a, b), (b, a)):
            if op == capi.EW_DIV and y is a:
                continue  # a has values near zero
            desc = capi.make_ew_desc(op, torch.empty(shape, dtype=dtype, device=cuda_device), [x.to(cuda_device), y.to(cuda_device)])
            assert capi.elementwise_path(desc) == 1
            out = _ew(cuda_device, op, shape, dtype, x, y)
            ref = fn(x, y)
            if dtype == torch.float32 or op in (capi.EW_ADD, capi.EW_SUB, capi.EW_MUL):
                assert torch.equal(out, ref), (op, x is a)
            else:
                _cmp(out, ref, dtype, "div")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_outer_broadcast_16_bit_on_every_bit_pattern(cuda_device, dtype):
    """add / sub / mul of the outer-broadcast form run on packed 16-bit pairs without widening.  Operands drawn from all
    65536 bit patterns (subnormals, infinities, NaNs, exponents 30 binades apart, sums that fall on rounding ties) must give
    the bits of the widen-operate-round route that PyTorch's CPU kernels take; with alpha != 1 the fp32 route is used."""
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(11)
    a = torch.randint(-32768, 32768, (24, 1, 4096), generator=g, dtype=torch.int32).to(torch.int16).view(dtype)
    b = torch.randint(-32768, 32768, (1, 20, 4096), generator=g, dtype=torch.int32).to(torch.int16).view(dtype)
    # neighbours in magnitude as well: the same patterns with a few low bits changed
    b[0, :10] = (a[:10, 0].view(torch.int16) ^ torch.randint(0, 8, (10, 4096), generator=g, dtype=torch.int32).to(torch.int16)).view(dtype)
    for op, fn in ((capi.EW_ADD, torch.add), (capi.EW_SUB, torch.sub), (capi.EW_MUL, torch.mul)):
        for x, y in ((a, b), (b, a)):
            out = _ew(cuda_device, op, (24, 20, 4096), dtype, x, y)
            ref = fn(x, y)
            nan = torch.isnan(ref)
            assert torch.equal(torch.isnan(out), nan), (op, "NaN positions")
            assert torch.equal(out.view(torch.int16)[~nan], ref.view(torch.int16)[~nan]), (op, x is a)
    out = _ew(cuda_device, capi.EW_ADD, (24, 20, 4096), dtype, a, b, alpha=0.5)
    ref = torch.add(a, b, alpha=0.5)
    ok = torch.isfinite(ref)
    assert torch.equal(out[ok], ref[ok])


def test_transposed_operand_mul_both_orders(cuda_device):
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(1)
    m = torch.randn(512, 256, generator=g)
    n = torch.randn(256, 512, generator=g)
    md, nd = m.to(cuda_device).t(), n.to(cuda_device)
    out_rm = torch.empty(256, 512, device=cuda_device)
    F2.elementwise(capi.EW_MUL, out_rm, nd, md)
    assert torch.equal(out_rm.cpu(), n * m.t())
    out_cm = torch.empty(512, 256, device=cuda_device).t()  # column-major output, as m.t() * n produces
    F2.elementwise(capi.EW_MUL, out_cm, md, nd)
    assert torch.equal(out_cm.cpu(), m.t() * n)
    # as_strided operand of the reference's add test: [1, 1024, 512] with strides [524288, 1, 1024]
    base = torch.randn(512 * 1024, generator=g)
    v = base.as_strided((1, 1024, 512), (524288, 1, 1024))
    w = torch.randn(1, 1024, 512, generator=g)
    out = _ew(cuda_device, capi.EW_ADD, (1, 1024, 512), torch.float32, base.to(cuda_device).as_strided((1, 1024, 512), (524288, 1, 1024)), w)
    assert torch.equal(out, v + w)


@pytest.mark.parametrize("pair", [(torch.int32, torch.float32), (torch.bfloat16, torch.float32), (torch.float32, torch.float16),
                                  (torch.int8, torch.int32), (torch.uint8, torch.int64), (torch.bool, torch.float32),
                                  (torch.int64, torch.float64), (torch.int16, torch.bfloat16)])
@pytest.mark.parametrize("op", ["add", "mul"])
def test_type_promotion(cuda_device, pair, op):
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(4)

    def make(dt):
        if dt == torch.bool:
            return torch.rand(131, 128, generator=g) > 0.5
        if dt.is_floating_point:
            return torch.randn(131, 128, generator=g).to(dt)
        return torch.randint(-100 if dt != torch.uint8 else 0, 100, (131, 128), generator=g).to(dt)

    a, b = make(pair[0]), make(pair[1])
    ref = a + b if op == "add" else a * b
    out = _ew(cuda_device, capi.EW_ADD if op == "add" else capi.EW_MUL, ref.shape, ref.dtype, a, b, common_dtype=ref.dtype)
    assert out.dtype == ref.dtype
    if ref.dtype.is_floating_point:
        assert torch.equal(out, ref), "a single correctly rounded operation must match bit for bit"
    else:
        assert torch.equal(out, ref)


def test_bool_and_integer_semantics(cuda_device):
    from torch_supa_b200 import capi

    a = torch.tensor([True, True, False, False])
    b = torch.tensor([True, False, True, False])
    assert torch.equal(_ew(cuda_device, capi.EW_ADD, (4,), torch.bool, a, b), a + b)
    assert torch.equal(_ew(cuda_device, capi.EW_MUL, (4,), torch.bool, a, b), a * b)
    i = torch.arange(-50, 50, dtype=torch.int16)
    assert torch.equal(_ew(cuda_device, capi.EW_ADD, (100,), torch.int16, i, i, alpha=3), torch.add(i, i, alpha=3))
    u = torch.arange(0, 256, dtype=torch.int32).to(torch.uint8)
    assert torch.equal(_ew(cuda_device, capi.EW_MUL, (256,), torch.uint8, u, u), u * u)


@pytest.mark.parametrize("src", [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int32, torch.int64,
                                 torch.uint8, torch.int8, torch.int16, torch.bool])
@pytest.mark.parametrize("dst", [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int32, torch.int64,
                                 torch.uint8, torch.int8, torch.int16, torch.bool])
def test_cast_copy_is_bit_exact(cuda_device, src, dst):
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(9)
    if src == torch.bool:
        x = torch.rand(1000, generator=g) > 0.5
    elif src.is_floating_point:
        x = (torch.rand(1000, generator=g) * 100).to(src)  # non-negative, in range of every target type
    else:
        x = torch.randint(0, 100, (1000,), generator=g).to(src)
    out = _ew(cuda_device, capi.EW_COPY, (1000,), dst, x, common_dtype=src)
    assert torch.equal(out, x.to(dst))


def test_fill_and_scalar_ops(cuda_device):
    from torch_supa_b200 import capi

    out = _ew(cuda_device, capi.EW_FILL, (7, 9), torch.bfloat16, scalar=1.5, common_dtype=torch.bfloat16)
    assert torch.equal(out, torch.full((7, 9), 1.5, dtype=torch.bfloat16))
    out = _ew(cuda_device, capi.EW_FILL, (5,), torch.int64, scalar=-3, common_dtype=torch.int64)
    assert torch.equal(out, torch.full((5,), -3))
    x = torch.randn(33, 65)
    assert torch.equal(_ew(cuda_device, capi.EW_MUL_SCALAR, x.shape, torch.float32, x, scalar=0.25), x * 0.25)
    assert torch.equal(_ew(cuda_device, capi.EW_ADD_SCALAR, x.shape, torch.float32, x, scalar=2.0, alpha=3.0), x + 6.0)
    assert torch.equal(_ew(cuda_device, capi.EW_NEG, x.shape, torch.float32, x), -x)
    assert torch.equal(_ew(cuda_device, capi.EW_DIV, x.shape, torch.float32, x, x + 3), x / (x + 3))
    assert torch.equal(_ew(cuda_device, capi.EW_SUB, x.shape, torch.float32, x, x.flip(0), alpha=0.5), torch.sub(x, x.flip(0), alpha=0.5))


def test_many_dims_generic_path(cuda_device):
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(6)
    x = torch.randn(2, 3, 2, 3, 2, 3, 2, 3, generator=g)
    y = torch.randn(3, 2, 3, 2, 3, 2, 3, 2, generator=g)
    xd = x.to(cuda_device).permute(7, 6, 5, 4, 3, 2, 1, 0)
    yd = y.to(cuda_device)
    out = torch.empty(3, 2, 3, 2, 3, 2, 3, 2, device=cuda_device)
    desc = capi.make_ew_desc(capi.EW_ADD, out, [xd, yd], coalesce=False)
    assert desc.ndim == 8
    capi.elementwise(desc)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), x.permute(7, 6, 5, 4, 3, 2, 1, 0) + y)
    F2.elementwise(capi.EW_MUL, out, xd, yd)
    assert torch.equal(out.cpu(), x.permute(7, 6, 5, 4, 3, 2, 1, 0) * y)


def test_zero_numel_is_a_no_op(cuda_device):
    from torch_supa_b200 import capi

    out = _ew(cuda_device, capi.EW_ADD, (0, 5), torch.float32, torch.empty(0, 5), torch.empty(0, 5))
    assert out.shape == (0, 5)


@pytest.mark.parametrize("name", ["bce_plain", "bce_pw", "bce_pw_w"])
def test_bce_with_logits_fixtures(golden, cuda_device, name):
    """Loss and derivative kernels of binary_cross_entropy_with_logits against the frozen PyTorch CPU results;
    pos_weight arrives as a broadcast operand (stride 0 along the dimensions it does not have)."""
    from torch_supa_b200 import capi

    x = torch.from_numpy(golden[name + "/x"])
    t = torch.from_numpy(golden[name + "/target"])
    go = torch.from_numpy(golden[name + "/grad_out"])
    has_pw = (name + "/pos_weight") in golden.files
    w = torch.from_numpy(golden[name + "/weight"]) if (name + "/weight") in golden.files else torch.ones_like(x)
    if has_pw:
        pw = torch.from_numpy(golden[name + "/pos_weight"]).expand_as(x)
        loss = _ew(cuda_device, capi.EW_BCE_LOGITS_PW, x.shape, torch.float32, x, t, pw)
        dx = _ew(cuda_device, capi.EW_BCE_LOGITS_PW_BWD, x.shape, torch.float32, x, t, pw)
    else:
        loss = _ew(cuda_device, capi.EW_BCE_LOGITS, x.shape, torch.float32, x, t)
        dx = _ew(cuda_device, capi.EW_BCE_LOGITS_BWD, x.shape, torch.float32, x, t, torch.ones_like(x))
    assert_close((loss * w).numpy(), golden[name + "/loss"], 2e-6, 2e-6, name)
    assert_close((dx * w * go).numpy(), golden[name + "/grad_in"], 4e-6, 2e-6, name + " backward")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", [(4,), (1024, 512), (1023, 511), (2, 3, 4)])
def test_bce_with_logits_and_sigmoid_against_oracle(cuda_device, shape, dtype):
    from oracle import oracle
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(len(shape) * 100 + shape[0])
    x = (torch.rand(*shape, generator=g) * 10 - 5).to(dtype)
    t = torch.rand(*shape, generator=g).to(dtype)
    pw = (torch.rand(shape[-1], generator=g) * 2.9 + 0.1).to(dtype)
    eloss, egrad = oracle.c_bce_with_logits(x.float().numpy(), t.float().numpy(), pw.float().numpy())
    loss = _ew(cuda_device, capi.EW_BCE_LOGITS_PW, shape, dtype, x, t, pw.expand(shape), alpha=0.5)
    dx = _ew(cuda_device, capi.EW_BCE_LOGITS_PW_BWD, shape, dtype, x, t, pw.expand(shape), alpha=0.5)
    _cmp(loss, torch.from_numpy(eloss * 0.5).to(dtype), dtype, "loss", loosen=4)
    _cmp(dx, torch.from_numpy(egrad * 0.5).to(dtype), dtype, "derivative", loosen=4)
    sg = _ew(cuda_device, capi.EW_SIGMOID, shape, dtype, x)
    _cmp(sg, torch.sigmoid(x.double()).to(dtype), dtype, "sigmoid", loosen=2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", [(4,), (1024, 512), (1023, 511), (7, 3, 1029)])
@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_bce_with_logits_fused_reduce(cuda_device, shape, dtype, reduction):
    """One-pass loss + mean / sum against the oracle's unreduced loss summed in float64; two runs give the same bits."""
    from oracle import oracle
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(shape[0] + len(shape))
    x = (torch.rand(*shape, generator=g) * 10 - 5).to(dtype)
    t = torch.rand(*shape, generator=g).to(dtype)
    w = (torch.rand(*shape, generator=g) * 1.9 + 0.1).to(dtype)
    pw = (torch.rand(shape[-1], generator=g) * 2.9 + 0.1).to(dtype)
    for weight, pos_weight in ((None, None), (w, None), (None, pw), (w, pw)):
        eloss, _ = oracle.c_bce_with_logits(x.float().numpy(), t.float().numpy(), None if pos_weight is None else pos_weight.float().numpy(),
                                            None if weight is None else weight.float().numpy())
        want = eloss.sum() if reduction == "sum" else eloss.mean()
        args = (x.to(cuda_device), t.to(cuda_device), None if pos_weight is None else pos_weight.to(cuda_device),
                None if weight is None else weight.to(cuda_device), reduction)
        got = F2.bce_with_logits_reduce(*args)
        again = F2.bce_with_logits_reduce(*args)
        torch.cuda.synchronize()
        assert got.dtype == dtype and torch.equal(got, again)
        rtol = {torch.float32: 4e-6, torch.float64: 1e-9, torch.bfloat16: 8e-3, torch.float16: 1e-3}[dtype]
        want_t = float(torch.tensor(want, dtype=torch.float64).to(dtype))  # a sum beyond the fp16 range is inf on both sides
        if want_t == float("inf"):
            assert float(got) == float("inf")
        else:
            assert abs(float(got) - want) <= rtol * abs(want) + 1e-7, (float(got), want)

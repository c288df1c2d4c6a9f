"""Device generator and random fills: the C ABI against the numpy restatement of the Philox stream, and the supa operators
(randn / rand / randint / bernoulli_ / dropout, generator state get / set) against the same stream (needs a GPU).  The
checkpoint test follows test/test_checkpoint_rng.py:12-46 of the reference."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu

SEED = 0x1234_5678_9ABC_DEF1


@pytest.fixture(scope="module")
def supa():
    import torch_supa_b200  # noqa: F401

    if not torch.supa.is_available():
        pytest.skip("no supa device")
    return torch.device("supa", 0)


def _fill(cuda_device, kind, dtype, numel, offset=0, misalign=0, **kw):
    from torch_supa_b200 import functional as F2

    buf = torch.zeros(numel + misalign + 8, dtype=dtype, device=cuda_device)
    out = buf[misalign:misalign + numel]
    F2.rng_fill(out, kind, SEED, offset, **kw)
    torch.cuda.synchronize()
    assert bool((buf[:misalign] == 0).all()) and bool((buf[misalign + numel:] == 0).all()), "wrote outside the destination"
    return out.cpu()


# ---- the C ABI against the stream's restatement ------------------------------------------------------------------------
@pytest.mark.parametrize("numel", [1, 3, 4, 17, 4099, (1 << 20) + 5])
@pytest.mark.parametrize("misalign", [0, 1])
def test_uniform_fp32_is_the_stream(cuda_device, numel, misalign):
    got = _fill(cuda_device, "uniform", torch.float32, numel, offset=8, misalign=misalign).numpy()
    want = oracle.rng_uniform(numel, SEED, 8)
    assert np.array_equal(got, want)  # bit-exact: (word >> 8) * 2^-24
    assert got.min() >= 0.0 and got.max() < 1.0


def test_uniform_range_and_16_bit_types(cuda_device):
    n = 100003
    ref32 = oracle.rng_uniform(n, SEED, 4, -3.0, 5.0)
    got = _fill(cuda_device, "uniform", torch.float32, n, offset=4, a=-3.0, b=5.0).numpy()
    np.testing.assert_allclose(got, ref32, rtol=0, atol=5e-7)  # one fused multiply-add against a product and a sum in fp64
    for dt in (torch.bfloat16, torch.float16):
        got = _fill(cuda_device, "uniform", dt, n, offset=4, a=-3.0, b=5.0)
        want = torch.from_numpy(ref32).to(dt)
        want = torch.where(want.float() >= 5.0, torch.tensor(-3.0, dtype=dt), want)  # a value rounded up to `to` becomes `from`
        assert float(got.float().max()) < 5.0 and float(got.float().min()) >= -3.0
        assert torch.equal(got, want)


def test_uniform_fp64_uses_53_bits(cuda_device):
    n = 50001
    got = _fill(cuda_device, "uniform", torch.float64, n, offset=12).numpy()
    want = oracle.rng_uniform(n, SEED, 12, wide=True)
    assert np.array_equal(got, want)
    assert len(np.unique(got)) == n  # 24-bit values would collide


@pytest.mark.parametrize("dtype,atol", [(torch.float32, 1e-5), (torch.float64, 1e-12), (torch.bfloat16, 0.07), (torch.float16, 0.01)])
def test_normal_is_box_muller_of_the_stream(cuda_device, dtype, atol):
    n = 200003
    wide = dtype == torch.float64
    got = _fill(cuda_device, "normal", dtype, n, offset=16, a=0.5, b=2.0).double().numpy()
    want = oracle.rng_normal(n, SEED, 16, 0.5, 2.0, wide=wide)
    np.testing.assert_allclose(got, want, rtol=1e-5 if not wide else 1e-12, atol=atol)
    assert np.isfinite(got).all()


def test_normal_moments(cuda_device):
    n = 1 << 24
    got = _fill(cuda_device, "normal", torch.float32, n).double()
    assert abs(float(got.mean())) < 4 / np.sqrt(n) * 1.5
    assert abs(float(got.std()) - 1.0) < 1e-3
    assert abs(float((got ** 3).mean())) < 5e-3           # skewness
    assert abs(float((got ** 4).mean()) - 3.0) < 2e-2     # kurtosis
    assert float(got.abs().max()) < 6.0                   # sqrt(-2 ln 2^-24) = 5.77


@pytest.mark.parametrize("dtype", [torch.bool, torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.float32,
                                   torch.bfloat16, torch.float16, torch.float64])
def test_integers(cuda_device, dtype):
    n = 70001
    wide = dtype in (torch.int64, torch.float64)
    low, rng = (0, 2) if dtype == torch.bool else (0, 200) if dtype == torch.uint8 else (-7, 100)
    got = _fill(cuda_device, "integer", dtype, n, offset=20, low=low, range_=rng)
    want = oracle.rng_integer(n, SEED, 20, low, rng, wide=wide)
    assert np.array_equal(got.to(torch.int64).numpy(), want)


def test_integers_full_width(cuda_device):
    n = 4097
    got = _fill(cuda_device, "integer", torch.int64, n, offset=24, low=-(1 << 63), range_=0)
    assert np.array_equal(got.numpy(), oracle.rng_integer(n, SEED, 24, -(1 << 63), 0, wide=True))
    got = _fill(cuda_device, "integer", torch.int64, n, offset=24, low=5, range_=(1 << 40) + 3)
    assert np.array_equal(got.numpy(), oracle.rng_integer(n, SEED, 24, 5, (1 << 40) + 3, wide=True))
    got = _fill(cuda_device, "integer", torch.int32, n, offset=24, low=-(1 << 31), range_=1 << 32)
    assert np.array_equal(got.to(torch.int64).numpy(), oracle.rng_integer(n, SEED, 24, -(1 << 31), 1 << 32))


@pytest.mark.parametrize("dtype", [torch.bool, torch.float32, torch.bfloat16, torch.int64, torch.float64])
@pytest.mark.parametrize("p", [0.0, 0.3, 1.0])
def test_bernoulli(cuda_device, dtype, p):
    n = 65537
    got = _fill(cuda_device, "bernoulli", dtype, n, offset=28, a=p)
    want = oracle.rng_bernoulli(n, SEED, 28, p, wide=dtype in (torch.int64, torch.float64))
    assert np.array_equal(got.to(torch.bool).numpy(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("numel,misalign", [(5, 0), (4096, 0), (100003, 0), (4099, 1)])
def test_dropout_kernel(cuda_device, dtype, numel, misalign):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(3)
    x_cpu = torch.randn(numel + misalign, generator=g).to(dtype)
    x = x_cpu.to(cuda_device)[misalign:]
    p = 0.25
    out, mask = F2.dropout(x, p, SEED, 32)
    torch.cuda.synchronize()
    keep = oracle.rng_dropout_keep(numel, SEED, 32, p)
    assert np.array_equal(mask.cpu().numpy(), keep)
    scale = np.float32(1.0 / (1.0 - p))
    want = torch.from_numpy(np.where(keep, x_cpu[misalign:].float().numpy() * scale, np.float32(0))).to(dtype)
    assert torch.equal(out.cpu(), want)


def test_argument_errors_do_not_launch(cuda_device):
    from torch_supa_b200 import capi, functional as F2

    out = torch.empty(16, dtype=torch.float32, device=cuda_device)
    with pytest.raises(capi.KernelError):
        F2.rng_fill(out, "uniform", 1, 2)            # offset not a multiple of 4
    with pytest.raises(capi.KernelError):
        F2.rng_fill(out, "uniform", 1, 0, a=2.0, b=1.0)
    with pytest.raises(capi.KernelError):
        F2.rng_fill(out, "normal", 1, 0, a=0.0, b=-1.0)
    with pytest.raises(capi.KernelError):
        F2.rng_fill(out.to(torch.int32), "uniform", 1, 0)
    with pytest.raises(capi.KernelError):
        F2.rng_fill(out.to(torch.int32), "integer", 1, 0, low=0, range_=(1 << 32) + 1)


# ---- the operators and the generator -------------------------------------------------------------------------------------
def test_generator_state_round_trip(supa):
    torch.supa.manual_seed(77)
    assert torch.supa.initial_seed() == 77
    state = torch.supa.get_rng_state()
    assert state.dtype == torch.uint8 and state.numel() == 16
    assert int.from_bytes(bytes(state[:8].tolist()), "little") == 77 and int.from_bytes(bytes(state[8:].tolist()), "little") == 0
    a = torch.randn(1000, device=supa)
    after = torch.supa.get_rng_state()
    assert int.from_bytes(bytes(after[8:].tolist()), "little") == 4  # one 128-bit block per fill
    b = torch.randn(1000, device=supa)
    assert not torch.equal(a.cpu(), b.cpu())
    torch.supa.set_rng_state(state)
    assert torch.equal(torch.randn(1000, device=supa).cpu(), a.cpu())
    assert torch.equal(torch.randn(1000, device=supa).cpu(), b.cpu())
    torch.supa.set_rng_state(state[:8])  # the seed alone: offset 0
    assert torch.equal(torch.randn(1000, device=supa).cpu(), a.cpu())
    with pytest.raises(RuntimeError):
        torch.supa.set_rng_state(torch.zeros(5, dtype=torch.uint8))


def test_operators_draw_from_the_stream(supa):
    torch.manual_seed(1234)  # reaches the device module's manual_seed_all
    n = 10007
    z = torch.randn(n, device=supa)
    np.testing.assert_allclose(z.cpu().numpy(), oracle.rng_normal(n, 1234, 0), rtol=1e-5, atol=1e-5)
    u = torch.rand(n, device=supa)
    assert np.array_equal(u.cpu().numpy(), oracle.rng_uniform(n, 1234, 4))
    r = torch.randint(-5, 17, (n,), device=supa)
    assert np.array_equal(r.cpu().numpy(), oracle.rng_integer(n, 1234, 8, -5, 22, wide=True))
    b = torch.empty(n, device=supa).bernoulli_(0.4)
    assert np.array_equal(b.cpu().numpy() != 0, oracle.rng_bernoulli(n, 1234, 12, 0.4))
    full = torch.empty(n, dtype=torch.int32, device=supa).random_()
    assert np.array_equal(full.cpu().numpy().astype(np.int64), oracle.rng_integer(n, 1234, 16, 0, 1 << 31))
    assert int(full.min()) >= 0
    f = torch.empty(n, dtype=torch.bfloat16, device=supa).random_()
    assert float(f.float().cpu().max()) <= 256.0
    # a non-contiguous destination holds the same stream in its logical order
    torch.manual_seed(1234)
    zt = torch.empty(2 * n, device=supa)[::2].normal_()
    assert torch.equal(zt.cpu(), z.cpu())


def test_own_generator_objects(supa):
    g1 = torch.Generator(device=supa)
    g1.manual_seed(5)
    g2 = torch.Generator(device=supa)
    g2.manual_seed(5)
    a = torch.rand(513, device=supa, generator=g1)
    default_before = torch.supa.get_rng_state()
    b = torch.rand(513, device=supa, generator=g2)
    assert torch.equal(a.cpu(), b.cpu())
    assert torch.equal(torch.supa.get_rng_state(), default_before)  # the default generator did not move
    g2.set_state(g1.get_state())
    assert g2.initial_seed() == 5 and torch.equal(torch.rand(7, device=supa, generator=g1).cpu(), torch.rand(7, device=supa, generator=g2).cpu())
    with pytest.raises(RuntimeError):
        torch.rand(4, device=supa, generator=torch.Generator())  # a CPU generator


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_operator_and_backward(supa, dtype):
    torch.supa.manual_seed(9)
    x_cpu = torch.randn(64, 1000).to(dtype)
    x = x_cpu.to(supa).requires_grad_()
    y = torch.nn.functional.dropout(x, 0.4, training=True)
    keep = oracle.rng_dropout_keep(x.numel(), 9, 0, 0.4).reshape(64, 1000)
    scale = np.float32(1.0 / 0.6)
    want = torch.from_numpy(np.where(keep, x_cpu.float().numpy() * scale, np.float32(0))).to(dtype)
    assert torch.equal(y.detach().cpu(), want)
    assert 0.55 < keep.mean() < 0.65
    y.sum().backward()
    want_grad = torch.from_numpy(np.where(keep, scale, np.float32(0))).to(dtype)
    assert torch.equal(x.grad.cpu(), want_grad)
    # evaluation mode and p = 0 pass the input through; p = 1 zeroes it
    assert torch.equal(torch.nn.functional.dropout(x.detach(), 0.4, training=False).cpu(), x_cpu)
    assert torch.equal(torch.nn.functional.dropout(x.detach(), 0.0, training=True).cpu(), x_cpu)
    assert float(torch.nn.functional.dropout(x.detach(), 1.0, training=True).float().cpu().abs().max()) == 0.0


def test_checkpoint_restores_the_generator(supa):
    """Activation checkpointing replays the forward under the saved generator state: gradients with and without it agree
    bit for bit."""
    from torch.utils.checkpoint import checkpoint

    for _ in range(3):
        inp = torch.randn(20000, device=supa).requires_grad_()
        phase1, phase2 = torch.nn.Dropout(), torch.nn.Dropout()

        def run_fn(t):
            return phase2(t)

        state = torch.supa.get_rng_state()
        out = checkpoint(run_fn, phase1(inp), use_reentrant=True)
        out.sum().backward()
        with_checkpoint = inp.grad.cpu().clone()
        torch.supa.set_rng_state(state)
        inp.grad = None
        run_fn(phase1(inp)).sum().backward()
        assert torch.equal(with_checkpoint, inp.grad.cpu())

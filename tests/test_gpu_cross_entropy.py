"""Fused cross entropy through the C ABI against the oracle, the fixtures and PyTorch CPU (needs a GPU)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.helpers import assert_close, rel_err

pytestmark = pytest.mark.gpu


def _run(dev, logits, target, **kw):
    from torch_supa_b200 import functional as F2

    loss, grad = F2.cross_entropy_forward_backward(logits.to(dev), target.to(dev), **kw)
    torch.cuda.synchronize()
    return loss.float().cpu().numpy(), (None if grad is None else grad.float().cpu().numpy())


def _ce_names(golden):
    return sorted({k.split("/")[0] for k in golden.files if k.startswith("ce_")})


@pytest.mark.parametrize("idx", range(32))
def test_golden_fixtures_fp32(golden, cuda_device, idx):
    names = _ce_names(golden)
    if idx >= len(names):
        pytest.skip("no such case")
    name = names[idx]
    red = name.split("_")[2]
    ignore_index, eps = golden[name + "/meta"]
    go = golden[name + "/grad_out"]
    kw = dict(ignore_index=int(ignore_index), label_smoothing=float(eps), reduction=red)
    if red == "none":
        kw["row_grad_out"] = torch.from_numpy(go).to(cuda_device)
    else:
        kw["grad_scale"] = float(go)
    loss, grad = _run(cuda_device, torch.from_numpy(golden[name + "/logits"]), torch.from_numpy(golden[name + "/target"]), **kw)
    assert_close(np.atleast_1d(loss), np.atleast_1d(golden[name + "/loss"]), 2e-6, 2e-6, name + " loss")
    # fp32: rtol 1.3e-6 is the reference's; the absolute floor is scaled to these O(1) gradients
    assert_close(grad, golden[name + "/grad"], 1e-5, 3e-7, name + " grad")


SHAPES = [(16, 1000), (1, 1000), (512, 1024), (512, 1027), (33, 4099), (7, 32000), (3, 50257), (64, 31), (130, 64),
          (5, 1), (2, 128256)]


@pytest.mark.parametrize("rows,classes", SHAPES)
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_against_oracle(cuda_device, rows, classes, reduction, dtype):
    g = torch.Generator().manual_seed(rows * 1000003 + classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    if rows > 4:
        target[torch.randperm(rows, generator=g)[: rows // 5]] = -100
    eps = 0.1 if (rows + classes) % 2 else 0.0
    target_before = target.clone()
    loss, grad = _run(cuda_device, logits, target, label_smoothing=eps, reduction=reduction)
    assert torch.equal(target, target_before)
    eloss, egrad, bad = oracle.c_cross_entropy(logits.float().numpy(), target.numpy(), -100, eps, reduction)
    assert bad == 0
    if dtype == torch.float32:
        assert_close(np.atleast_1d(loss), eloss, 2e-6, 2e-6, "loss")
        scale = max(1.0, float((target != -100).sum())) if reduction == "mean" else 1.0
        assert_close(grad * scale, egrad * scale, 1e-5, 3e-7, "grad (scaled to per-row magnitude)")
    else:
        # 16-bit: the oracle result cast to the dtype, rtol 1.6e-2 (bf16) / 1e-3 (fp16) plus rounding of the cast
        rtol = 1.6e-2 if dtype == torch.bfloat16 else 2e-3
        if reduction == "none":
            assert_close(loss, eloss, 2e-6, 2e-6, "row loss (fp32 output)")
        else:
            assert rel_err(loss, eloss[0]) <= 1e-2
        scale = max(1.0, float((target != -100).sum())) if reduction == "mean" else 1.0
        assert_close(grad * scale, egrad * scale, rtol, 1e-4 if dtype == torch.bfloat16 else 2e-5, "grad")
    ignored = (target == -100).numpy()
    assert np.all(grad[ignored] == 0), "ignored rows must have an exactly zero gradient"


def test_matches_pytorch_cpu_fp32_config1_slice(cuda_device):
    """A 256-row slice of the fp32 [4096, 32000] configuration against F.cross_entropy on the CPU."""
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(256, 32000, generator=g) * 2
    target = torch.randint(0, 32000, (256,), generator=g)
    loss, grad = _run(cuda_device, logits, target)
    ref_loss, ref_grad = oracle.aten_cross_entropy(logits, target)
    assert rel_err(loss, ref_loss) <= 1e-5
    assert_close(grad * 256, ref_grad.numpy() * 256, 1e-5, 3e-7, "grad")


def test_all_rows_ignored(cuda_device):
    logits = torch.randn(4, 10)
    target = torch.full((4,), -100)
    loss, grad = _run(cuda_device, logits, target, reduction="mean")
    assert np.isnan(loss)
    assert np.all(grad == 0)
    loss, _ = _run(cuda_device, logits, target, reduction="sum")
    assert loss == 0
    loss, _ = _run(cuda_device, logits, target, reduction="none")
    assert np.all(loss == 0)


def test_ignore_index_may_be_a_valid_class(cuda_device):
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(9, 12, generator=g)
    target = torch.randint(0, 12, (9,), generator=g)
    target[:3] = 2
    loss, grad = _run(cuda_device, logits, target, ignore_index=2)
    eloss, egrad, _ = oracle.c_cross_entropy(logits.numpy(), target.numpy(), 2, 0.0, "mean")
    assert_close(np.atleast_1d(loss), eloss, 2e-6, 2e-6, "loss")
    assert np.all(grad[:3] == 0)


def test_out_of_range_target_sets_status_and_does_not_trap(cuda_device):
    from torch_supa_b200 import capi, functional as F2

    logits = torch.randn(6, 8).to(cuda_device)
    target = torch.tensor([1, 2, 8, 3, -7, 0]).to(cuda_device)
    ws = F2.CrossEntropyWorkspace(6, cuda_device)
    loss, grad = F2.cross_entropy_forward_backward(logits, target, reduction="sum", workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.status.item()) & capi.STATUS_TARGET_OUT_OF_RANGE
    assert torch.all(grad[2] == 0) and torch.all(grad[4] == 0)
    eloss, _, bad = oracle.c_cross_entropy(logits.cpu().numpy(), target.cpu().numpy(), -100, 0.0, "sum")
    assert bad == 2
    assert rel_err(loss.item(), eloss[0]) <= 2e-6
    # the context is still healthy
    assert torch.isfinite(torch.ones(4, device=cuda_device).sum()).item()


def test_forward_only_and_in_place_gradient(cuda_device):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(40, 3000, generator=g) * 2).to(cuda_device)
    target = torch.randint(0, 3000, (40,), generator=g).to(cuda_device)
    loss_a, none = F2.cross_entropy_forward_backward(logits, target, want_grad=False)
    assert none is None
    loss_b, grad = F2.cross_entropy_forward_backward(logits, target)
    buf = logits.clone()
    loss_c, grad_inplace = F2.cross_entropy_forward_backward(buf, target, grad=buf)
    torch.cuda.synchronize()
    assert loss_a.item() == loss_b.item() == loss_c.item()
    assert torch.equal(grad, grad_inplace)


def test_results_are_bit_reproducible(cuda_device):
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(300, 5000, generator=g) * 2).bfloat16().to(cuda_device)
    target = torch.randint(0, 5000, (300,), generator=g).to(cuda_device)
    l1, g1 = F2.cross_entropy_forward_backward(logits, target, label_smoothing=0.1)
    l2, g2 = F2.cross_entropy_forward_backward(logits, target, label_smoothing=0.1)
    torch.cuda.synchronize()
    assert l1.item() == l2.item() and torch.equal(g1, g2)


def test_rescale_grad(cuda_device):
    from torch_supa_b200 import capi

    grad = torch.randn(1000, device=cuda_device)
    ref = grad.clone()
    applied = torch.full((2,), float("nan"), device=cuda_device)  # two words, used alternately; none valid yet
    slot = None
    for s in (1.0, 0.25, 0.25, 2.0):
        scale = torch.tensor(s, device=cuda_device)
        nxt = 0 if slot is None else 1 - slot
        capi.ce_rescale_grad(grad, grad, capi.F32, grad.numel(), scale, capi.F32, None if slot is None else applied[slot:slot + 1],
                             applied[nxt:nxt + 1])
        slot = nxt
        torch.cuda.synchronize()
        assert_close(grad.cpu().numpy(), (ref * s).cpu().numpy(), 2e-7, 0, f"scale {s}")
        assert applied[slot].item() == s
    with pytest.raises(capi.KernelError):
        capi.ce_rescale_grad(grad, grad, capi.F32, grad.numel(), scale, capi.F32, applied[0:1], applied[0:1])
    # out of place: the source and the recorded factor stay as they are, a factor of exactly 1 still copies
    out = torch.zeros_like(grad)
    before = grad.clone()
    for s in (2.0, 6.0):
        capi.ce_rescale_grad(grad, out, capi.F32, grad.numel(), torch.tensor(s, device=cuda_device), capi.F32, applied[slot:slot + 1], None)
        torch.cuda.synchronize()
        assert torch.equal(grad, before) and applied[slot].item() == 2.0
        assert_close(out.cpu().numpy(), (ref * s).cpu().numpy(), 2e-7, 0, f"out of place {s}")
    # a recorded factor of zero cannot be undone: NaN and a status bit, unless the new factor is zero too
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    zero = torch.zeros(1, device=cuda_device)
    capi.ce_rescale_grad(grad, out, capi.F32, grad.numel(), zero, capi.F32, zero, None, status)
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.count_nonzero(out).item() == 0
    capi.ce_rescale_grad(grad, out, capi.F32, grad.numel(), torch.ones(1, device=cuda_device), capi.F32, zero, None, status)
    torch.cuda.synchronize()
    assert status.item() == capi.STATUS_GRADIENT_LOST and torch.isnan(out).all()


def test_linearity_property_full_vocab(cuda_device):
    """Size-independent checks at the large-vocabulary row length: gradient rows sum to ~0 (softmax sums to 1,
    the smoothed one-hot sums to 1) and the loss of row-permuted inputs is unchanged."""
    from torch_supa_b200 import functional as F2

    rows, classes = 64, 128256
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = (torch.randn(rows, classes, device=cuda_device, generator=g) * 2).bfloat16()
    target = torch.randint(0, classes, (rows,), device=cuda_device, generator=g)
    loss, grad = F2.cross_entropy_forward_backward(logits.float(), target, label_smoothing=0.1, reduction="sum")
    row_sums = grad.double().sum(1)
    assert float(row_sums.abs().max()) < 1e-4
    perm = torch.randperm(rows, device=cuda_device)
    loss_p, _ = F2.cross_entropy_forward_backward(logits.float()[perm].contiguous(), target[perm].contiguous(),
                                                  label_smoothing=0.1, reduction="sum")
    assert rel_err(loss_p.item(), loss.item()) <= 1e-6


@pytest.mark.parametrize("rows,classes,dtype,variant", [
    (300, 4100, torch.float32, 16),     # 16400 B: the shortest rows a team of four warps sweeps (1025 units)
    (200, 8192, torch.float32, 16),     # 32 KB: the longest rows of the slot ring (6 slots, three teams)
    (200, 16384, torch.bfloat16, 16),   # 32 KB of bf16
    (300, 12000, torch.float16, 16),    # 24000 B
    (100, 8196, torch.float32, 1),      # 32784 B: just past the ring, resident in one CTA (five chunks, the last one short)
    (300, 32000, torch.float32, 1),     # the fp32 benchmark row
    (200, 45000, torch.float32, 1),     # 180000 B: about the largest single-CTA rows
    (200, 50000, torch.float32, 2),     # 200000 B: leaves no spare buffers in one CTA, goes to a 2-CTA cluster
    (150, 128256, torch.bfloat16, 2),   # the bf16 benchmark row, split over a 2-CTA cluster
    (150, 90004, torch.float32, 2),     # odd unit count: the two slices differ in length
    (150, 100004, torch.float32, 4),    # 400016 B: odd unit count over four CTAs
    (148, 150000, torch.float32, 4),    # 600000 B: 4-CTA cluster
    (75, 300008, torch.float16, 4),
    (30, 128256, torch.bfloat16, 2),    # fewer rows than clusters: some SMs idle, still one read and one write
    (64, 32002, torch.float32, 1),      # row pitch not a multiple of 16 bytes: edge units handled apart
    (64, 50257, torch.bfloat16, 1),     # real vocabularies whose rows start at every 2-byte phase of a 16-byte unit
    (64, 32001, torch.float32, 1),
    (64, 151643, torch.bfloat16, 2),
    (37, 300007, torch.float16, 4),
    (150, 50257, torch.float32, 2),     # 201028 B: ragged rows over a 2-CTA cluster
    (4096, 2048, torch.float32, 16),    # short aligned rows: one warp per row on the shared-memory slot ring
    (2000, 1000, torch.bfloat16, 16),   # 2000 B rows
    (701, 512, torch.bfloat16, 16),     # 1 KB: the shortest rows the ring takes; two rows per warp, an odd row count
    (900, 256, torch.float32, 16),      # 1 KB of fp32
    (3001, 128, torch.float32, 16),     # 512 B: four rows per warp
    (3001, 64, torch.float32, 16),      # 256 B: eight rows per warp, the shortest rows the ring takes
    (1500, 136, torch.bfloat16, 16),    # 272 B = 17 units: eight lanes per row, most lanes' third unit is missing
    (333, 500, torch.float32, 16),      # 2000 B of fp32: 125 units, the last lanes' fourth unit is missing
    (500, 4088, torch.float16, 16),     # 8176 B: 511 units
    (300, 4092, torch.float32, 16),     # 16368 B: the longest (13 slots, 6 consumer warps)
    (20, 2048, torch.float32, 16),      # fewer rows than SMs
    (4097, 1024, torch.float32, 16),    # a row count that leaves CTAs with unequal shares
    (1000, 4093, torch.bfloat16, 8),    # short ragged rows, one 128-thread group each
    (3000, 100, torch.float32, 16),     # 400 B = 25 units over eight lanes
    (3000, 50, torch.float32, 8),       # 200 B: under the ring's 256 B, rows in registers (part of a warp each)
    (777, 1023, torch.float16, 8),
])
def test_resident_variants(cuda_device, rows, classes, dtype, variant):
    """The shared-memory-resident kernels (single CTA and 2/4-CTA clusters) against the oracle."""
    from torch_supa_b200 import capi

    assert capi.ce_kernel_variant(capi.torch_dtype_code(dtype), rows, classes) == variant
    g = torch.Generator().manual_seed(classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::11] = -100
    target[1] = 0
    target[2] = classes - 1
    for eps, red in ((0.1, "mean"), (0.0, "sum")):
        loss, grad = _run(cuda_device, logits, target, label_smoothing=eps, reduction=red)
        eloss, egrad, bad = oracle.c_cross_entropy(logits.float().numpy(), target.numpy(), -100, eps, red)
        scale = float((target != -100).sum()) if red == "mean" else 1.0
        if dtype == torch.float32:
            assert rel_err(loss, eloss[0]) <= 2e-6
            assert_close(grad * scale, egrad * scale, 1e-5, 3e-7, f"grad {red}")
        else:
            assert rel_err(loss, eloss[0]) <= 1e-2
            # fp16 stores p / |V|: one subnormal step (2^-24) of the stored value is the floor of what can be resolved
            assert_close(grad * scale, egrad * scale, 1.6e-2 if dtype == torch.bfloat16 else 2e-3,
                         1e-4 if dtype == torch.bfloat16 else max(2e-5, 2.0 ** -24 * scale), f"grad {red}")
        assert np.all(grad[(target == -100).numpy()] == 0)
    # forward only and per-row losses
    loss_n, none = _run(cuda_device, logits, target, reduction="none", want_grad=False)
    eloss_n, _, _ = oracle.c_cross_entropy(logits.float().numpy(), target.numpy(), -100, 0.0, "none", want_grad=False)
    assert none is None
    assert_close(loss_n, eloss_n, 2e-6, 2e-6, "row losses")


@pytest.mark.parametrize("rows,classes,dtype", [(4096, 2048, torch.float32), (3000, 1000, torch.bfloat16), (900, 4088, torch.float16)])
def test_short_rows_in_registers_when_forced(cuda_device, rows, classes, dtype):
    """The register kernel still serves the shapes the slot ring has taken over (tuning key 1 = 8), and both kernels agree
    with the oracle; between themselves the fp32 results differ only by summation order."""
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(rows + classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::7] = -100
    code = capi.torch_dtype_code(dtype)
    assert capi.ce_kernel_variant(code, rows, classes) == 16
    loss_ring, grad_ring = _run(cuda_device, logits, target, label_smoothing=0.1, reduction="mean")
    capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, 8))
    try:
        assert capi.ce_kernel_variant(code, rows, classes) == 8
        loss_reg, grad_reg = _run(cuda_device, logits, target, label_smoothing=0.1, reduction="mean")
    finally:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(1, -1))
    eloss, egrad, _ = oracle.c_cross_entropy(logits.float().numpy(), target.numpy(), -100, 0.1, "mean")
    scale = float((target != -100).sum())
    for loss, grad in ((loss_ring, grad_ring), (loss_reg, grad_reg)):
        assert rel_err(loss, eloss[0]) <= (2e-6 if dtype == torch.float32 else 1e-2)
        if dtype == torch.float32:
            assert_close(grad * scale, egrad * scale, 1e-5, 3e-7, "grad")
        else:
            assert_close(grad * scale, egrad * scale, 1.6e-2 if dtype == torch.bfloat16 else 2e-3,
                         1e-4 if dtype == torch.bfloat16 else max(2e-5, 2.0 ** -24 * scale), "grad")


@pytest.mark.parametrize("rows,classes,dtype", [(40, 50257, torch.bfloat16), (40, 32001, torch.float32), (300, 1001, torch.bfloat16),
                                                (33, 151643, torch.bfloat16)])
def test_unaligned_base_and_in_place(cuda_device, rows, classes, dtype):
    """Logits that start in the middle of a 16-byte unit (a view one element into a larger buffer), overwritten in place
    by their gradient: neither the element before the first row nor the one after the last row may change."""
    from torch_supa_b200 import capi

    g = torch.Generator().manual_seed(classes + rows)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::9] = -100
    buf = torch.full((rows * classes + 16,), 7.0, dtype=dtype, device=cuda_device)
    view = buf[1:1 + rows * classes].view(rows, classes)
    view.copy_(logits)
    row_loss = torch.empty(rows, dtype=torch.float32, device=cuda_device)
    acc = torch.zeros(2, dtype=torch.float64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    td = target.to(cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    capi.ce_count_valid(td, rows, classes, -100, acc, status, stream)
    a = capi.CEArgs()
    a.logits = a.grad_logits = view.data_ptr()
    a.dtype, a.reduction, a.target = capi.torch_dtype_code(dtype), capi.REDUCTION_MEAN, td.data_ptr()
    a.row_loss, a.acc, a.rows, a.classes, a.ignore_index = row_loss.data_ptr(), acc.data_ptr(), rows, classes, -100
    a.label_smoothing, a.grad_scale, a.status, a.flags = 0.1, 1.0, status.data_ptr(), capi.CE_FLAG_AFTER_COUNT
    capi.ce_forward_backward(a, stream)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert float(buf[0]) == 7.0 and bool((buf[1 + rows * classes:] == 7.0).all()), "bytes outside the rows were written"
    eloss, egrad, bad = oracle.c_cross_entropy(logits.float().numpy(), target.numpy(), -100, 0.1, "mean")
    scale = float((target != -100).sum())
    grad = view.float().cpu().numpy()
    tol = {torch.float32: (1e-5, 3e-7), torch.bfloat16: (1.6e-2, 1e-4), torch.float16: (2e-3, 2e-5)}[dtype]
    assert_close(grad * scale, egrad * scale, tol[0], tol[1], "in-place gradient")
    assert np.all(grad[(target == -100).numpy()] == 0)
    want = float(row_loss.double().sum()) / scale
    assert rel_err(want, eloss[0]) <= (2e-6 if dtype == torch.float32 else 1e-3)


@pytest.mark.parametrize("rows,classes,dtype", [(64, 32000, torch.float32), (48, 50257, torch.bfloat16), (300, 1000, torch.float32),
                                                (16, 10, torch.float32), (40, 5003, torch.float16)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_class_weights_with_label_smoothing(cuda_device, rows, classes, dtype, reduction):
    """Class weights together with label smoothing: the smoothing term weights every class by its own weight; against
    PyTorch CPU in float64."""
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(3 * rows + classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::5] = -100
    w = torch.rand(classes, generator=g) + 0.25
    xr = logits.double().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr, target, weight=w.double(), reduction=reduction, label_smoothing=0.2)
    go = torch.ones(rows) if reduction == "none" else None
    ref.backward(go.double() if go is not None else None)
    loss, grad = F2.cross_entropy_forward_backward(logits.to(cuda_device), target.to(cuda_device), reduction=reduction,
                                                   class_weight=w.to(cuda_device), label_smoothing=0.2)
    torch.cuda.synchronize()
    tol = {torch.float32: (1e-5, 3e-7), torch.bfloat16: (1.6e-2, 1e-4), torch.float16: (2e-3, 2e-5)}[dtype]
    ltol = 4e-6 if (dtype == torch.float32 or reduction == "none") else tol[0]
    assert_close(np.atleast_1d(loss.double().cpu().numpy()), np.atleast_1d(ref.detach().numpy()), ltol, 4e-6, "loss")
    scale = float(w[target[target >= 0]].sum()) if reduction == "mean" else 1.0
    assert_close(grad.double().cpu().numpy() * scale, xr.grad.numpy() * scale, tol[0], tol[1], "grad")
    assert float(grad[0].abs().max()) == 0.0, "ignored rows get a zero gradient"


def _xchg(cuda_device, nranks, rank, seq, slot_arrays):
    from torch_supa_b200 import capi

    x = capi.Xchg()
    for r in range(nranks):
        x.slots[r] = slot_arrays[r].data_ptr()
    x.rank, x.nranks, x.seq = rank, nranks, seq
    return x


def test_scalar_exchange_kernels_on_one_gpu(cuda_device):
    """The exchange inside the count and loss kernels, on one GPU: a job of one rank (its own partial travels through its
    slot array), and rank 0 of a job of two whose peer's partials are already in place when the kernels start (put
    there by the host: no kernel here waits for another launch).  The sum runs in rank order."""
    import struct

    from torch_supa_b200 import capi

    rows, classes = 5000, 300
    g = torch.Generator().manual_seed(9)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::4] = -100
    valid = int((target != -100).sum())
    td = target.to(cuda_device)
    row_loss = torch.rand(rows, generator=g).to(cuda_device)
    local_sum = float(row_loss.double().sum())
    acc = torch.zeros(2, dtype=torch.float64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    loss = torch.empty((), device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    mine = torch.zeros(capi.XCHG_SLOT_BYTES, dtype=torch.uint8, device=cuda_device)
    # one rank
    capi.ce_count_exchange(td, None, rows, classes, -100, acc, status, _xchg(cuda_device, 1, 0, 1, [mine]), stream)
    capi.ce_loss_exchange(row_loss, rows, acc, capi.REDUCTION_MEAN, loss, capi.F32, status, _xchg(cuda_device, 1, 0, 2, [mine]), stream)
    torch.cuda.synchronize()
    assert status.item() == 0 and acc[1].item() == valid
    assert abs(acc[0].item() - local_sum) <= 1e-9 * local_sum and abs(loss.item() - local_sum / valid) <= 2e-7 * local_sum / valid
    # rank 0 of two: the peer's slots (source rank 1) of exchanges 3 and 4 are filled before the launches
    other = torch.zeros(capi.XCHG_SLOT_BYTES, dtype=torch.uint8, device=cuda_device)  # stands for the peer's array: only written to
    host = bytearray(capi.XCHG_SLOT_BYTES)
    for seq, value in ((3, 1234.0), (4, 0.5)):
        off = ((seq % capi.XCHG_DEPTH) * capi.XCHG_MAX_RANKS + 1) * 16
        host[off:off + 16] = struct.pack("<dQ", value, seq)
    mine.copy_(torch.frombuffer(host, dtype=torch.uint8))
    capi.ce_count_exchange(td, None, rows, classes, -100, acc, status, _xchg(cuda_device, 2, 0, 3, [mine, other]), stream)
    capi.ce_loss_exchange(row_loss, rows, acc, capi.REDUCTION_SUM, loss, capi.F32, status, _xchg(cuda_device, 2, 0, 4, [mine, other]), stream)
    torch.cuda.synchronize()
    assert status.item() == 0 and acc[1].item() == valid + 1234.0
    assert abs(acc[0].item() - (local_sum + 0.5)) <= 1e-9 * local_sum
    # what this rank published for its peer: its partials under the right sequence numbers, at source-rank slot 0
    pub = bytes(other.cpu().numpy())
    v3, s3 = struct.unpack_from("<dQ", pub, ((3 % capi.XCHG_DEPTH) * capi.XCHG_MAX_RANKS + 0) * 16)
    v4, s4 = struct.unpack_from("<dQ", pub, ((4 % capi.XCHG_DEPTH) * capi.XCHG_MAX_RANKS + 0) * 16)
    assert (s3, s4) == (3, 4) and v3 == valid and abs(v4 - local_sum) <= 1e-9 * local_sum


def test_scalar_exchange_wait_runs_out(cuda_device):
    """A peer that never publishes: the bounded wait gives up after its limit, the kernel finishes with the local partial
    and sets SB_STATUS_KERNEL_TIMEOUT; the context stays usable."""
    from torch_supa_b200 import capi

    rows, classes = 100, 10
    td = torch.zeros(rows, dtype=torch.int64, device=cuda_device)
    acc = torch.zeros(2, dtype=torch.float64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    mine = torch.zeros(capi.XCHG_SLOT_BYTES, dtype=torch.uint8, device=cuda_device)
    other = torch.zeros(capi.XCHG_SLOT_BYTES, dtype=torch.uint8, device=cuda_device)
    capi.check("sb_set_tuning", capi.lib().sb_set_tuning(5, 50))  # 50 ms
    try:
        capi.ce_count_exchange(td, None, rows, classes, -100, acc, status, _xchg(cuda_device, 2, 0, 1, [mine, other]),
                               torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
    finally:
        capi.check("sb_set_tuning", capi.lib().sb_set_tuning(5, 10000))
    assert status.item() == capi.STATUS_KERNEL_TIMEOUT
    assert acc[1].item() == rows
    assert float((torch.ones(4, device=cuda_device) * 2).sum()) == 8.0


def test_resident_matches_generic_bitwise_loss_order(cuda_device):
    """Running twice gives identical bits (persistent grid, fixed row->CTA map, no atomics on floats)."""
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(2)
    logits = (torch.randn(600, 32000, generator=g) * 2).to(cuda_device)
    target = torch.randint(0, 32000, (600,), generator=g).to(cuda_device)
    l1, g1 = F2.cross_entropy_forward_backward(logits, target)
    l2, g2 = F2.cross_entropy_forward_backward(logits, target)
    torch.cuda.synchronize()
    assert l1.item() == l2.item() and torch.equal(g1, g2)


@pytest.mark.parametrize("rows,classes,dtype", [(200, 32000, torch.float32), (160, 128256, torch.bfloat16), (50, 3000, torch.float32),
                                                (64, 500, torch.float16)])
def test_masked_logits_minus_inf(cuda_device, rows, classes, dtype):
    """Rows where most classes are masked with -inf (and one row that is entirely -inf) behave as on the CPU."""
    g = torch.Generator().manual_seed(7)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    logits[:, : classes // 2] = float("-inf")          # the first chunks of every row hold no finite value
    logits[3, :] = float("-inf")
    target = torch.randint(classes // 2, classes, (rows,), generator=g)
    loss, grad = _run(cuda_device, logits, target, reduction="none")
    ref_loss, ref_grad = oracle.aten_cross_entropy(logits, target, reduction="none", grad_out=torch.ones(rows))
    ok = torch.ones(rows, dtype=torch.bool)
    ok[3] = False
    assert np.isnan(loss[3]) and torch.isnan(ref_loss[3])
    assert_close(loss[ok.numpy()], ref_loss[ok].numpy(), 2e-6 if dtype == torch.float32 else 2e-6, 4e-6, "loss")
    assert np.all(grad[ok.numpy()][:, : classes // 2] == 0)
    tol = {torch.float32: (1e-5, 3e-7), torch.bfloat16: (1.6e-2, 1e-4), torch.float16: (2e-3, 2e-5)}[dtype]
    assert_close(grad[ok.numpy()], ref_grad[ok].numpy(), tol[0], tol[1], "grad")


@pytest.mark.parametrize("rows,classes,dtype", [(200, 32000, torch.float32), (160, 128256, torch.bfloat16), (160, 64000, torch.float16),
                                                (50, 3000, torch.float32), (64, 500, torch.bfloat16)])
def test_nan_logit_poisons_its_row_only(cuda_device, rows, classes, dtype):
    """A NaN logit makes the loss and every gradient element of its row NaN, as on the CPU; other rows are untouched.
    Positions are chosen so that the NaN falls on each of the four 4-byte pairs of a 16-byte vector."""
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    bad = {2: 5, 7: classes - 1, 11: classes // 2 + 6, 13: 16 * 9 + 3, 17: 8 * 1001 + 7}
    for r, c in bad.items():
        logits[r, c % classes] = float("nan")
    loss, grad = _run(cuda_device, logits, target, reduction="none")
    ref_loss, ref_grad = oracle.aten_cross_entropy(logits, target, reduction="none", grad_out=torch.ones(rows))
    ok = np.ones(rows, dtype=bool)
    for r in bad:
        ok[r] = False
        assert np.isnan(loss[r]) and bool(torch.isnan(ref_loss[r]))
        assert np.all(np.isnan(grad[r])), f"row {r}: {np.count_nonzero(~np.isnan(grad[r]))} finite gradient elements"
        assert bool(torch.isnan(ref_grad[r].float()).all())
    assert not np.isnan(loss[ok]).any() and not np.isnan(grad[ok]).any()
    tol = {torch.float32: (1e-5, 3e-7), torch.bfloat16: (1.6e-2, 1e-4), torch.float16: (2e-3, 2e-5)}[dtype]
    assert_close(loss[ok], ref_loss[torch.from_numpy(ok)].numpy(), 2e-6, 4e-6, "loss")
    assert_close(grad[ok], ref_grad[torch.from_numpy(ok)].numpy(), tol[0], tol[1], "grad")


@pytest.mark.parametrize("rows,classes,dtype", [(64, 32000, torch.float32), (160, 128256, torch.bfloat16), (37, 1000, torch.float32),
                                                (300, 3000, torch.float16), (16, 10, torch.float32)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_class_weights(cuda_device, rows, classes, dtype, reduction):
    """Per-class weights (no label smoothing): row i is scaled by w[target_i], mean divides by the sum of those
    weights; resident and generic kernels against PyTorch CPU in float64."""
    from torch_supa_b200 import functional as F2

    g = torch.Generator().manual_seed(rows + classes)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::6] = -100
    w = torch.rand(classes, generator=g) + 0.25
    xr = logits.double().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr, target, weight=w.double(), reduction=reduction)
    go = torch.ones(rows) if reduction == "none" else None
    ref.backward(go.double() if go is not None else None)
    loss, grad = F2.cross_entropy_forward_backward(logits.to(cuda_device), target.to(cuda_device), reduction=reduction,
                                                   class_weight=w.to(cuda_device))
    torch.cuda.synchronize()
    tol = {torch.float32: (1e-5, 3e-7), torch.bfloat16: (1.6e-2, 1e-4), torch.float16: (2e-3, 2e-5)}[dtype]
    ltol = 2e-6 if (dtype == torch.float32 or reduction == "none") else tol[0]
    assert_close(np.atleast_1d(loss.double().cpu().numpy()), np.atleast_1d(ref.detach().numpy()), ltol, 4e-6, "loss")
    scale = float(w[target[target >= 0]].sum()) if reduction == "mean" else 1.0
    assert_close(grad.double().cpu().numpy() * scale, xr.grad.numpy() * scale, tol[0], tol[1], "grad")
    assert float(grad[0].abs().max()) == 0.0, "ignored rows get a zero gradient"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_chunks_with_in_place_gradient_equal_one_call(cuda_device, dtype):
    """The protocol a producer of logits uses to avoid holding [rows, classes] twice: count the valid targets once, then
    hand over row blocks as they are produced, each overwritten by its gradient (grad_logits aliases logits), and sum
    the per-row losses at the end.  Same loss and gradients as one call over all rows."""
    from torch_supa_b200 import capi
    from torch_supa_b200 import functional as F2

    rows, classes, chunk = 1200, 32000, 400
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype).to(cuda_device)
    target = torch.randint(0, classes, (rows,), generator=g)
    target[::13] = -100
    target = target.to(cuda_device)
    loss_ref, grad_ref = F2.cross_entropy_forward_backward(logits, target, label_smoothing=0.1)

    work = logits.clone()
    row_loss = torch.empty(rows, dtype=torch.float32, device=cuda_device)
    acc = torch.zeros(2, dtype=torch.float64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    capi.ce_count_valid(target, rows, classes, -100, acc, status, stream)
    esize = work.element_size()
    for r0 in range(0, rows, chunk):
        a = capi.CEArgs()
        a.logits = work.data_ptr() + r0 * classes * esize
        a.grad_logits = a.logits                         # in place
        a.dtype, a.reduction = capi.torch_dtype_code(dtype), capi.REDUCTION_MEAN
        a.target = target.data_ptr() + r0 * 8
        a.row_loss = row_loss.data_ptr() + r0 * 4
        a.acc = acc.data_ptr()
        a.rows, a.classes, a.ignore_index, a.label_smoothing, a.grad_scale = min(chunk, rows - r0), classes, -100, 0.1, 1.0
        a.status = status.data_ptr()
        capi.ce_forward_backward(a, stream)
    loss = torch.empty((), dtype=dtype, device=cuda_device)
    capi.ce_loss_sum_finish(row_loss, rows, acc, capi.REDUCTION_MEAN, loss, capi.torch_dtype_code(dtype), stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float(loss) == float(loss_ref), "per-row losses do not depend on how the rows are grouped"
    assert torch.equal(work, grad_ref)


def test_headline_size_properties_and_row_subset(cuda_device):
    """The benchmark's full configuration (bf16 [32768, 128256], 5 % ignored rows, label smoothing 0.1, mean): checks that
    do not need a CPU pass over 8.4 GB — every ignored row's gradient is exactly zero, gradient rows sum to ~0, the loss
    equals the mean of the per-row losses — plus a seeded 1024-row subset against the CPU oracle."""
    from torch_supa_b200 import functional as F2

    rows, classes, eps = 32768, 128256, 0.1
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.empty(rows, classes, dtype=torch.bfloat16, device=cuda_device)
    for r0 in range(0, rows, 2048):
        logits[r0:r0 + 2048] = (torch.randn(2048, classes, device=cuda_device, generator=g) * 2).bfloat16()
    cg = torch.Generator().manual_seed(1)
    target = torch.randint(0, classes, (rows,), generator=cg)
    ignored = torch.randperm(rows, generator=cg)[:1638]
    target[ignored] = -100
    target_d = target.to(cuda_device)
    ws = F2.CrossEntropyWorkspace(rows, cuda_device)
    loss, grad = F2.cross_entropy_forward_backward(logits, target_d, label_smoothing=eps, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
    count = rows - 1638
    # (1) ignored rows: exactly zero gradient and zero loss
    assert int(grad[ignored.to(cuda_device)].ne(0).sum()) == 0
    assert float(ws.row_loss[ignored.to(cuda_device)].abs().max()) == 0.0
    # (2) the scalar is the mean of the per-row losses (rounded to bf16)
    want = float(ws.row_loss.double().sum()) / count
    assert abs(float(loss) - want) <= 4e-3 * want
    # (3) rows of the gradient sum to zero: softmax sums to 1 and so does the smoothed one-hot (bf16 rounding noise only);
    # (4) a seeded 1024-row subset against the CPU oracle (fp32 math on the bf16 logits), gradients scaled back by the
    #     row count, in four batches to bound the host memory
    pick_all = torch.randperm(rows, generator=cg)[:1024]
    checked = 0
    for b0 in range(0, 1024, 256):
        pick = pick_all[b0:b0 + 256]
        pick = pick[target[pick] != -100]
        sub_grad = grad[pick.to(cuda_device)].double()
        assert float(sub_grad.sum(1).abs().max()) * count < 2e-2
        sub_logits = logits[pick.to(cuda_device)].float().cpu()
        eloss, egrad, bad = oracle.c_cross_entropy(sub_logits.numpy(), target[pick].numpy(), -100, eps, "none")
        assert bad == 0
        assert_close(ws.row_loss[pick.to(cuda_device)].cpu().numpy(), eloss, 2e-6, 4e-6, "row losses")
        assert_close(sub_grad.cpu().numpy() * count, egrad, 1.6e-2, 1e-4, "gradient subset")
        checked += int(pick.numel())
        del sub_grad, sub_logits, egrad
    assert checked >= 900
    del logits, grad
    torch.cuda.empty_cache()

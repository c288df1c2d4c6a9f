"""The cross-entropy entry point that brings its own scratch memory (needs a GPU; collected last).

It serves callers that cannot allocate on the device: a foreign-language host bound to the C ABI that has
no device allocator of its own, or a process whose device memory is fully committed.  The check: through the
C ABI, its loss and gradient equal those of the ordinary launch sequence (which takes caller-allocated
scratch) bit for bit, on two calls in a row that share the library's static array."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_call(logits, target, grad, loss, status, reduction, eps):
    from torch_supa_b200 import capi

    a = capi.CEArgs()
    a.logits, a.dtype, a.reduction = logits.data_ptr(), capi.torch_dtype_code(logits.dtype), reduction
    a.target, a.grad_logits = target.data_ptr(), grad.data_ptr()
    a.rows, a.classes, a.ignore_index = logits.shape[0], logits.shape[1], -100
    a.label_smoothing, a.grad_scale, a.status = eps, 1.0, status.data_ptr()
    capi.ce_loss_static_scratch(a, loss, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_caller_scratch_twice(cuda_device, dtype):
    from torch_supa_b200 import capi, functional as F2

    g = torch.Generator().manual_seed(17)
    # second call: fewer rows and other data, so stale per-row losses of the first call would show up in the sum
    for rows, classes, red_name, red, eps in ((700, 32000, "mean", capi.REDUCTION_MEAN, 0.1), (300, 5000, "sum", capi.REDUCTION_SUM, 0.0)):
        logits = (torch.randn(rows, classes, generator=g) * 2).to(dtype).to(cuda_device)
        target = torch.randint(0, classes, (rows,), generator=g)
        target[::6] = -100
        target = target.to(cuda_device)
        ref_loss, ref_grad = F2.cross_entropy_forward_backward(logits, target, label_smoothing=eps, reduction=red_name)
        grad = torch.empty_like(logits)
        loss = torch.empty((), dtype=dtype, device=cuda_device)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        _static_call(logits, target, grad, loss, status, red, eps)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert loss.item() == ref_loss.item(), "same kernels, same order: the loss is bit-identical"
        assert torch.equal(grad, ref_grad)
        # the reason this entry point exists: a repeated call (the first one per device resolves the array's address) takes no
        # memory from the device, neither through the caching allocator of the process nor behind its back
        grad.zero_()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        stats_before = torch.cuda.memory_stats()
        _static_call(logits, target, grad, loss, status, red, eps)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        stats_after = torch.cuda.memory_stats()
        assert free_after == free_before, "device memory was allocated during the call"
        for key in ("allocation.all.allocated", "segment.all.allocated", "reserved_bytes.all.current"):
            assert stats_after[key] == stats_before[key], key
        assert loss.item() == ref_loss.item() and torch.equal(grad, ref_grad)


def test_static_scratch_rejects_what_it_cannot_hold(cuda_device):
    from torch_supa_b200 import capi

    rows = capi.CE_STATIC_MAX_ROWS + 1
    logits = torch.zeros(rows, 8, device=cuda_device)
    target = torch.zeros(rows, dtype=torch.int64, device=cuda_device)
    grad = torch.empty_like(logits)
    loss = torch.empty((), device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    with pytest.raises(capi.KernelError) as err:
        _static_call(logits, target, grad, loss, status, capi.REDUCTION_MEAN, 0.0)
    assert err.value.status == -4 and "maximum" in str(err.value)
    # caller-provided scratch pointers are a misuse of this entry point
    a = capi.CEArgs()
    a.logits, a.dtype, a.reduction, a.target = logits.data_ptr(), capi.F32, capi.REDUCTION_MEAN, target.data_ptr()
    a.rows, a.classes, a.row_loss = 4, 8, grad.data_ptr()
    with pytest.raises(capi.KernelError):
        capi.ce_loss_static_scratch(a, loss)

"""Functional front-end of the C ABI for tensors whose ``data_ptr()`` is a CUDA address.

torch is used here for device memory and the current stream only; every computation is a call into
``libsupa_b200_kernels.so`` through :mod:`torch_supa_b200.capi`.  The functions accept ordinary
``device="cuda"`` tensors, which is how the parity tests and the benchmark drive the kernels at the C
boundary; the ``"supa"`` device registered by the C++ host layer reaches the same entry points
through the ATen dispatcher instead.
"""
from __future__ import annotations

import torch

from . import capi

_RED = {"none": capi.REDUCTION_NONE, "mean": capi.REDUCTION_MEAN, "sum": capi.REDUCTION_SUM}


def _stream(t: torch.Tensor) -> int:
    if t.device.type == "supa":
        return torch.supa.current_stream_handle(t.device.index)
    if t.device.type == "cuda":
        return torch.cuda.current_stream(t.device).cuda_stream
    return 0


class CrossEntropyWorkspace:
    """Device buffers one fused cross-entropy call needs besides its inputs and outputs."""

    def __init__(self, rows: int, device):
        self.row_loss = torch.empty(max(rows, 1), dtype=torch.float32, device=device)
        self.acc = torch.zeros(2, dtype=torch.float64, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


def cross_entropy_forward_backward(logits, target, *, ignore_index=-100, label_smoothing=0.0, reduction="mean",
                                   grad=None, want_grad=True, workspace=None, grad_scale=1.0, row_grad_out=None,
                                   row_lse=None, all_reduce=None, class_weight=None):
    """Fused cross entropy: returns ``(loss, grad_logits)``.

    ``loss`` is a 0-d tensor in the logits' dtype for mean/sum and an fp32 ``[rows]`` tensor for none.
    ``all_reduce``, when given, is called as ``all_reduce(acc_view)`` on a one-element float64 view of the
    device accumulator, first for the valid-row count and then for the loss sum: this is the hook the
    row-sharded multi-GPU path uses.  ``class_weight`` (fp32 ``[classes]``) multiplies each row's loss and
    gradient by the weight of its target; ``mean`` then divides by the sum of those weights; with label
    smoothing the smoothing term weights every class by its own weight, as ``F.cross_entropy`` does.
    """
    assert logits.dim() == 2 and target.dim() == 1 and logits.is_contiguous() and target.is_contiguous()
    rows, classes = logits.shape
    ws = workspace or CrossEntropyWorkspace(rows, logits.device)
    st = _stream(logits)
    if want_grad and grad is None:
        grad = torch.empty_like(logits)
    red = _RED[reduction]
    if class_weight is not None:
        assert class_weight.dtype == torch.float32 and class_weight.is_contiguous() and class_weight.numel() == classes
    if red != capi.REDUCTION_NONE:
        if class_weight is not None:
            capi.ce_count_weighted(target, class_weight, rows, classes, ignore_index, ws.acc, ws.status, st)
        else:
            capi.ce_count_valid(target, rows, classes, ignore_index, ws.acc, ws.status, st)
        if all_reduce is not None:
            all_reduce(ws.acc[1:2])
    args = capi.CEArgs()
    args.logits = logits.data_ptr()
    args.dtype = capi.torch_dtype_code(logits.dtype)
    args.reduction = red
    args.target = target.data_ptr()
    args.grad_logits = grad.data_ptr() if want_grad else None
    args.row_loss = ws.row_loss.data_ptr()
    args.row_lse = row_lse.data_ptr() if row_lse is not None else None
    args.row_grad_out = row_grad_out.data_ptr() if row_grad_out is not None else None
    args.acc = ws.acc.data_ptr()
    args.rows, args.classes, args.ignore_index = rows, classes, ignore_index
    args.label_smoothing = label_smoothing
    args.grad_scale = grad_scale
    args.status = ws.status.data_ptr()
    args.class_weight = class_weight.data_ptr() if class_weight is not None else None
    # the count is the launch directly before the sweep: the sweep may start under it
    args.flags = capi.CE_FLAG_AFTER_COUNT if (red != capi.REDUCTION_NONE and all_reduce is None) else 0
    capi.ce_forward_backward(args, st)
    if red == capi.REDUCTION_NONE:
        return ws.row_loss[:rows], (grad if want_grad else None)
    loss = torch.empty((), dtype=logits.dtype, device=logits.device)
    code = capi.torch_dtype_code(logits.dtype)
    if all_reduce is None:
        capi.ce_loss_sum_finish(ws.row_loss, rows, ws.acc, red, loss, code, st)
    else:
        capi.ce_loss_sum(ws.row_loss, rows, ws.acc, st)
        all_reduce(ws.acc[0:1])
        capi.ce_loss_finish(ws.acc, red, loss, code, st)
    return loss, (grad if want_grad else None)


def cross_entropy_prob_forward_backward(logits, target, *, label_smoothing=0.0, reduction="mean", want_grad=True, grad_scale=1.0,
                                        row_grad_out=None, class_weight=None):
    """Cross entropy with class-probability targets of the logits' shape and dtype: returns ``(loss, grad_logits)``; ``mean``
    divides by the number of rows."""
    assert logits.dim() == 2 and target.shape == logits.shape and target.dtype == logits.dtype
    assert logits.is_contiguous() and target.is_contiguous()
    rows, classes = logits.shape
    st = _stream(logits)
    row_loss = torch.empty(max(rows, 1), dtype=torch.float32, device=logits.device)
    grad = torch.empty_like(logits) if want_grad else None
    inv = 1.0 / rows if (reduction == "mean" and rows) else 1.0
    a = capi.CEProbArgs()
    a.logits, a.target, a.dtype = logits.data_ptr(), target.data_ptr(), capi.torch_dtype_code(logits.dtype)
    a.grad_logits = grad.data_ptr() if want_grad else None
    a.row_loss = row_loss.data_ptr()
    a.row_grad_out = row_grad_out.data_ptr() if row_grad_out is not None else None
    a.class_weight = class_weight.data_ptr() if class_weight is not None else None
    a.rows, a.classes, a.label_smoothing = rows, classes, label_smoothing
    a.grad_scale, a.loss_scale = grad_scale * inv, inv
    capi.ce_prob_forward_backward(a, st)
    if reduction == "none":
        return row_loss[:rows], grad
    acc = torch.zeros(2, dtype=torch.float64, device=logits.device)
    loss = torch.empty((), dtype=logits.dtype, device=logits.device)
    capi.ce_loss_sum_finish(row_loss, rows, acc, capi.REDUCTION_SUM, loss, capi.torch_dtype_code(logits.dtype), st)
    return loss, grad


def arg_reduce(x, dim, is_max=True, want_values=True):
    """(values, indices) of the extremum along ``dim`` of a contiguous tensor."""
    x = x.contiguous()
    dim %= max(x.dim(), 1)
    shape = list(x.shape) or [1]
    outer = 1
    for s_ in shape[:dim]:
        outer *= s_
    inner = 1
    for s_ in shape[dim + 1:]:
        inner *= s_
    out_shape = shape[:dim] + shape[dim + 1:]
    values = torch.empty(out_shape, dtype=x.dtype, device=x.device) if want_values else None
    indices = torch.empty(out_shape, dtype=torch.int64, device=x.device)
    code = capi.torch_dtype_code(x.dtype)
    need = capi.reduce_ext_scratch_bytes(code, outer, shape[dim], inner, False)
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=x.device)
    capi.arg_reduce(x, code, outer, shape[dim], inner, is_max, values, indices, scratch if need else None, need, _stream(x))
    return values, indices


def moments(x, dim, correction=1.0, take_sqrt=False):
    """(variance or standard deviation, mean) along ``dim`` of a contiguous floating tensor."""
    x = x.contiguous()
    dim %= max(x.dim(), 1)
    shape = list(x.shape) or [1]
    outer = 1
    for s_ in shape[:dim]:
        outer *= s_
    inner = 1
    for s_ in shape[dim + 1:]:
        inner *= s_
    out_shape = shape[:dim] + shape[dim + 1:]
    out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    mean = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    code = capi.torch_dtype_code(x.dtype)
    need = capi.reduce_ext_scratch_bytes(code, outer, shape[dim], inner, True)
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=x.device)
    capi.moments(x, code, outer, shape[dim], inner, correction, take_sqrt, out, mean, scratch if need else None, need, _stream(x))
    return out, mean


_RNG_KINDS = {"uniform": capi.SB_RNG_UNIFORM, "normal": capi.SB_RNG_NORMAL, "integer": capi.SB_RNG_INTEGER,
              "bernoulli": capi.SB_RNG_BERNOULLI}


def rng_fill(out, kind, seed, offset, a=0.0, b=1.0, low=0, range_=0):
    """Fills the contiguous tensor ``out`` from the Philox stream of (seed, offset): ``kind`` is "uniform" ([a, b)),
    "normal" (mean a, std b), "integer" (low + r mod range_) or "bernoulli" (probability a).  The caller advances the
    offset by 4 per fill."""
    assert out.is_contiguous()
    args = capi.RngArgs()
    args.dst = out.data_ptr()
    args.dtype = capi.torch_dtype_code(out.dtype)
    args.kind = _RNG_KINDS[kind]
    args.numel = out.numel()
    args.a, args.b = float(a), float(b)
    args.low = int(low)
    args.range = int(range_)
    args.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    args.offset = int(offset)
    capi.rng_fill(args, _stream(out))
    return out


def dropout(x, p, seed, offset):
    """(x * keep / (1 - p), keep) with keep drawn from the Philox stream of (seed, offset)."""
    x = x.contiguous()
    out = torch.empty_like(x)
    mask = torch.empty(x.shape, dtype=torch.bool, device=x.device)
    capi.dropout(x, out, mask, capi.torch_dtype_code(x.dtype), x.numel(), p, int(seed) & 0xFFFFFFFFFFFFFFFF, int(offset), _stream(x))
    return out, mask


def log_softmax(x, dim=-1, out_dtype=None):
    x = x.contiguous()
    dim %= max(x.dim(), 1)
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    shape = list(x.shape) or [1]
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    capi.log_softmax_forward(x, capi.torch_dtype_code(x.dtype), out, capi.torch_dtype_code(out.dtype), outer, shape[dim],
                             inner, _stream(x))
    return out


def log_softmax_backward(grad_out, out, dim=-1, input_dtype=None):
    grad_out, out = grad_out.contiguous(), out.contiguous()
    dim %= max(out.dim(), 1)
    gi = torch.empty(out.shape, dtype=input_dtype or out.dtype, device=out.device)
    shape = list(out.shape) or [1]
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    capi.log_softmax_backward(grad_out, out, capi.torch_dtype_code(out.dtype), gi, capi.torch_dtype_code(gi.dtype), outer,
                              shape[dim], inner, _stream(out))
    return gi


def softmax(x, dim=-1, out_dtype=None):
    x = x.contiguous()
    dim %= max(x.dim(), 1)
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    shape = list(x.shape) or [1]
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    capi.softmax_forward(x, capi.torch_dtype_code(x.dtype), out, capi.torch_dtype_code(out.dtype), outer, shape[dim], inner, _stream(x))
    return out


def softmax_backward(grad_out, out, dim=-1, input_dtype=None):
    grad_out, out = grad_out.contiguous(), out.contiguous()
    dim %= max(out.dim(), 1)
    gi = torch.empty(out.shape, dtype=input_dtype or out.dtype, device=out.device)
    shape = list(out.shape) or [1]
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    capi.softmax_backward(grad_out, out, capi.torch_dtype_code(out.dtype), gi, capi.torch_dtype_code(gi.dtype), outer, shape[dim],
                          inner, _stream(out))
    return gi


def _nll_args(logp, target, weight, ignore_index, reduction, status):
    a = capi.NLLArgs()
    a.log_probs = logp.data_ptr()
    a.dtype = capi.torch_dtype_code(logp.dtype)
    a.target_dtype = capi.torch_dtype_code(target.dtype)
    a.target = target.data_ptr()
    a.weight = weight.data_ptr() if weight is not None else None
    a.rows, a.classes = logp.shape
    a.ignore_index = ignore_index
    a.reduction = _RED[reduction]
    a.status = status.data_ptr() if status is not None else None
    return a


def nll_loss_forward(logp, target, weight=None, ignore_index=-100, reduction="mean", status=None):
    logp, target = logp.contiguous(), target.contiguous()
    rows = logp.shape[0]
    out = torch.empty(rows if reduction == "none" else (), dtype=logp.dtype, device=logp.device)
    total_weight = torch.zeros((), dtype=logp.dtype, device=logp.device)
    capi.nll_loss_forward(_nll_args(logp, target, weight, ignore_index, reduction, status), out, total_weight, _stream(logp))
    return out, total_weight


def nll_loss_backward(grad_out, logp, target, weight=None, ignore_index=-100, reduction="mean", total_weight=None,
                      status=None):
    logp, target = logp.contiguous(), target.contiguous()
    gi = torch.empty_like(logp)
    capi.nll_loss_backward(_nll_args(logp, target, weight, ignore_index, reduction, status), grad_out.contiguous(),
                           total_weight, gi, _stream(logp))
    return gi


def _nll_nd_args(logp, target, weight, ignore_index, reduction, status):
    a = capi.NLLNdArgs()
    a.log_probs = logp.data_ptr()
    a.dtype = capi.torch_dtype_code(logp.dtype)
    a.target_dtype = capi.torch_dtype_code(target.dtype)
    a.target = target.data_ptr()
    a.weight = weight.data_ptr() if weight is not None else None
    a.outer, a.classes = logp.shape[0], logp.shape[1]
    inner = 1
    for s in logp.shape[2:]:
        inner *= s
    a.inner = inner
    a.ignore_index = ignore_index
    a.reduction = _RED[reduction]
    a.status = status.data_ptr() if status is not None else None
    return a


def nll_loss_nd_forward(logp, target, weight=None, ignore_index=-100, reduction="mean", status=None):
    """nll_loss for ``logp`` of shape (N, C, d1, ...) and ``target`` of shape (N, d1, ...)."""
    logp, target = logp.contiguous(), target.contiguous()
    out = torch.empty(target.shape if reduction == "none" else (), dtype=logp.dtype, device=logp.device)
    total_weight = torch.zeros((), dtype=logp.dtype, device=logp.device)
    a = _nll_nd_args(logp, target, weight, ignore_index, reduction, status)
    need = capi.nll_loss_nd_scratch_bytes(a)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=logp.device)
    a.scratch, a.scratch_bytes = scratch.data_ptr(), need
    capi.nll_loss_nd_forward(a, out, total_weight, _stream(logp))
    return out, total_weight


def nll_loss_nd_backward(grad_out, logp, target, weight=None, ignore_index=-100, reduction="mean", total_weight=None,
                         status=None):
    logp, target = logp.contiguous(), target.contiguous()
    gi = torch.empty_like(logp)
    a = _nll_nd_args(logp, target, weight, ignore_index, reduction, status)
    capi.nll_loss_nd_backward(a, grad_out.contiguous(), total_weight, gi, _stream(logp))
    return gi


def bce_with_logits_reduce(x, target, pos_weight=None, weight=None, reduction="mean"):
    """Fused binary_cross_entropy_with_logits + mean / sum for contiguous same-dtype inputs; ``pos_weight`` runs
    along the last dimension."""
    x, target = x.contiguous(), target.contiguous()
    out = torch.empty((), dtype=x.dtype, device=x.device)
    need = capi.bce_logits_scratch_bytes(x.numel())
    scratch = torch.empty(max(need, 8), dtype=torch.uint8, device=x.device)
    capi.bce_logits_reduce(x, target, pos_weight, 0 if pos_weight is None else pos_weight.numel(),
                           None if weight is None else weight.contiguous(), capi.torch_dtype_code(x.dtype), x.numel(),
                           _RED[reduction], out, scratch, need, _stream(x))
    return out


def elementwise(op, out, *inputs, common_dtype=None, alpha=1.0, scalar=0.0):
    """out = op(*inputs) with broadcasting to ``out.shape``; strides of every operand are honoured."""
    desc = capi.make_ew_desc(op, out, inputs, common_dtype=common_dtype, alpha=alpha, scalar=scalar)
    capi.elementwise(desc, _stream(out))
    return out


def reduce(op, inp, dims, keepdim=False, out_dtype=None):
    """sum / mean / amax / amin of ``inp`` over ``dims`` (a list of dimensions)."""
    nd = inp.dim()
    dims = sorted({d % nd for d in dims}) if nd else []
    shape = [s for d, s in enumerate(inp.shape) if d not in dims] if not keepdim else \
        [1 if d in dims else s for d, s in enumerate(inp.shape)]
    if out_dtype is None:
        integral = inp.dtype in (torch.bool, torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64)
        out_dtype = torch.int64 if (integral and op == capi.RED_SUM) else inp.dtype
    out = torch.empty(shape, dtype=out_dtype, device=inp.device)
    desc = capi.make_reduce_desc(op, inp, out, dims)
    need = capi.reduce_scratch_bytes(desc)
    scratch = None
    if need:
        scratch = torch.empty(need, dtype=torch.uint8, device=inp.device)
        desc.scratch = scratch.data_ptr()
        desc.scratch_bytes = need
    capi.reduce(desc, _stream(inp))
    return out

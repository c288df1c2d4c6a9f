"""ctypes view of the C ABI in ``include/supa_b200_kernels.h``.

This is the binding a host written in another language would make: it passes raw device pointers,
sizes and a stream handle, and nothing torch-specific crosses the boundary.  The GPU parity tests and
``bench.py`` call the kernels through it.  There is no fallback: if the shared library has not been
built, importing the symbols raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsupa_b200_kernels.so"

SB_MAX_DIMS = 25
SB_MAX_OPERANDS = 4

# sb_dtype
BOOL, U8, I8, I16, I32, I64, F16, BF16, F32, F64 = range(10)
# sb_reduction
REDUCTION_NONE, REDUCTION_MEAN, REDUCTION_SUM = 0, 1, 2
STATUS_TARGET_OUT_OF_RANGE = 0x1
STATUS_KERNEL_TIMEOUT = 0x2
STATUS_GRADIENT_LOST = 0x4

# sb_ew_op
(EW_COPY, EW_FILL, EW_ADD, EW_MUL, EW_SUB, EW_DIV, EW_GELU_ERF, EW_GELU_TANH, EW_SILU, EW_GLU, EW_GELU_ERF_BWD,
 EW_GELU_TANH_BWD, EW_SILU_BWD, EW_GLU_BWD_A, EW_GLU_BWD_B, EW_ADD_SCALAR, EW_MUL_SCALAR, EW_NEG, EW_BCE_LOGITS,
 EW_BCE_LOGITS_PW, EW_BCE_LOGITS_BWD, EW_BCE_LOGITS_PW_BWD, EW_SIGMOID, EW_TANH, EW_EXP, EW_LOG, EW_SIGMOID_BWD, EW_TANH_BWD,
 EW_MAXIMUM, EW_MINIMUM, EW_EQ, EW_NE, EW_LT, EW_LE, EW_GT, EW_GE, EW_WHERE, EW_MASKED_FILL, EW_DIV_TRUNC, EW_DIV_FLOOR) = range(40)
# sb_reduce_op
RED_SUM, RED_MEAN, RED_AMAX, RED_AMIN, RED_PROD, RED_NANSUM = range(6)


class CEArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("dtype", C.c_int32), ("reduction", C.c_int32), ("target", C.c_void_p),
        ("grad_logits", C.c_void_p), ("row_loss", C.c_void_p), ("row_lse", C.c_void_p),
        ("row_grad_out", C.c_void_p), ("acc", C.c_void_p), ("rows", C.c_int64), ("classes", C.c_int64),
        ("ignore_index", C.c_int64), ("label_smoothing", C.c_float), ("grad_scale", C.c_float),
        ("status", C.c_void_p), ("class_weight", C.c_void_p), ("flags", C.c_uint32),
    ]


CE_FLAG_AFTER_COUNT = 0x1
XCHG_MAX_RANKS, XCHG_DEPTH = 8, 4
XCHG_SLOT_BYTES = XCHG_DEPTH * XCHG_MAX_RANKS * 16


class Xchg(C.Structure):
    """sb_xchg: where the ranks of a row-sharded job publish their partial sums."""
    _fields_ = [("slots", C.c_void_p * XCHG_MAX_RANKS), ("rank", C.c_int32), ("nranks", C.c_int32), ("seq", C.c_uint64)]


class CEProbArgs(C.Structure):
    """sb_ce_prob_args: cross entropy with class-probability targets."""
    _fields_ = [
        ("logits", C.c_void_p), ("target", C.c_void_p), ("dtype", C.c_int32), ("grad_logits", C.c_void_p), ("row_loss", C.c_void_p),
        ("row_grad_out", C.c_void_p), ("class_weight", C.c_void_p), ("rows", C.c_int64), ("classes", C.c_int64),
        ("label_smoothing", C.c_float), ("grad_scale", C.c_float), ("loss_scale", C.c_float),
    ]


class RngArgs(C.Structure):
    """sb_rng_args: a random fill from a (seed, offset) pair."""
    _fields_ = [
        ("dst", C.c_void_p), ("dtype", C.c_int32), ("kind", C.c_int32), ("numel", C.c_int64), ("a", C.c_double), ("b", C.c_double),
        ("low", C.c_int64), ("range", C.c_uint64), ("seed", C.c_uint64), ("offset", C.c_uint64),
    ]


SB_RNG_UNIFORM, SB_RNG_NORMAL, SB_RNG_INTEGER, SB_RNG_BERNOULLI = 0, 1, 2, 3


class NLLArgs(C.Structure):
    _fields_ = [
        ("log_probs", C.c_void_p), ("dtype", C.c_int32), ("target_dtype", C.c_int32), ("target", C.c_void_p),
        ("weight", C.c_void_p), ("rows", C.c_int64), ("classes", C.c_int64), ("ignore_index", C.c_int64),
        ("reduction", C.c_int32), ("status", C.c_void_p),
    ]


class NLLNdArgs(C.Structure):
    _fields_ = [
        ("log_probs", C.c_void_p), ("dtype", C.c_int32), ("target_dtype", C.c_int32), ("target", C.c_void_p),
        ("weight", C.c_void_p), ("outer", C.c_int64), ("classes", C.c_int64), ("inner", C.c_int64),
        ("ignore_index", C.c_int64), ("reduction", C.c_int32), ("status", C.c_void_p), ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_size_t),
    ]


class EWDesc(C.Structure):
    _fields_ = [
        ("op", C.c_int32), ("ndim", C.c_int32), ("noperands", C.c_int32), ("common_dtype", C.c_int32),
        ("sizes", C.c_int64 * SB_MAX_DIMS), ("strides", (C.c_int64 * SB_MAX_DIMS) * SB_MAX_OPERANDS),
        ("data", C.c_void_p * SB_MAX_OPERANDS), ("dtype", C.c_int32 * SB_MAX_OPERANDS),
        ("alpha", C.c_double), ("ialpha", C.c_int64), ("scalar", C.c_double), ("iscalar", C.c_int64),
    ]


class ReduceDesc(C.Structure):
    _fields_ = [
        ("op", C.c_int32), ("ndim", C.c_int32), ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("sizes", C.c_int64 * SB_MAX_DIMS), ("in_strides", C.c_int64 * SB_MAX_DIMS),
        ("out_strides", C.c_int64 * SB_MAX_DIMS), ("in_", C.c_void_p), ("out", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
    ]


class KernelError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded kernel library; raises if it was not built (there is no CPU path behind it)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m torch_supa_b200._build` "
                "(the operators have no fallback implementation)")
        _lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
        _lib.sb_version.restype = C.c_char_p
        _lib.sb_status_string.restype = C.c_char_p
        _lib.sb_status_string.argtypes = [C.c_int]
        _lib.sb_dtype_size.restype = C.c_size_t
        _lib.sb_reduce_scratch_bytes.restype = C.c_size_t
        _lib.sb_nll_loss_nd_scratch_bytes.restype = C.c_size_t
        _lib.sb_bce_logits_scratch_bytes.restype = C.c_size_t
        _lib.sb_reduce_ext_scratch_bytes.restype = C.c_size_t
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        raise KernelError(fn, status, lib().sb_status_string(status).decode())


def _p(x) -> C.c_void_p:
    """Device address of a torch tensor, an int address, or None."""
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, int):
        return C.c_void_p(x)
    return C.c_void_p(x.data_ptr())


def torch_dtype_code(dt) -> int:
    import torch

    table = {torch.bool: BOOL, torch.uint8: U8, torch.int8: I8, torch.int16: I16, torch.int32: I32,
             torch.int64: I64, torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.float64: F64}
    return table[dt]


# ---- thin callable wrappers (raise on a non-zero status) ------------------------------------------

def ce_count_valid(target, rows, classes, ignore_index, acc, status=None, stream=0):
    check("sb_ce_count_valid", lib().sb_ce_count_valid(_p(target), C.c_int64(rows), C.c_int64(classes),
                                                       C.c_int64(ignore_index), _p(acc), _p(status), C.c_void_p(stream)))


def ce_count_weighted(target, class_weight, rows, classes, ignore_index, acc, status=None, stream=0):
    check("sb_ce_count_weighted", lib().sb_ce_count_weighted(_p(target), _p(class_weight), C.c_int64(rows), C.c_int64(classes),
                                                             C.c_int64(ignore_index), _p(acc), _p(status), C.c_void_p(stream)))


def ce_forward_backward(args: CEArgs, stream=0):
    check("sb_ce_forward_backward", lib().sb_ce_forward_backward(C.byref(args), C.c_void_p(stream)))


def ce_loss_sum(row_loss, rows, acc, stream=0):
    check("sb_ce_loss_sum", lib().sb_ce_loss_sum(_p(row_loss), C.c_int64(rows), _p(acc), C.c_void_p(stream)))


def ce_loss_finish(acc, reduction, out, dtype, stream=0):
    check("sb_ce_loss_finish", lib().sb_ce_loss_finish(_p(acc), C.c_int32(reduction), _p(out), C.c_int32(dtype),
                                                       C.c_void_p(stream)))


def ce_loss_sum_finish(row_loss, rows, acc, reduction, out, dtype, stream=0):
    check("sb_ce_loss_sum_finish", lib().sb_ce_loss_sum_finish(_p(row_loss), C.c_int64(rows), _p(acc),
                                                               C.c_int32(reduction), _p(out), C.c_int32(dtype),
                                                               C.c_void_p(stream)))


def ce_rescale_grad(src, dst, dtype, numel, scale, scale_dtype, applied_in, applied_out, status=None, stream=0):
    check("sb_ce_rescale_grad", lib().sb_ce_rescale_grad(_p(src), _p(dst), C.c_int32(dtype), C.c_int64(numel), _p(scale),
                                                         C.c_int32(scale_dtype), _p(applied_in), _p(applied_out), _p(status),
                                                         C.c_void_p(stream)))


def ce_count_exchange(target, class_weight, rows, classes, ignore_index, acc, status=None, xchg: "Xchg | None" = None, stream=0):
    check("sb_ce_count_exchange", lib().sb_ce_count_exchange(_p(target), _p(class_weight), C.c_int64(rows), C.c_int64(classes),
                                                             C.c_int64(ignore_index), _p(acc), _p(status),
                                                             C.byref(xchg) if xchg is not None else None, C.c_void_p(stream)))


def ce_loss_exchange(row_loss, rows, acc, reduction, out, dtype, status=None, xchg: "Xchg | None" = None, stream=0):
    check("sb_ce_loss_exchange", lib().sb_ce_loss_exchange(_p(row_loss), C.c_int64(rows), _p(acc), C.c_int32(reduction), _p(out),
                                                           C.c_int32(dtype), _p(status),
                                                           C.byref(xchg) if xchg is not None else None, C.c_void_p(stream)))


CE_STATIC_MAX_ROWS = 65536


def ce_loss_static_scratch(args: CEArgs, loss_out, stream=0):
    """Whole mean/sum cross entropy with the scratch buffers inside the library (no device allocation)."""
    check("sb_ce_loss_static_scratch", lib().sb_ce_loss_static_scratch(C.byref(args), _p(loss_out), C.c_void_p(stream)))


def ce_prob_forward_backward(args: CEProbArgs, stream=0):
    check("sb_ce_prob_forward_backward", lib().sb_ce_prob_forward_backward(C.byref(args), C.c_void_p(stream)))


def reduce_ext_scratch_bytes(dtype, outer, length, inner, moments) -> int:
    return int(lib().sb_reduce_ext_scratch_bytes(C.c_int32(dtype), C.c_int64(outer), C.c_int64(length), C.c_int64(inner),
                                                 C.c_int32(1 if moments else 0)))


def arg_reduce(inp, dtype, outer, length, inner, is_max, values, indices, scratch=None, scratch_bytes=0, stream=0):
    check("sb_arg_reduce", lib().sb_arg_reduce(_p(inp), C.c_int32(dtype), C.c_int64(outer), C.c_int64(length), C.c_int64(inner),
                                               C.c_int32(1 if is_max else 0), _p(values), _p(indices), _p(scratch),
                                               C.c_size_t(scratch_bytes), C.c_void_p(stream)))


def moments(inp, dtype, outer, length, inner, correction, take_sqrt, out, mean_out=None, scratch=None, scratch_bytes=0, stream=0):
    check("sb_moments", lib().sb_moments(_p(inp), C.c_int32(dtype), C.c_int64(outer), C.c_int64(length), C.c_int64(inner),
                                         C.c_double(correction), C.c_int32(1 if take_sqrt else 0), _p(out), _p(mean_out), _p(scratch),
                                         C.c_size_t(scratch_bytes), C.c_void_p(stream)))


def rng_fill(args: RngArgs, stream=0):
    check("sb_rng_fill", lib().sb_rng_fill(C.byref(args), C.c_void_p(stream)))


def dropout(x, out, mask, dtype, numel, p, seed, offset, stream=0):
    check("sb_dropout", lib().sb_dropout(_p(x), _p(out), _p(mask), C.c_int32(dtype), C.c_int64(numel), C.c_double(p),
                                         C.c_uint64(seed), C.c_uint64(offset), C.c_void_p(stream)))


def ce_kernel_variant(dtype, rows, classes) -> int:
    return lib().sb_ce_kernel_variant(C.c_int32(dtype), C.c_int64(rows), C.c_int64(classes))


def log_softmax_forward(inp, in_dtype, out, out_dtype, outer, dim, inner, stream=0):
    check("sb_log_softmax_forward", lib().sb_log_softmax_forward(_p(inp), C.c_int32(in_dtype), _p(out),
                                                                 C.c_int32(out_dtype), C.c_int64(outer), C.c_int64(dim),
                                                                 C.c_int64(inner), C.c_void_p(stream)))


def log_softmax_backward(grad_out, out, dtype, grad_in, grad_in_dtype, outer, dim, inner, stream=0):
    check("sb_log_softmax_backward", lib().sb_log_softmax_backward(_p(grad_out), _p(out), C.c_int32(dtype), _p(grad_in),
                                                                   C.c_int32(grad_in_dtype), C.c_int64(outer),
                                                                   C.c_int64(dim), C.c_int64(inner), C.c_void_p(stream)))


def softmax_forward(inp, in_dtype, out, out_dtype, outer, dim, inner, stream=0):
    check("sb_softmax_forward", lib().sb_softmax_forward(_p(inp), C.c_int32(in_dtype), _p(out), C.c_int32(out_dtype), C.c_int64(outer),
                                                         C.c_int64(dim), C.c_int64(inner), C.c_void_p(stream)))


def softmax_backward(grad_out, out, dtype, grad_in, grad_in_dtype, outer, dim, inner, stream=0):
    check("sb_softmax_backward", lib().sb_softmax_backward(_p(grad_out), _p(out), C.c_int32(dtype), _p(grad_in), C.c_int32(grad_in_dtype),
                                                           C.c_int64(outer), C.c_int64(dim), C.c_int64(inner), C.c_void_p(stream)))


def nll_loss_forward(args: NLLArgs, output, total_weight, stream=0):
    check("sb_nll_loss_forward", lib().sb_nll_loss_forward(C.byref(args), _p(output), _p(total_weight), C.c_void_p(stream)))


def nll_loss_backward(args: NLLArgs, grad_output, total_weight, grad_input, stream=0):
    check("sb_nll_loss_backward", lib().sb_nll_loss_backward(C.byref(args), _p(grad_output), _p(total_weight),
                                                             _p(grad_input), C.c_void_p(stream)))


def nll_loss_nd_scratch_bytes(args: NLLNdArgs) -> int:
    return int(lib().sb_nll_loss_nd_scratch_bytes(C.byref(args)))


def nll_loss_nd_forward(args: NLLNdArgs, output, total_weight, stream=0):
    check("sb_nll_loss_nd_forward", lib().sb_nll_loss_nd_forward(C.byref(args), _p(output), _p(total_weight), C.c_void_p(stream)))


def nll_loss_nd_backward(args: NLLNdArgs, grad_output, total_weight, grad_input, stream=0):
    check("sb_nll_loss_nd_backward", lib().sb_nll_loss_nd_backward(C.byref(args), _p(grad_output), _p(total_weight),
                                                                   _p(grad_input), C.c_void_p(stream)))


def bce_logits_scratch_bytes(numel: int) -> int:
    return int(lib().sb_bce_logits_scratch_bytes(C.c_int64(numel)))


def bce_logits_reduce(x, target, pos_weight, pw_len, weight, dtype, numel, reduction, out, scratch, scratch_bytes, stream=0):
    check("sb_bce_logits_reduce", lib().sb_bce_logits_reduce(_p(x), _p(target), _p(pos_weight), C.c_int64(pw_len), _p(weight),
                                                             C.c_int32(dtype), C.c_int64(numel), C.c_int32(reduction), _p(out),
                                                             _p(scratch), C.c_size_t(scratch_bytes), C.c_void_p(stream)))


def elementwise(desc: EWDesc, stream=0):
    check("sb_elementwise", lib().sb_elementwise(C.byref(desc), C.c_void_p(stream)))


def elementwise_path(desc: EWDesc) -> int:
    return lib().sb_elementwise_path(C.byref(desc))


def reduce_scratch_bytes(desc: ReduceDesc) -> int:
    return lib().sb_reduce_scratch_bytes(C.byref(desc))


def reduce(desc: ReduceDesc, stream=0):
    check("sb_reduce", lib().sb_reduce(C.byref(desc), C.c_void_p(stream)))


def reduce_path(desc: ReduceDesc) -> int:
    return lib().sb_reduce_path(C.byref(desc))


# ---- descriptor builders from torch tensors (any device whose data_ptr() is a CUDA address) ------

def make_ew_desc(op, out, inputs, common_dtype=None, alpha=1.0, scalar=0.0, coalesce=True) -> EWDesc:
    """Builds an elementwise descriptor the way TensorIterator would: broadcast to the output's shape,
    dimensions fastest-first, adjacent dimensions merged when every operand allows it."""
    import torch

    shape = list(out.shape) if out.dim() > 0 else [1]
    ops = [out] + list(inputs)
    strides = []
    for t in ops:
        tt = t if t.dim() > 0 else t.reshape(1)
        tt = tt.expand(shape) if list(tt.shape) != shape else tt
        strides.append(list(tt.stride()))
    # fastest-first: order dims by the output's stride (ascending), size-1 dims dropped
    dims = [d for d in range(len(shape)) if shape[d] != 1] or [len(shape) - 1]
    dims.sort(key=lambda d: (strides[0][d], -d))
    sizes = [shape[d] for d in dims]
    strs = [[s[d] for d in dims] for s in strides]
    if coalesce:
        i = 0
        while i + 1 < len(sizes):
            if all(st[i + 1] == st[i] * sizes[i] for st in strs):
                sizes[i] *= sizes[i + 1]
                del sizes[i + 1]
                for st in strs:
                    del st[i + 1]
            else:
                i += 1
    d = EWDesc()
    d.op = op
    d.ndim = len(sizes)
    d.noperands = len(ops)
    if common_dtype is None:
        common_dtype = out.dtype if not inputs else torch.result_type(*inputs[:2]) if len(inputs) > 1 else inputs[0].dtype
    d.common_dtype = torch_dtype_code(common_dtype)
    for i, s in enumerate(sizes):
        d.sizes[i] = s
    for k, st in enumerate(strs):
        for i, s in enumerate(st):
            d.strides[k][i] = s
        d.data[k] = ops[k].data_ptr()
        d.dtype[k] = torch_dtype_code(ops[k].dtype)
    d.alpha = float(alpha)
    d.ialpha = int(alpha) if float(alpha).is_integer() else 0
    d.scalar = float(scalar)
    d.iscalar = int(scalar) if float(scalar).is_integer() else 0
    return d


def make_reduce_desc(op, inp, out, dims, scratch=None) -> ReduceDesc:
    """Reduce `inp` over `dims` into `out` (shape of inp with reduced dims removed or kept as 1)."""
    nd = inp.dim()
    dims = sorted(d % nd for d in dims)
    out_full = out
    if out.dim() != nd:
        shape = [1 if d in dims else inp.shape[d] for d in range(nd)]
        out_full = out.reshape(shape)
    order = sorted(range(nd), key=lambda d: (inp.stride(d), -d))
    d = ReduceDesc()
    d.op = op
    k = 0
    for dim in order:
        if inp.shape[dim] == 1:
            continue
        d.sizes[k] = inp.shape[dim]
        d.in_strides[k] = inp.stride(dim)
        d.out_strides[k] = 0 if dim in dims else out_full.stride(dim)
        k += 1
    if k == 0:
        d.sizes[0], d.in_strides[0], d.out_strides[0] = 1, 1, 0
        k = 1
    d.ndim = k
    d.in_dtype = torch_dtype_code(inp.dtype)
    d.out_dtype = torch_dtype_code(out.dtype)
    d.in_ = inp.data_ptr()
    d.out = out.data_ptr()
    if scratch is not None:
        d.scratch = scratch.data_ptr()
        d.scratch_bytes = scratch.numel() * scratch.element_size()
    return d

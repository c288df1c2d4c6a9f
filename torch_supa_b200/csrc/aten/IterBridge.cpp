// TensorIterator -> C-ABI descriptors, and the PrivateUse1 slots of the ATen dispatch stubs.
//
// libtorch's TensorIterator has already done broadcasting, type promotion, dimension reordering and
// coalescing when a stub is called (the meta step of the structured operators); what is left is to hand
// shapes, element strides, dtypes and pointers to the kernel library.  This is the role gpu_kernel /
// gpu_reduce_kernel play in the reference (torch_supa/csrc/aten/ops/kernels/elementwise/Loops.cpp:110-134,
// reduce/Reduce.cuh:1231-1333); the stub registrations mirror REGISTER_PRIVATEUSE1_DISPATCH in
// kernels/kernelDispatch.h:11-28.
#include <ATen/native/Activation.h>
#include <ATen/native/BinaryOps.h>
#include <ATen/native/DispatchStub.h>
#include <ATen/native/ReduceOps.h>
#include <ATen/native/TensorCompare.h>
#include <ATen/native/TensorIterator.h>
#include <ATen/native/UnaryOps.h>

#include "Common.h"

namespace supa {

namespace {

// A CPU 0-dim operand ("wrapped number" or scalar tensor): its value, read on the host.
at::Scalar cpu_scalar_value(at::TensorIteratorBase& iter, int arg) { return iter.scalar_value<at::Scalar>(arg); }

void fill_operand(sb_ew_desc& d, int k, at::TensorIteratorBase& iter, int arg) {
  const int64_t es = static_cast<int64_t>(c10::elementSize(iter.dtype(arg)));
  d.data[k] = iter.data_ptr(arg);
  d.dtype[k] = dtype_code(iter.dtype(arg));
  const auto strides = iter.strides(arg);
  for (int i = 0; i < iter.ndim(); ++i) {
    TORCH_INTERNAL_ASSERT(strides[i] % es == 0, "supa: byte stride is not a multiple of the element size");
    d.strides[k][i] = strides[i] / es;
  }
}

void fill_shape(sb_ew_desc& d, at::TensorIteratorBase& iter) {
  TORCH_CHECK(iter.ndim() <= SB_MAX_DIMS, "supa: tensors with more than ", SB_MAX_DIMS, " non-coalescible dimensions are not supported");
  d.ndim = iter.ndim();
  for (int i = 0; i < iter.ndim(); ++i) d.sizes[i] = iter.shape()[i];
  if (d.ndim == 0) {  // 0-dim tensors
    d.ndim = 1;
    d.sizes[0] = 1;
  }
}

}  // namespace

void launch_elementwise(at::TensorIteratorBase& iter, int op, at::ScalarType common, double alpha, int64_t ialpha, double scalar,
                        int64_t iscalar) {
  if (iter.numel() == 0) return;
  TORCH_CHECK(iter.noutputs() == 1, "supa: elementwise kernels have exactly one output");
  TORCH_CHECK(iter.device_type(0) == c10::DeviceType::PrivateUse1, "supa: output must be a supa tensor");
  sb_ew_desc d{};
  d.op = op;
  d.noperands = iter.ntensors();
  TORCH_CHECK(d.noperands <= SB_MAX_OPERANDS, "supa: too many operands");
  d.common_dtype = dtype_code(common);
  fill_shape(d, iter);
  for (int k = 0; k < iter.ntensors(); ++k) {
    TORCH_CHECK(iter.device_type(k) == c10::DeviceType::PrivateUse1, "supa: expected all tensors to be on a supa device, operand ", k,
                " is on ", iter.device(k));
    fill_operand(d, k, iter, k);
  }
  d.alpha = alpha;
  d.ialpha = ialpha;
  d.scalar = scalar;
  d.iscalar = iscalar;
  const c10::Device dev = iter.device(0);
  const c10::DeviceGuard guard(dev);
  check_kernel(sb_elementwise(&d, static_cast<sb_stream_t>(current_cuda_stream(dev.index()))), "supa elementwise kernel");
}

namespace {

struct ScalarPair {
  double d = 0.0;
  int64_t i = 0;
};
ScalarPair split_scalar(const at::Scalar& s, at::ScalarType common) {
  ScalarPair r;
  if (c10::isFloatingType(common)) r.d = s.to<double>();
  else if (common == at::kBool) r.i = s.to<bool>() ? 1 : 0;
  else r.i = s.to<int64_t>();
  return r;
}

// Launches a binary-style kernel where one input may be a CPU scalar: the scalar is lifted into the
// kernel parameters (Loops.cuh:211-249 does the same with opmath_symmetric_gpu_kernel_with_scalars).
// `scalar_op` is the unary kernel "tensor (op) scalar"; when the scalar is the *first* operand and the op
// is not symmetric in it, `materialize` is used instead: the scalar is copied into a device 0-dim tensor
// and broadcast.
void launch_binary(at::TensorIteratorBase& iter, int tensor_op, int scalar_op, bool scalar_first_ok, double alpha, int64_t ialpha) {
  if (iter.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  const bool s1 = iter.is_cpu_scalar(1), s2 = iter.is_cpu_scalar(2);
  TORCH_CHECK(!(s1 && s2), "supa: both operands are CPU scalars");
  if (!s1 && !s2) {
    launch_elementwise(iter, tensor_op, common, alpha, ialpha);
    return;
  }
  const int sarg = s1 ? 1 : 2, targ = s1 ? 2 : 1;
  const at::Scalar value = cpu_scalar_value(iter, sarg);
  const c10::Device dev = iter.device(0);
  const c10::DeviceGuard guard(dev);
  sb_ew_desc d{};
  d.common_dtype = dtype_code(common);
  fill_shape(d, iter);
  fill_operand(d, 0, iter, 0);
  fill_operand(d, 1, iter, targ);
  d.alpha = alpha;
  d.ialpha = ialpha;
  if (scalar_op >= 0 && (s2 || scalar_first_ok)) {
    const ScalarPair sp = split_scalar(value, common);
    d.op = scalar_op;
    d.noperands = 2;
    d.scalar = sp.d;
    d.iscalar = sp.i;
  } else {
    // keep operand order: in0 = scalar (device 0-dim, stride 0), in1 = tensor, or the other way round
    at::Tensor dev_scalar = at::empty({}, at::TensorOptions().dtype(common).device(dev));
    dev_scalar.fill_(value);
    d.op = tensor_op;
    d.noperands = 3;
    if (s1) {
      for (int i = 0; i < SB_MAX_DIMS; ++i) d.strides[2][i] = d.strides[1][i];
      d.data[2] = d.data[1];
      d.dtype[2] = d.dtype[1];
      for (int i = 0; i < SB_MAX_DIMS; ++i) d.strides[1][i] = 0;
      d.data[1] = dev_scalar.data_ptr();
      d.dtype[1] = dtype_code(common);
    } else {
      for (int i = 0; i < SB_MAX_DIMS; ++i) d.strides[2][i] = 0;
      d.data[2] = dev_scalar.data_ptr();
      d.dtype[2] = dtype_code(common);
    }
    // dev_scalar is freed in stream order after the launch below
    check_kernel(sb_elementwise(&d, static_cast<sb_stream_t>(current_cuda_stream(dev.index()))), "supa elementwise kernel");
    return;
  }
  check_kernel(sb_elementwise(&d, static_cast<sb_stream_t>(current_cuda_stream(dev.index()))), "supa elementwise kernel");
}

void alpha_parts(const at::Scalar& alpha, at::ScalarType common, double& a, int64_t& ia) {
  a = 1.0;
  ia = 1;
  if (c10::isFloatingType(common)) a = alpha.to<double>();
  else if (common == at::kBool) ia = alpha.to<bool>() ? 1 : 0;
  else ia = alpha.to<int64_t>();
}

// ---- stub kernels (signatures fixed by ATen's DispatchStub declarations) ---------------------------------------
void add_kernel(at::TensorIteratorBase& iter, const at::Scalar& alpha) {
  double a;
  int64_t ia;
  alpha_parts(alpha, iter.common_dtype(), a, ia);
  // scalar + alpha * tensor is "tensor + scalar" only when alpha is 1
  const bool alpha_is_one = c10::isFloatingType(iter.common_dtype()) ? a == 1.0 : ia == 1;
  launch_binary(iter, SB_EW_ADD, SB_EW_ADD_SCALAR, /*scalar_first_ok=*/alpha_is_one, a, ia);
}

void mul_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_MUL, SB_EW_MUL_SCALAR, /*scalar_first_ok=*/true, 1.0, 1); }

void div_true_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_DIV, -1, false, 1.0, 1); }
// div with rounding_mode = "trunc" / "floor" (torch_supa/csrc/aten/ops/kernels/elementwise/BinaryDivTruncKernel.cu, BinaryDivFloorKernel.cu)
void div_trunc_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_DIV_TRUNC, -1, false, 1.0, 1); }
void div_floor_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_DIV_FLOOR, -1, false, 1.0, 1); }

void neg_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_NEG, iter.common_dtype()); }

void gelu_kernel(at::TensorIteratorBase& iter, at::native::GeluType approximate) {
  launch_elementwise(iter, approximate == at::native::GeluType::Tanh ? SB_EW_GELU_TANH : SB_EW_GELU_ERF, iter.common_dtype());
}
void gelu_backward_kernel(at::TensorIteratorBase& iter, at::native::GeluType approximate) {
  launch_elementwise(iter, approximate == at::native::GeluType::Tanh ? SB_EW_GELU_TANH_BWD : SB_EW_GELU_ERF_BWD, iter.common_dtype());
}
void silu_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_SILU, iter.common_dtype()); }
void silu_backward_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_SILU_BWD, iter.common_dtype()); }
// glu: the iterator's inputs are the two halves of the split dimension (strided views).
void glu_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_GLU, iter.common_dtype()); }

// Neighbouring TensorIterator operators on the same engine.
void sigmoid_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_SIGMOID, iter.common_dtype()); }
void tanh_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_TANH, iter.common_dtype()); }
void exp_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_EXP, iter.common_dtype()); }
void log_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_LOG, iter.common_dtype()); }
void sigmoid_backward_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_SIGMOID_BWD, iter.common_dtype()); }
void tanh_backward_kernel(at::TensorIteratorBase& iter) { launch_elementwise(iter, SB_EW_TANH_BWD, iter.common_dtype()); }
void maximum_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_MAXIMUM, -1, false, 1.0, 1); }
void minimum_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_MINIMUM, -1, false, 1.0, 1); }
void eq_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_EQ, -1, false, 1.0, 1); }
void ne_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_NE, -1, false, 1.0, 1); }
void lt_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_LT, -1, false, 1.0, 1); }
void le_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_LE, -1, false, 1.0, 1); }
void gt_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_GT, -1, false, 1.0, 1); }
void ge_kernel(at::TensorIteratorBase& iter) { launch_binary(iter, SB_EW_GE, -1, false, 1.0, 1); }
// where(condition, self, other): operand 1 is the condition; the values share a dtype (libtorch promotes them first)
void where_kernel_supa(at::TensorIterator& iter) { launch_elementwise(iter, SB_EW_WHERE, iter.dtype(2)); }

void sum_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_SUM); }
void mean_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_MEAN); }
void max_values_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_AMAX); }
void min_values_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_AMIN); }

}  // namespace

void launch_reduce(at::TensorIterator& iter, int op) {
  TORCH_CHECK(iter.ntensors() == 2 && iter.noutputs() == 1, "supa: reductions take one input and one output");
  TORCH_CHECK(iter.device_type(0) == c10::DeviceType::PrivateUse1 && iter.device_type(1) == c10::DeviceType::PrivateUse1,
              "supa: reduction operands must be supa tensors");
  TORCH_CHECK(iter.ndim() <= SB_MAX_DIMS, "supa: too many dimensions in a reduction");
  const c10::Device dev = iter.device(0);
  const c10::DeviceGuard guard(dev);
  sb_reduce_desc d{};
  d.op = op;
  d.ndim = iter.ndim();
  d.in_dtype = dtype_code(iter.dtype(1));
  d.out_dtype = dtype_code(iter.dtype(0));
  const int64_t out_es = static_cast<int64_t>(c10::elementSize(iter.dtype(0)));
  const int64_t in_es = static_cast<int64_t>(c10::elementSize(iter.dtype(1)));
  for (int i = 0; i < iter.ndim(); ++i) {
    d.sizes[i] = iter.shape()[i];
    d.out_strides[i] = iter.strides(0)[i] / out_es;
    d.in_strides[i] = iter.strides(1)[i] / in_es;
  }
  if (d.ndim == 0) {
    d.ndim = 1;
    d.sizes[0] = 1;
    d.in_strides[0] = 1;
    d.out_strides[0] = 0;
  }
  d.in = iter.data_ptr(1);
  d.out = iter.data_ptr(0);
  at::Tensor scratch;
  const size_t need = sb_reduce_scratch_bytes(&d);
  if (need) {
    scratch = at::empty({static_cast<int64_t>(need)}, at::TensorOptions().dtype(at::kByte).device(dev));
    d.scratch = scratch.data_ptr();
    d.scratch_bytes = need;
  }
  check_kernel(sb_reduce(&d, static_cast<sb_stream_t>(current_cuda_stream(dev.index()))), "supa reduction kernel");
}

}  // namespace supa

namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(add_stub, &supa::add_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(mul_stub, &supa::mul_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(div_true_stub, &supa::div_true_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(div_trunc_stub, &supa::div_trunc_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(div_floor_stub, &supa::div_floor_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(neg_stub, &supa::neg_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(GeluKernel, &supa::gelu_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(GeluBackwardKernel, &supa::gelu_backward_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(silu_stub, &supa::silu_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(silu_backward_stub, &supa::silu_backward_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(glu_stub, &supa::glu_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(sigmoid_stub, &supa::sigmoid_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(tanh_stub, &supa::tanh_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(exp_stub, &supa::exp_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(log_stub, &supa::log_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(sigmoid_backward_stub, &supa::sigmoid_backward_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(tanh_backward_stub, &supa::tanh_backward_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(maximum_stub, &supa::maximum_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(minimum_stub, &supa::minimum_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(eq_stub, &supa::eq_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(ne_stub, &supa::ne_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(lt_stub, &supa::lt_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(le_stub, &supa::le_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(gt_stub, &supa::gt_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(ge_stub, &supa::ge_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(where_kernel, &supa::where_kernel_supa)
REGISTER_PRIVATEUSE1_DISPATCH(sum_stub, &supa::sum_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(mean_stub, &supa::mean_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(max_values_stub, &supa::max_values_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(min_values_stub, &supa::min_values_kernel)
}  // namespace at::native

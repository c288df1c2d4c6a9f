// PrivateUse1 registrations of the elementwise and reduction operators on the hot path.
//
// In the reference these wrappers are generated: RegisterCUDA_0.cpp is text-rewritten to PrivateUse1
// (script/codegen_native/gen.py:106-191) so that each wrapper instantiates the structured operator class of
// libtorch, runs its meta() (broadcasting, type promotion, output allocation through empty_strided) and its
// impl(), which calls the dispatch stub for the iterator's device.  The same three variants per operator
// (functional, in-place, out=) are written here by hand around small templates.
#include <ATen/native/Activation.h>
#include <ATen/native/ReduceOpsUtils.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/add_native.h>
#include <ATen/ops/amax_native.h>
#include <ATen/ops/amin_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/as_strided_ops.h>
#include <ATen/ops/div_native.h>
#include <ATen/ops/floor_divide_native.h>
#include <ATen/ops/eq_native.h>
#include <ATen/ops/exp_native.h>
#include <ATen/ops/ge_native.h>
#include <ATen/ops/gt_native.h>
#include <ATen/ops/le_native.h>
#include <ATen/ops/log_native.h>
#include <ATen/ops/lt_native.h>
#include <ATen/ops/maximum_native.h>
#include <ATen/ops/minimum_native.h>
#include <ATen/ops/ne_native.h>
#include <ATen/ops/sigmoid_backward_native.h>
#include <ATen/ops/sigmoid_native.h>
#include <ATen/ops/tanh_backward_native.h>
#include <ATen/ops/tanh_native.h>
#include <ATen/ops/where_native.h>
#include <ATen/ops/gelu_backward_meta.h>
#include <ATen/ops/gelu_meta.h>
#include <ATen/ops/glu_native.h>
#include <ATen/ops/mean_meta.h>
#include <ATen/ops/mul_native.h>
#include <ATen/ops/neg_native.h>
#include <ATen/ops/silu_backward_native.h>
#include <ATen/ops/silu_native.h>
#include <ATen/ops/sub_native.h>
#include <ATen/ops/sum_meta.h>
#include <torch/library.h>

#include "Common.h"

namespace supa {

namespace {

at::Tensor create_out(c10::IntArrayRef sizes, c10::IntArrayRef strides, const at::TensorOptions& options) {
  if (strides.empty()) return at::empty(sizes, options);
  return at::empty_strided(sizes, strides, options);
}

void resize_out(const at::Tensor& out, c10::IntArrayRef sizes, c10::IntArrayRef strides, const at::TensorOptions& options) {
  TORCH_CHECK(options.dtype() == out.dtype(), "Expected out tensor to have dtype ", options.dtype(), ", but got ", out.dtype(),
              " instead");
  TORCH_CHECK(options.device() == out.device(), "Expected out tensor to have device ", options.device(), ", but got ", out.device(),
              " instead");
  const bool resized = at::native::resize_output(out, sizes);
  if (resized) {
    if (!strides.empty()) {
      TORCH_INTERNAL_ASSERT(!options.memory_format_opt().has_value());
      out.as_strided_(sizes, strides);
    } else if (options.memory_format_opt().has_value()) {
      out.unsafeGetTensorImpl()->empty_tensor_restride(*options.memory_format_opt());
    }
  }
}

void check_inplace(const at::Tensor& self, c10::IntArrayRef sizes, const at::TensorOptions& options) {
  TORCH_CHECK(options.dtype() == self.dtype(), "Bad in-place call: input tensor dtype ", self.dtype(), " and output tensor dtype ",
              options.dtype(), " should match");
  TORCH_CHECK(options.device() == self.device(), "Bad in-place call: input tensor device ", self.device(),
              " and output tensor device ", options.device(), " should match");
  TORCH_CHECK(sizes == self.sizes(), "Bad in-place call: input tensor size ", self.sizes(), " and output tensor size ", sizes,
              " should match");
}

// TensorIterator-based structured operators record the output in the iterator; plain MetaBase ones
// (reductions) have nothing further to do.
template <class Base>
void forward_to_iterator(Base* self, int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                         at::DimnameList names) {
  if constexpr (std::is_base_of<at::TensorIteratorBase, Base>::value) self->Base::set_output_raw_strided(idx, sizes, strides, options, names);
}

// ---- the three flavours of a structured operator --------------------------------------------------------------
template <class Base, int N = 1>
struct FunctionalOp final : public Base {
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                          at::DimnameList names) override {
    outputs_[idx] = create_out(sizes, strides, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    outputs_[idx] = create_out(sizes, strides, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t idx) override { return outputs_[idx]; }
  std::array<at::Tensor, N> outputs_;
};

template <class Base, int N = 1>
struct OutOp final : public Base {
  explicit OutOp(at::Tensor& out0) : outputs_{std::ref(out0)} {}
  OutOp(at::Tensor& out0, at::Tensor& out1) : outputs_{std::ref(out0), std::ref(out1)} {}
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                          at::DimnameList names) override {
    const at::Tensor& out = outputs_[idx].get();
    resize_out(out, sizes, strides, options);
    // An out= tensor with other strides than the operator wants: compute into a proxy, copy back afterwards
    // (torch_supa/csrc/aten/common/native.h:80-89).
    if (out.strides() != strides) proxies_[idx] = at::empty_strided(sizes, strides, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    resize_out(outputs_[idx].get(), sizes, strides, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t idx) override { return proxies_[idx].has_value() ? *proxies_[idx] : outputs_[idx].get(); }
  void finish() {
    for (int i = 0; i < N; ++i)
      if (proxies_[i].has_value()) outputs_[i].get().copy_(*proxies_[i]);
  }
  std::array<std::reference_wrapper<at::Tensor>, N> outputs_;
  std::array<c10::optional<at::Tensor>, N> proxies_;
};

template <class Base>
struct InplaceOp final : public Base {
  explicit InplaceOp(at::Tensor& self) : self_(self) {}
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                          at::DimnameList names) override {
    check_inplace(self_, sizes, options);
    if (self_.strides() != strides) proxy_ = at::empty_strided(sizes, strides, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    check_inplace(self_, sizes, options);
    forward_to_iterator<Base>(this, idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t) override { return proxy_.has_value() ? *proxy_ : self_; }
  void finish() {
    if (proxy_.has_value()) self_.copy_(*proxy_);
  }
  at::Tensor& self_;
  c10::optional<at::Tensor> proxy_;
};

// Device of the first supa tensor among the arguments (CPU scalars may ride along in binary operators).
c10::Device device_of_args(std::initializer_list<std::reference_wrapper<const at::Tensor>> tensors) {
  for (const at::Tensor& t : tensors)
    if (is_supa(t)) return t.device();
  TORCH_CHECK(false, "supa operator called without a supa tensor");
}

template <class Base, class Meta, class Impl>
at::Tensor run_functional(c10::Device dev, Meta&& meta, Impl&& impl) {
  const c10::DeviceGuard guard(dev);
  FunctionalOp<Base> op;
  meta(op);
  impl(op, op.outputs_[0]);
  return std::move(op.outputs_[0]);
}
template <class Base, class Meta, class Impl>
at::Tensor& run_out(c10::Device dev, at::Tensor& out, Meta&& meta, Impl&& impl) {
  const c10::DeviceGuard guard(dev);
  OutOp<Base> op(out);
  meta(op);
  impl(op, op.maybe_get_output(0));
  op.finish();
  return out;
}
template <class Base, class Meta, class Impl>
at::Tensor& run_inplace(c10::Device dev, at::Tensor& self, Meta&& meta, Impl&& impl) {
  const c10::DeviceGuard guard(dev);
  InplaceOp<Base> op(self);
  meta(op);
  impl(op, op.maybe_get_output(0));
  op.finish();
  return self;
}

// ---- binary operators whose impl() calls a stub with the iterator's device ---------------------------------------
#define SUPA_BINARY_ALPHA(NAME, BASE)                                                                                  \
  at::Tensor NAME##_tensor(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha) {                 \
    return run_functional<BASE>(                                                                                        \
        device_of_args({self, other}), [&](auto& op) { op.meta(self, other, alpha); },                                  \
        [&](auto& op, const at::Tensor& out) { op.impl(self, other, alpha, out); });                                    \
  }                                                                                                                     \
  at::Tensor& NAME##_tensor_(at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha) {                     \
    return run_inplace<BASE>(                                                                                           \
        device_of_args({self, other}), self, [&](auto& op) { op.meta(self, other, alpha); },                            \
        [&](auto& op, const at::Tensor& out) { op.impl(self, other, alpha, out); });                                    \
  }                                                                                                                     \
  at::Tensor& NAME##_out(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha, at::Tensor& out) {  \
    return run_out<BASE>(                                                                                               \
        device_of_args({self, other, out}), out, [&](auto& op) { op.meta(self, other, alpha); },                        \
        [&](auto& op, const at::Tensor& o) { op.impl(self, other, alpha, o); });                                        \
  }

#define SUPA_BINARY(NAME, BASE)                                                                                        \
  at::Tensor NAME##_tensor(const at::Tensor& self, const at::Tensor& other) {                                          \
    return run_functional<BASE>(                                                                                        \
        device_of_args({self, other}), [&](auto& op) { op.meta(self, other); },                                         \
        [&](auto& op, const at::Tensor& out) { op.impl(self, other, out); });                                           \
  }                                                                                                                     \
  at::Tensor& NAME##_tensor_(at::Tensor& self, const at::Tensor& other) {                                              \
    return run_inplace<BASE>(                                                                                           \
        device_of_args({self, other}), self, [&](auto& op) { op.meta(self, other); },                                   \
        [&](auto& op, const at::Tensor& out) { op.impl(self, other, out); });                                           \
  }                                                                                                                     \
  at::Tensor& NAME##_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {                           \
    return run_out<BASE>(                                                                                               \
        device_of_args({self, other, out}), out, [&](auto& op) { op.meta(self, other); },                               \
        [&](auto& op, const at::Tensor& o) { op.impl(self, other, o); });                                               \
  }

#define SUPA_UNARY(NAME, BASE)                                                                                         \
  at::Tensor NAME(const at::Tensor& self) {                                                                             \
    return run_functional<BASE>(                                                                                        \
        self.device(), [&](auto& op) { op.meta(self); }, [&](auto& op, const at::Tensor& out) { op.impl(self, out); }); \
  }                                                                                                                     \
  at::Tensor& NAME##_(at::Tensor& self) {                                                                               \
    return run_inplace<BASE>(                                                                                           \
        self.device(), self, [&](auto& op) { op.meta(self); }, [&](auto& op, const at::Tensor& out) { op.impl(self, out); }); \
  }                                                                                                                     \
  at::Tensor& NAME##_out(const at::Tensor& self, at::Tensor& out) {                                                     \
    return run_out<BASE>(                                                                                               \
        self.device(), out, [&](auto& op) { op.meta(self); }, [&](auto& op, const at::Tensor& o) { op.impl(self, o); }); \
  }

SUPA_BINARY_ALPHA(add, at::native::structured_ufunc_add_CPU)  // impl: add_stub(device_type(), *this, alpha)
SUPA_BINARY_ALPHA(sub, at::native::structured_sub_out)        // impl: add_stub(device_type(), *this, -alpha)
SUPA_BINARY(mul, at::native::structured_mul_out)              // impl: mul_stub(device_type(), *this)
SUPA_BINARY(div, at::native::structured_div_out)              // impl: div_true_stub(device_type(), *this)
// div(self, other, rounding_mode): impl picks div_true_stub / div_trunc_stub / div_floor_stub by the mode
at::Tensor div_mode(const at::Tensor& self, const at::Tensor& other, c10::optional<c10::string_view> mode) {
  return run_functional<at::native::structured_div_out_mode>(
      device_of_args({self, other}), [&](auto& op) { op.meta(self, other, mode); },
      [&](auto& op, const at::Tensor& out) { op.impl(self, other, mode, out); });
}
at::Tensor& div_mode_(at::Tensor& self, const at::Tensor& other, c10::optional<c10::string_view> mode) {
  return run_inplace<at::native::structured_div_out_mode>(
      device_of_args({self, other}), self, [&](auto& op) { op.meta(self, other, mode); },
      [&](auto& op, const at::Tensor& out) { op.impl(self, other, mode, out); });
}
at::Tensor& div_mode_out(const at::Tensor& self, const at::Tensor& other, c10::optional<c10::string_view> mode, at::Tensor& out) {
  return run_out<at::native::structured_div_out_mode>(
      device_of_args({self, other, out}), out, [&](auto& op) { op.meta(self, other, mode); },
      [&](auto& op, const at::Tensor& o) { op.impl(self, other, mode, o); });
}
// floor_divide (the // operator): libtorch's device-generic functions build the iterator and call div_floor_stub
at::Tensor floor_divide(const at::Tensor& self, const at::Tensor& other) {
  const c10::DeviceGuard guard(device_of_args({self, other}));
  return at::native::floor_divide(self, other);
}
at::Tensor& floor_divide_(at::Tensor& self, const at::Tensor& other) {
  const c10::DeviceGuard guard(device_of_args({self, other}));
  return at::native::floor_divide_(self, other);
}
at::Tensor& floor_divide_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  const c10::DeviceGuard guard(device_of_args({self, other, out}));
  return at::native::floor_divide_out(self, other, out);
}
SUPA_UNARY(neg, at::native::structured_neg_out)
SUPA_UNARY(silu, at::native::structured_silu_out)

// ---- neighbouring operators served by the same engine -----------------------------------------------------------
SUPA_UNARY(sigmoid, at::native::structured_sigmoid_out)
SUPA_UNARY(tanh, at::native::structured_tanh_out)
SUPA_UNARY(exp, at::native::structured_exp_out)
SUPA_UNARY(log, at::native::structured_log_out)
SUPA_BINARY(maximum, at::native::structured_maximum_out)
SUPA_BINARY(minimum, at::native::structured_minimum_out)
SUPA_BINARY(sigmoid_backward, at::native::structured_sigmoid_backward_out)  // (grad_output, output)
SUPA_BINARY(tanh_backward, at::native::structured_tanh_backward_out)
SUPA_BINARY(eq, at::native::structured_eq_Tensor_out)
SUPA_BINARY(ne, at::native::structured_ne_Tensor_out)
SUPA_BINARY(lt, at::native::structured_lt_Tensor_out)
SUPA_BINARY(le, at::native::structured_le_Tensor_out)
SUPA_BINARY(gt, at::native::structured_gt_Tensor_out)
SUPA_BINARY(ge, at::native::structured_ge_Tensor_out)

// comparison with a Scalar: the meta step wraps the scalar into a 0-dim CPU tensor, which the stub lifts
#define SUPA_COMPARE_SCALAR(NAME, BASE)                                                                                 \
  at::Tensor NAME##_scalar(const at::Tensor& self, const at::Scalar& other) {                                           \
    return run_functional<BASE>(                                                                                        \
        self.device(), [&](auto& op) { op.meta(self, other); }, [&](auto& op, const at::Tensor& out) { op.impl(self, other, out); }); \
  }                                                                                                                     \
  at::Tensor& NAME##_scalar_(at::Tensor& self, const at::Scalar& other) {                                              \
    return run_inplace<BASE>(                                                                                           \
        self.device(), self, [&](auto& op) { op.meta(self, other); }, [&](auto& op, const at::Tensor& out) { op.impl(self, other, out); }); \
  }                                                                                                                     \
  at::Tensor& NAME##_scalar_out(const at::Tensor& self, const at::Scalar& other, at::Tensor& out) {                    \
    return run_out<BASE>(                                                                                               \
        self.device(), out, [&](auto& op) { op.meta(self, other); }, [&](auto& op, const at::Tensor& o) { op.impl(self, other, o); }); \
  }
SUPA_COMPARE_SCALAR(eq, at::native::structured_eq_Scalar_out)
SUPA_COMPARE_SCALAR(ne, at::native::structured_ne_Scalar_out)
SUPA_COMPARE_SCALAR(lt, at::native::structured_lt_Scalar_out)
SUPA_COMPARE_SCALAR(le, at::native::structured_le_Scalar_out)
SUPA_COMPARE_SCALAR(gt, at::native::structured_gt_Scalar_out)
SUPA_COMPARE_SCALAR(ge, at::native::structured_ge_Scalar_out)

// where: libtorch's own functions promote the values and build the iterator; the kernel comes through where_kernel
at::Tensor where_self(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other) {
  const c10::DeviceGuard guard(condition.device());
  return at::native::where(condition, self, other);
}
at::Tensor& where_self_out(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  const c10::DeviceGuard guard(condition.device());
  return at::native::where_self_out(condition, self, other, out);
}

// masked_fill_(self, mask, value): self[mask] = value; the mask broadcasts against self
at::Tensor& masked_fill_scalar_(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ", mask.scalar_type());
  TORCH_CHECK(is_supa(mask) && mask.device() == self.device(), "masked_fill_: expected self and mask on the same supa device");
  const c10::DeviceGuard guard(self.device());
  auto iter = at::TensorIteratorConfig()
                  .set_check_mem_overlap(false)
                  .check_all_same_dtype(false)
                  .resize_outputs(false)
                  .add_output(self)
                  .add_const_input(self)
                  .add_const_input(mask)
                  .build();
  if (iter.numel() == 0) return self;
  const at::ScalarType dt = self.scalar_type();
  double d = 0.0;
  int64_t i = 0;
  if (c10::isFloatingType(dt)) d = value.to<double>();
  else if (dt == at::kBool) i = value.to<bool>() ? 1 : 0;
  else i = value.to<int64_t>();
  launch_elementwise(iter, SB_EW_MASKED_FILL, dt, 1.0, 1, d, i);
  return self;
}
at::Tensor& masked_fill_tensor_(at::Tensor& self, const at::Tensor& mask, const at::Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "masked_fill_ only supports a 0-dimensional value tensor, but got tensor with ", value.dim(), " dimension(s).");
  return masked_fill_scalar_(self, mask, value.item());
}

// silu_backward(grad_output, self)
at::Tensor silu_backward(const at::Tensor& grad_output, const at::Tensor& self) {
  return run_functional<at::native::structured_silu_backward_out>(
      self.device(), [&](auto& op) { op.meta(grad_output, self); },
      [&](auto& op, const at::Tensor& out) { op.impl(grad_output, self, out); });
}
at::Tensor& silu_backward_out(const at::Tensor& grad_output, const at::Tensor& self, at::Tensor& grad_input) {
  return run_out<at::native::structured_silu_backward_out>(
      self.device(), grad_input, [&](auto& op) { op.meta(grad_output, self); },
      [&](auto& op, const at::Tensor& out) { op.impl(grad_output, self, out); });
}

// gelu: libtorch's impl functions are CPU / CUDA specific, so only the meta step is shared and the kernel
// is launched from the iterator directly.
void gelu_launch(at::TensorIteratorBase& iter, c10::string_view approximate, bool backward) {
  const bool tanh = at::native::get_gelutype_enum(approximate) == at::native::GeluType::Tanh;
  const int op = backward ? (tanh ? SB_EW_GELU_TANH_BWD : SB_EW_GELU_ERF_BWD) : (tanh ? SB_EW_GELU_TANH : SB_EW_GELU_ERF);
  launch_elementwise(iter, op, iter.common_dtype());
}
at::Tensor gelu(const at::Tensor& self, c10::string_view approximate) {
  return run_functional<at::meta::structured_gelu>(
      self.device(), [&](auto& op) { op.meta(self, approximate); },
      [&](auto& op, const at::Tensor&) { gelu_launch(op, approximate, false); });
}
at::Tensor& gelu_(at::Tensor& self, c10::string_view approximate) {
  return run_inplace<at::meta::structured_gelu>(
      self.device(), self, [&](auto& op) { op.meta(self, approximate); },
      [&](auto& op, const at::Tensor&) { gelu_launch(op, approximate, false); });
}
at::Tensor& gelu_out(const at::Tensor& self, c10::string_view approximate, at::Tensor& out) {
  return run_out<at::meta::structured_gelu>(
      self.device(), out, [&](auto& op) { op.meta(self, approximate); },
      [&](auto& op, const at::Tensor&) { gelu_launch(op, approximate, false); });
}
at::Tensor gelu_backward(const at::Tensor& grad_output, const at::Tensor& self, c10::string_view approximate) {
  return run_functional<at::meta::structured_gelu_backward>(
      self.device(), [&](auto& op) { op.meta(grad_output, self, approximate); },
      [&](auto& op, const at::Tensor&) { gelu_launch(op, approximate, true); });
}
at::Tensor& gelu_backward_out(const at::Tensor& grad_output, const at::Tensor& self, c10::string_view approximate,
                              at::Tensor& grad_input) {
  return run_out<at::meta::structured_gelu_backward>(
      self.device(), grad_input, [&](auto& op) { op.meta(grad_output, self, approximate); },
      [&](auto& op, const at::Tensor&) { gelu_launch(op, approximate, true); });
}

// glu(self, dim): meta splits `dim` into two strided halves and builds a binary iterator over them.
at::Tensor glu(const at::Tensor& self, int64_t dim) {
  return run_functional<at::native::structured_glu_out>(
      self.device(), [&](auto& op) { op.meta(self, dim); }, [&](auto& op, const at::Tensor& out) { op.impl(self, dim, out); });
}
at::Tensor& glu_out(const at::Tensor& self, int64_t dim, at::Tensor& out) {
  return run_out<at::native::structured_glu_out>(
      self.device(), out, [&](auto& op) { op.meta(self, dim); }, [&](auto& op, const at::Tensor& o) { op.impl(self, dim, o); });
}

// glu_backward: grad_input[first half] = sigmoid(b) * g, grad_input[second half] = (1 - s) s g a.
at::Tensor& glu_backward_out(const at::Tensor& grad_output, const at::Tensor& self, int64_t dim, at::Tensor& grad_input) {
  TORCH_CHECK(self.dim() > 0, "glu does not support 0-dimensional tensors");
  const int64_t wrap_dim = at::maybe_wrap_dim(dim, self.dim());
  const int64_t n = self.size(wrap_dim);
  TORCH_CHECK(n % 2 == 0, "Halving dimension must be even, but dimension ", wrap_dim, " is size ", n);
  const c10::DeviceGuard guard(self.device());
  at::native::resize_output(grad_input, self.sizes());
  const int64_t half = n / 2;
  const at::Tensor a = self.narrow(wrap_dim, 0, half), b = self.narrow(wrap_dim, half, half);
  at::Tensor ga = grad_input.narrow(wrap_dim, 0, half), gb = grad_input.narrow(wrap_dim, half, half);
  TORCH_CHECK(grad_output.sizes() == a.sizes(), "glu_backward: grad_output has shape ", grad_output.sizes(), ", expected ", a.sizes());
  {
    auto iter = at::TensorIteratorConfig().add_output(ga).add_const_input(grad_output).add_const_input(b).resize_outputs(false).build();
    launch_elementwise(iter, SB_EW_GLU_BWD_A, iter.common_dtype());
  }
  {
    auto iter = at::TensorIteratorConfig()
                    .add_output(gb)
                    .add_const_input(grad_output)
                    .add_const_input(b)
                    .add_const_input(a)
                    .resize_outputs(false)
                    .build();
    launch_elementwise(iter, SB_EW_GLU_BWD_B, iter.common_dtype());
  }
  return grad_input;
}
at::Tensor glu_backward(const at::Tensor& grad_output, const at::Tensor& self, int64_t dim) {
  at::Tensor grad_input = at::empty({0}, self.options());
  return glu_backward_out(grad_output, self, dim, grad_input);
}

// ---- reductions ------------------------------------------------------------------------------------------------
// The reduction kernels convert on load and on store, so the input keeps its own dtype whenever the
// accumulation type that dtype implies is the one the result asks for; otherwise it is cast first, as
// libtorch does (make_reduction_from_out_ty).  bf16/fp16 inputs with an fp32 result stay fused
// (torch_supa/csrc/aten/ops/kernels/reduce/ReduceSumKernel.cu:88-98).
at::ScalarType reduce_input_dtype(at::ScalarType in, at::ScalarType out) {
  const auto f32_family = [](at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16 || t == at::kFloat; };
  if (in == out) return in;
  if (f32_family(in) && f32_family(out)) return in;
  if (in == at::kDouble && c10::isFloatingType(out)) return in;
  if (c10::isIntegralType(in, /*includeBool=*/true) && out == at::kLong) return in;
  return out;
}

void sum_impl(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, const at::Tensor& result, int op) {
  auto iter = at::meta::make_reduction(self, result, dim, keepdim, reduce_input_dtype(self.scalar_type(), result.scalar_type()));
  if (iter.numel() == 0) {
    if (op == SB_RED_MEAN) result.fill_(std::numeric_limits<double>::quiet_NaN());
    else result.zero_();
    return;
  }
  launch_reduce(iter, op);
}

at::Tensor sum_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
  return run_functional<at::meta::structured_sum_dim_IntList>(
      self.device(), [&](auto& op) { op.meta(self, dim, keepdim, dtype); },
      [&](auto&, const at::Tensor& out) { sum_impl(self, dim, keepdim, out, SB_RED_SUM); });
}
at::Tensor& sum_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype,
                    at::Tensor& out) {
  return run_out<at::meta::structured_sum_dim_IntList>(
      self.device(), out, [&](auto& op) { op.meta(self, dim, keepdim, dtype); },
      [&](auto&, const at::Tensor& o) { sum_impl(self, dim, keepdim, o, SB_RED_SUM); });
}
at::Tensor mean_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
  return run_functional<at::meta::structured_mean_dim>(
      self.device(), [&](auto& op) { op.meta(self, dim, keepdim, dtype); },
      [&](auto&, const at::Tensor& out) { sum_impl(self, dim, keepdim, out, SB_RED_MEAN); });
}
at::Tensor& mean_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype,
                     at::Tensor& out) {
  return run_out<at::meta::structured_mean_dim>(
      self.device(), out, [&](auto& op) { op.meta(self, dim, keepdim, dtype); },
      [&](auto&, const at::Tensor& o) { sum_impl(self, dim, keepdim, o, SB_RED_MEAN); });
}

#define SUPA_MINMAX(NAME, BASE)                                                                                         \
  at::Tensor NAME(const at::Tensor& self, at::IntArrayRef dim, bool keepdim) {                                          \
    return run_functional<BASE>(                                                                                        \
        self.device(), [&](auto& op) { op.meta(self, dim, keepdim); },                                                  \
        [&](auto& op, const at::Tensor& out) { op.impl(self, dim, keepdim, out); });                                    \
  }                                                                                                                     \
  at::Tensor& NAME##_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, at::Tensor& out) {                  \
    return run_out<BASE>(                                                                                               \
        self.device(), out, [&](auto& op) { op.meta(self, dim, keepdim); },                                             \
        [&](auto& op, const at::Tensor& o) { op.impl(self, dim, keepdim, o); });                                        \
  }
SUPA_MINMAX(amax, at::native::structured_amax_out)  // impl: max_values_stub(iter.device_type(), iter)
SUPA_MINMAX(amin, at::native::structured_amin_out)

}  // namespace
}  // namespace supa

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("add.Tensor", TORCH_FN(supa::add_tensor));
  m.impl("add_.Tensor", TORCH_FN(supa::add_tensor_));
  m.impl("add.out", TORCH_FN(supa::add_out));
  m.impl("sub.Tensor", TORCH_FN(supa::sub_tensor));
  m.impl("sub_.Tensor", TORCH_FN(supa::sub_tensor_));
  m.impl("sub.out", TORCH_FN(supa::sub_out));
  m.impl("mul.Tensor", TORCH_FN(supa::mul_tensor));
  m.impl("mul_.Tensor", TORCH_FN(supa::mul_tensor_));
  m.impl("mul.out", TORCH_FN(supa::mul_out));
  m.impl("div.Tensor", TORCH_FN(supa::div_tensor));
  m.impl("div_.Tensor", TORCH_FN(supa::div_tensor_));
  m.impl("div.out", TORCH_FN(supa::div_out));
  m.impl("div.Tensor_mode", TORCH_FN(supa::div_mode));
  m.impl("div_.Tensor_mode", TORCH_FN(supa::div_mode_));
  m.impl("div.out_mode", TORCH_FN(supa::div_mode_out));
  m.impl("floor_divide", TORCH_FN(supa::floor_divide));
  m.impl("floor_divide_.Tensor", TORCH_FN(supa::floor_divide_));
  m.impl("floor_divide.out", TORCH_FN(supa::floor_divide_out));
  m.impl("neg", TORCH_FN(supa::neg));
  m.impl("neg_", TORCH_FN(supa::neg_));
  m.impl("neg.out", TORCH_FN(supa::neg_out));
#define SUPA_REG_UNARY(NAME) \
  m.impl(#NAME, TORCH_FN(supa::NAME)); m.impl(#NAME "_", TORCH_FN(supa::NAME##_)); m.impl(#NAME ".out", TORCH_FN(supa::NAME##_out));
  SUPA_REG_UNARY(sigmoid) SUPA_REG_UNARY(tanh) SUPA_REG_UNARY(exp) SUPA_REG_UNARY(log)
#undef SUPA_REG_UNARY
  m.impl("maximum", TORCH_FN(supa::maximum_tensor));
  m.impl("maximum.out", TORCH_FN(supa::maximum_out));
  m.impl("minimum", TORCH_FN(supa::minimum_tensor));
  m.impl("minimum.out", TORCH_FN(supa::minimum_out));
  m.impl("sigmoid_backward", TORCH_FN(supa::sigmoid_backward_tensor));
  m.impl("sigmoid_backward.grad_input", TORCH_FN(supa::sigmoid_backward_out));
  m.impl("tanh_backward", TORCH_FN(supa::tanh_backward_tensor));
  m.impl("tanh_backward.grad_input", TORCH_FN(supa::tanh_backward_out));
#define SUPA_REG_COMPARE(NAME)                                        \
  m.impl(#NAME ".Tensor", TORCH_FN(supa::NAME##_tensor));             \
  m.impl(#NAME "_.Tensor", TORCH_FN(supa::NAME##_tensor_));           \
  m.impl(#NAME ".Tensor_out", TORCH_FN(supa::NAME##_out));            \
  m.impl(#NAME ".Scalar", TORCH_FN(supa::NAME##_scalar));             \
  m.impl(#NAME "_.Scalar", TORCH_FN(supa::NAME##_scalar_));           \
  m.impl(#NAME ".Scalar_out", TORCH_FN(supa::NAME##_scalar_out));
  SUPA_REG_COMPARE(eq) SUPA_REG_COMPARE(ne) SUPA_REG_COMPARE(lt) SUPA_REG_COMPARE(le) SUPA_REG_COMPARE(gt) SUPA_REG_COMPARE(ge)
#undef SUPA_REG_COMPARE
  m.impl("where.self", TORCH_FN(supa::where_self));
  m.impl("where.self_out", TORCH_FN(supa::where_self_out));
  m.impl("masked_fill_.Scalar", TORCH_FN(supa::masked_fill_scalar_));
  m.impl("masked_fill_.Tensor", TORCH_FN(supa::masked_fill_tensor_));
  m.impl("silu", TORCH_FN(supa::silu));
  m.impl("silu_", TORCH_FN(supa::silu_));
  m.impl("silu.out", TORCH_FN(supa::silu_out));
  m.impl("silu_backward", TORCH_FN(supa::silu_backward));
  m.impl("silu_backward.grad_input", TORCH_FN(supa::silu_backward_out));
  m.impl("gelu", TORCH_FN(supa::gelu));
  m.impl("gelu_", TORCH_FN(supa::gelu_));
  m.impl("gelu.out", TORCH_FN(supa::gelu_out));
  m.impl("gelu_backward", TORCH_FN(supa::gelu_backward));
  m.impl("gelu_backward.grad_input", TORCH_FN(supa::gelu_backward_out));
  m.impl("glu", TORCH_FN(supa::glu));
  m.impl("glu.out", TORCH_FN(supa::glu_out));
  m.impl("glu_backward", TORCH_FN(supa::glu_backward));
  m.impl("glu_backward.grad_input", TORCH_FN(supa::glu_backward_out));
  m.impl("sum.dim_IntList", TORCH_FN(supa::sum_dim));
  m.impl("sum.IntList_out", TORCH_FN(supa::sum_out));
  m.impl("mean.dim", TORCH_FN(supa::mean_dim));
  m.impl("mean.out", TORCH_FN(supa::mean_out));
  m.impl("amax", TORCH_FN(supa::amax));
  m.impl("amax.out", TORCH_FN(supa::amax_out));
  m.impl("amin", TORCH_FN(supa::amin));
  m.impl("amin.out", TORCH_FN(supa::amin_out));
}

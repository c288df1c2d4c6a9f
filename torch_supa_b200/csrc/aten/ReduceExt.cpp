// Reductions beside sum / mean / amax on the supa device: argmax / argmin, max.dim / min.dim (values and indices),
// max / min of a whole tensor, var / std (+ var_mean, std_mean), prod, nansum.
//
// In the reference these come from the same reduce family as sum (torch_supa/csrc/aten/ops/kernels/reduce/Reduce.cuh,
// torch_supa/csrc/aten/ops/StdVar.cpp:34-63) behind generated wrappers; here the index and moment reductions run the
// kernels of reduce_ext.cu on a contiguous [outer, L, inner] view, and prod / nansum ride on the sum engine through
// their dispatch stubs.
#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/ReduceOps.h>
#include <ATen/native/ReduceOpsUtils.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/argmax_meta.h>
#include <ATen/ops/argmin_meta.h>
#include <ATen/ops/max_meta.h>
#include <ATen/ops/min_meta.h>
#include <ATen/ops/nansum_native.h>
#include <ATen/ops/prod_meta.h>
#include <torch/library.h>

#include "Common.h"

namespace supa {

namespace {

// [outer, L, inner] of a contiguous tensor reduced over `dim`.
void split_at(const at::Tensor& t, int64_t dim, int64_t& outer, int64_t& L, int64_t& inner) {
  outer = inner = 1;
  L = t.dim() == 0 ? 1 : t.size(dim);
  for (int64_t i = 0; i < dim; ++i) outer *= t.size(i);
  for (int64_t i = dim + 1; i < t.dim(); ++i) inner *= t.size(i);
}

at::Tensor ext_scratch(const at::Tensor& like, int64_t outer, int64_t L, int64_t inner, bool moments) {
  const size_t need = sb_reduce_ext_scratch_bytes(dtype_code(like.scalar_type()), outer, L, inner, moments ? 1 : 0);
  if (!need) return at::Tensor();
  return at::empty({static_cast<int64_t>(need)}, like.options().dtype(at::kByte));
}

// values (may be undefined) and indices (may be undefined) of the extremum along `dim` (nullopt: the flattened tensor).
// Both outputs are contiguous tensors with outer * inner elements.
void arg_reduce(const at::Tensor& self, c10::optional<int64_t> dim, bool is_max, const at::Tensor& values, const at::Tensor& indices,
                const char* name) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor x = self.contiguous();
  int64_t outer = 1, L = x.numel(), inner = 1;
  if (dim.has_value() && x.dim() > 0) split_at(x, at::maybe_wrap_dim(*dim, x.dim()), outer, L, inner);
  if (outer * inner == 0) return;
  TORCH_CHECK_INDEX(L > 0, name, "(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");
  at::Tensor scratch = ext_scratch(x, outer, L, inner, false);
  check_kernel(sb_arg_reduce(x.const_data_ptr(), dtype_code(x.scalar_type()), outer, L, inner, is_max ? 1 : 0,
                             values.defined() ? values.data_ptr() : nullptr, indices.defined() ? indices.data_ptr<int64_t>() : nullptr,
                             scratch.defined() ? scratch.data_ptr() : nullptr, scratch.defined() ? static_cast<size_t>(scratch.numel()) : 0,
                             stream_of(x)),
               name);
}

// An output the kernel can write directly (contiguous), or a contiguous stand-in that is copied back afterwards.
struct OutProxy {
  explicit OutProxy(const at::Tensor& out) : out_(out), work_(out.is_contiguous() ? out : at::empty(out.sizes(), out.options())) {}
  const at::Tensor& get() const { return work_; }
  void finish() const {
    if (!work_.is_same(out_)) out_.copy_(work_);
  }
  const at::Tensor& out_;
  at::Tensor work_;
};

template <class Meta>
struct Functional2 final : public Meta {
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options, at::DimnameList) override {
    outputs_[idx] = strides.empty() ? at::empty(sizes, options) : at::empty_strided(sizes, strides, options);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    set_output_strided(idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t idx) override { return outputs_[idx]; }
  std::array<at::Tensor, 2> outputs_;
};
template <class Meta>
struct Out2 final : public Meta {
  Out2(at::Tensor& a, at::Tensor& b) : outputs_{&a, &b} {}
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef, at::TensorOptions options, at::DimnameList) override {
    at::Tensor& out = *outputs_[idx];
    TORCH_CHECK(options.dtype() == out.dtype(), "Expected out tensor to have dtype ", options.dtype(), ", but got ", out.dtype(), " instead");
    TORCH_CHECK(options.device() == out.device(), "Expected out tensor to have device ", options.device(), ", but got ", out.device(),
                " instead");
    at::native::resize_output(out, sizes);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    set_output_strided(idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t idx) override { return *outputs_[idx]; }
  std::array<at::Tensor*, 2> outputs_;
};

// ---- argmax / argmin ----------------------------------------------------------------------------------------------
template <class Meta, bool IS_MAX>
at::Tensor arg_functional(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim) {
  const c10::DeviceGuard guard(self.device());
  Functional2<Meta> op;
  op.meta(self, dim, keepdim);
  const OutProxy idx(op.outputs_[0]);
  arg_reduce(self, dim, IS_MAX, at::Tensor(), idx.get(), IS_MAX ? "argmax" : "argmin");
  idx.finish();
  return std::move(op.outputs_[0]);
}
template <class Meta, bool IS_MAX>
at::Tensor& arg_out(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim, at::Tensor& out) {
  const c10::DeviceGuard guard(self.device());
  Out2<Meta> op(out, out);
  op.meta(self, dim, keepdim);
  const OutProxy idx(out);
  arg_reduce(self, dim, IS_MAX, at::Tensor(), idx.get(), IS_MAX ? "argmax" : "argmin");
  idx.finish();
  return out;
}

// ---- max.dim / min.dim ---------------------------------------------------------------------------------------------
template <class Meta, bool IS_MAX>
std::tuple<at::Tensor, at::Tensor> minmax_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
  const c10::DeviceGuard guard(self.device());
  Functional2<Meta> op;
  op.meta(self, dim, keepdim);
  const OutProxy values(op.outputs_[0]), indices(op.outputs_[1]);
  arg_reduce(self, dim, IS_MAX, values.get(), indices.get(), IS_MAX ? "max" : "min");
  values.finish();
  indices.finish();
  return std::make_tuple(std::move(op.outputs_[0]), std::move(op.outputs_[1]));
}
template <class Meta, bool IS_MAX>
std::tuple<at::Tensor&, at::Tensor&> minmax_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& values_out,
                                                     at::Tensor& indices_out) {
  const c10::DeviceGuard guard(self.device());
  Out2<Meta> op(values_out, indices_out);
  op.meta(self, dim, keepdim);
  const OutProxy values(values_out), indices(indices_out);
  arg_reduce(self, dim, IS_MAX, values.get(), indices.get(), IS_MAX ? "max" : "min");
  values.finish();
  indices.finish();
  return std::forward_as_tuple(values_out, indices_out);
}

// max / min of all elements (NaN propagates), through the extremum kernel without indices.
template <bool IS_MAX>
at::Tensor minmax_all(const at::Tensor& self) {
  TORCH_CHECK(self.numel() > 0, IS_MAX ? "max" : "min", "(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");
  const c10::DeviceGuard guard(self.device());
  at::Tensor out = at::empty({}, self.options());
  arg_reduce(self, c10::nullopt, IS_MAX, out, at::Tensor(), IS_MAX ? "max" : "min");
  return out;
}

// ---- var / std --------------------------------------------------------------------------------------------------
// Reduced dimensions are moved behind the kept ones and the tensor made contiguous: [outer, L]; a single reduced
// dimension of a contiguous tensor is used where it lies, as [outer, L, inner].
void moments_impl(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim, bool take_sqrt,
                  at::Tensor& out, at::Tensor* mean_out, const char* name) {
  TORCH_CHECK(at::isFloatingType(self.scalar_type()), name, " only support floating point dtypes on the supa device, got ", self.scalar_type());
  TORCH_CHECK(out.scalar_type() == self.scalar_type(), name, ": expected an out tensor of dtype ", self.scalar_type());
  const c10::DeviceGuard guard(self.device());
  const int64_t nd = self.dim();
  const auto mask = at::native::make_dim_mask(dim, nd);
  const auto shape = at::meta::get_reduction_shape(self, dim.has_value() ? dim.value() : at::IntArrayRef{}, keepdim);
  at::native::resize_output(out, shape);
  if (mean_out) at::native::resize_output(*mean_out, shape);
  const double corr = correction.has_value() ? correction->toDouble() : 1.0;
  int64_t nred = 0, last_red = -1;
  for (int64_t i = 0; i < nd; ++i)
    if (mask[i]) {
      ++nred;
      last_red = i;
    }
  at::Tensor x;
  int64_t outer = 1, L = 1, inner = 1;
  if (nd == 0) {
    x = self.contiguous();
  } else if (nred == 1 && self.is_contiguous()) {
    x = self;
    split_at(x, last_red, outer, L, inner);
  } else {
    std::vector<int64_t> perm;
    for (int64_t i = 0; i < nd; ++i)
      if (!mask[i]) perm.push_back(i);
    for (int64_t i = 0; i < nd; ++i)
      if (mask[i]) perm.push_back(i);
    x = self.permute(perm).contiguous();
    for (int64_t i = 0; i < nd; ++i) (mask[i] ? L : outer) *= self.size(i);
  }
  if (outer * inner == 0) return;
  if (L == 0) {
    out.fill_(std::numeric_limits<double>::quiet_NaN());
    if (mean_out) mean_out->fill_(std::numeric_limits<double>::quiet_NaN());
    return;
  }
  const OutProxy o(out);
  c10::optional<OutProxy> m;
  if (mean_out) m.emplace(*mean_out);
  at::Tensor scratch = ext_scratch(x, outer, L, inner, true);
  check_kernel(sb_moments(x.const_data_ptr(), dtype_code(x.scalar_type()), outer, L, inner, corr, take_sqrt ? 1 : 0, o.get().data_ptr(),
                          m.has_value() ? m->get().data_ptr() : nullptr, scratch.defined() ? scratch.data_ptr() : nullptr,
                          scratch.defined() ? static_cast<size_t>(scratch.numel()) : 0, stream_of(x)),
               name);
  o.finish();
  if (m.has_value()) m->finish();
}

at::Tensor var_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
  at::Tensor out = at::empty({0}, self.options());
  moments_impl(self, dim, correction, keepdim, false, out, nullptr, "var");
  return out;
}
at::Tensor& var_correction_out(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim,
                               at::Tensor& out) {
  moments_impl(self, dim, correction, keepdim, false, out, nullptr, "var");
  return out;
}
at::Tensor std_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
  at::Tensor out = at::empty({0}, self.options());
  moments_impl(self, dim, correction, keepdim, true, out, nullptr, "std");
  return out;
}
at::Tensor& std_correction_out(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim,
                               at::Tensor& out) {
  moments_impl(self, dim, correction, keepdim, true, out, nullptr, "std");
  return out;
}
std::tuple<at::Tensor, at::Tensor> var_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim,
                                                       const c10::optional<at::Scalar>& correction, bool keepdim) {
  at::Tensor out = at::empty({0}, self.options()), mean = at::empty({0}, self.options());
  moments_impl(self, dim, correction, keepdim, false, out, &mean, "var_mean");
  return std::make_tuple(std::move(out), std::move(mean));
}
std::tuple<at::Tensor, at::Tensor> std_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim,
                                                       const c10::optional<at::Scalar>& correction, bool keepdim) {
  at::Tensor out = at::empty({0}, self.options()), mean = at::empty({0}, self.options());
  moments_impl(self, dim, correction, keepdim, true, out, &mean, "std_mean");
  return std::make_tuple(std::move(out), std::move(mean));
}

// ---- prod / nansum: the sum engine with another functor ------------------------------------------------------------
void prod_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_PROD); }
void nansum_kernel(at::TensorIterator& iter) { launch_reduce(iter, SB_RED_NANSUM); }

at::ScalarType prod_in_dtype(at::ScalarType in, at::ScalarType out) {
  const auto f32_family = [](at::ScalarType t) { return t == at::kHalf || t == at::kBFloat16 || t == at::kFloat; };
  if (in == out || (f32_family(in) && f32_family(out))) return in;
  if (c10::isIntegralType(in, true) && out == at::kLong) return in;
  return out;
}
void prod_impl(const at::Tensor& self, at::OptionalIntArrayRef dims, bool keepdim, const at::Tensor& result) {
  auto iter = at::meta::make_reduction(self, result, dims, keepdim, prod_in_dtype(self.scalar_type(), result.scalar_type()));
  if (iter.numel() == 0) {
    result.fill_(1);
    return;
  }
  launch_reduce(iter, SB_RED_PROD);
}
at::Tensor prod_dim(const at::Tensor& self, int64_t dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
  const c10::DeviceGuard guard(self.device());
  Functional2<at::meta::structured_prod_dim_int> op;
  op.meta(self, dim, keepdim, dtype);
  prod_impl(self, at::IntArrayRef(dim), keepdim, op.outputs_[0]);
  return std::move(op.outputs_[0]);
}
at::Tensor& prod_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
  const c10::DeviceGuard guard(self.device());
  Out2<at::meta::structured_prod_dim_int> op(out, out);
  op.meta(self, dim, keepdim, dtype);
  prod_impl(self, at::IntArrayRef(dim), keepdim, out);
  return out;
}
at::Tensor prod_all(const at::Tensor& self, c10::optional<at::ScalarType> dtype) {
  const c10::DeviceGuard guard(self.device());
  at::ScalarType out_dtype = dtype.has_value() ? *dtype : (c10::isIntegralType(self.scalar_type(), true) ? at::kLong : self.scalar_type());
  at::Tensor out = at::empty({}, self.options().dtype(out_dtype));
  prod_impl(self, at::OptionalIntArrayRef(at::IntArrayRef{}), false, out);
  return out;
}
at::Tensor nansum(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
  const c10::DeviceGuard guard(self.device());
  return at::native::nansum(self, dim, keepdim, dtype);  // device-generic: builds the iterator, then nansum_stub
}
at::Tensor& nansum_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
  const c10::DeviceGuard guard(self.device());
  return at::native::nansum_out(self, dim, keepdim, dtype, out);
}

}  // namespace
}  // namespace supa

namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(prod_stub, &supa::prod_kernel)
REGISTER_PRIVATEUSE1_DISPATCH(nansum_stub, &supa::nansum_kernel)
}  // namespace at::native

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("argmax", TORCH_FN((supa::arg_functional<at::meta::structured_argmax, true>)));
  m.impl("argmax.out", TORCH_FN((supa::arg_out<at::meta::structured_argmax, true>)));
  m.impl("argmin", TORCH_FN((supa::arg_functional<at::meta::structured_argmin, false>)));
  m.impl("argmin.out", TORCH_FN((supa::arg_out<at::meta::structured_argmin, false>)));
  m.impl("max.dim", TORCH_FN((supa::minmax_dim<at::meta::structured_max_dim, true>)));
  m.impl("max.dim_max", TORCH_FN((supa::minmax_dim_out<at::meta::structured_max_dim, true>)));
  m.impl("min.dim", TORCH_FN((supa::minmax_dim<at::meta::structured_min_dim, false>)));
  m.impl("min.dim_min", TORCH_FN((supa::minmax_dim_out<at::meta::structured_min_dim, false>)));
  m.impl("max", TORCH_FN(supa::minmax_all<true>));
  m.impl("min", TORCH_FN(supa::minmax_all<false>));
  m.impl("var.correction", TORCH_FN(supa::var_correction));
  m.impl("var.correction_out", TORCH_FN(supa::var_correction_out));
  m.impl("std.correction", TORCH_FN(supa::std_correction));
  m.impl("std.correction_out", TORCH_FN(supa::std_correction_out));
  m.impl("var_mean.correction", TORCH_FN(supa::var_mean_correction));
  m.impl("std_mean.correction", TORCH_FN(supa::std_mean_correction));
  m.impl("prod", TORCH_FN(supa::prod_all));
  m.impl("prod.dim_int", TORCH_FN(supa::prod_dim));
  m.impl("prod.int_out", TORCH_FN(supa::prod_dim_out));
  m.impl("nansum", TORCH_FN(supa::nansum));
  m.impl("nansum.out", TORCH_FN(supa::nansum_out));
}

// log_softmax, nll_loss and cross_entropy_loss on the supa device.
//
// cross_entropy_loss is registered as a backend kernel, as the reference does
// (torch_supa/csrc/aten/supa_native_functions.yaml:59-61, torch_supa/csrc/aten/ops/CrossEntropyLoss.cpp:140-151): with a
// backend kernel present the operator no longer decomposes under autograd, so the kernel builds the graph
// itself with a torch::autograd::Function and the AutogradPrivateUse1 key falls through
// (torch_supa/csrc/aten/VariableFallbackKernel.cpp:31-33).  Unlike the reference's node, which keeps an
// [N, C] log-probability buffer and runs nll_loss_backward + _log_softmax_backward_data in backward
// (CrossEntropyLoss.cpp:76-83, 94-135), the forward sweep here already writes the logit gradient, scaled for
// an upstream gradient of one; backward only rescales it when the upstream gradient is something else.
#include <ATen/native/Resize.h>
#include <ATen/ops/_log_softmax_backward_data_meta.h>
#include <ATen/ops/_log_softmax_meta.h>
#include <ATen/ops/cross_entropy_loss_native.h>
#include <ATen/ops/nll_loss_backward_meta.h>
#include <ATen/ops/nll_loss_forward_meta.h>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/library.h>

#include "Common.h"
#include "dist/NcclComm.h"

namespace supa {

namespace {

int reduction_code(int64_t reduction) {
  switch (reduction) {
    case at::Reduction::None: return SB_REDUCTION_NONE;
    case at::Reduction::Mean: return SB_REDUCTION_MEAN;
    case at::Reduction::Sum: return SB_REDUCTION_SUM;
    default: TORCH_CHECK(false, "Invalid reduction type encountered in loss: ", reduction);
  }
}

// ---- log_softmax -----------------------------------------------------------------------------------------------
void split_dims(const at::Tensor& t, int64_t dim, int64_t& outer, int64_t& size, int64_t& inner) {
  outer = 1;
  inner = 1;
  if (t.dim() == 0) {
    size = 1;
    return;
  }
  size = t.size(dim);
  for (int64_t i = 0; i < dim; ++i) outer *= t.size(i);
  for (int64_t i = dim + 1; i < t.dim(); ++i) inner *= t.size(i);
}

void log_softmax_impl(const at::Tensor& self, int64_t dim, bool half_to_float, const at::Tensor& out, bool log = true) {
  if (half_to_float)
    TORCH_CHECK(self.scalar_type() == at::kHalf || self.scalar_type() == at::kBFloat16,
                "conversion is supported for Half and BFloat16 type only");
  if (self.numel() == 0) return;
  const int64_t wdim = at::maybe_wrap_dim(dim, self.dim());
  const at::Tensor input = self.contiguous();
  at::Tensor result = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  int64_t outer, size, inner;
  split_dims(input, wdim, outer, size, inner);
  check_kernel((log ? sb_log_softmax_forward : sb_softmax_forward)(input.const_data_ptr(), dtype_code(input.scalar_type()),
                                                                  result.data_ptr(), dtype_code(result.scalar_type()), outer, size,
                                                                  inner, stream_of(input)),
               log ? "supa log_softmax" : "supa softmax");
  if (!result.is_same(out)) out.copy_(result);
}

void log_softmax_backward_impl(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype,
                               const at::Tensor& grad_input, bool log = true) {
  if (output.numel() == 0) return;
  const int64_t wdim = at::maybe_wrap_dim(dim, output.dim());
  at::Tensor go = grad_output.contiguous();
  if (go.scalar_type() != output.scalar_type()) go = go.to(output.scalar_type());
  const at::Tensor y = output.contiguous();
  at::Tensor result = grad_input.is_contiguous() ? grad_input : at::empty(grad_input.sizes(), grad_input.options());
  int64_t outer, size, inner;
  split_dims(y, wdim, outer, size, inner);
  check_kernel((log ? sb_log_softmax_backward : sb_softmax_backward)(go.const_data_ptr(), y.const_data_ptr(), dtype_code(y.scalar_type()),
                                                                    result.data_ptr(), dtype_code(result.scalar_type()), outer, size,
                                                                    inner, stream_of(y)),
               log ? "supa log_softmax backward" : "supa softmax backward");
  if (!result.is_same(grad_input)) grad_input.copy_(result);
}

// Minimal functional / out= shells around the libtorch meta classes (shape, dtype and argument checks).
template <class Meta>
struct FunctionalMeta final : public Meta {
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                          at::DimnameList) override {
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
struct OutMeta final : public Meta {
  OutMeta(at::Tensor& a, at::Tensor& b) : outputs_{&a, &b} {}
  void set_output_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef, at::TensorOptions options, at::DimnameList) override {
    at::Tensor& out = *outputs_[idx];
    TORCH_CHECK(options.dtype() == out.dtype(), "Expected out tensor to have dtype ", options.dtype(), ", but got ", out.dtype(),
                " instead");
    TORCH_CHECK(options.device() == out.device(), "Expected out tensor to have device ", options.device(), ", but got ",
                out.device(), " instead");
    at::native::resize_output(out, sizes);
  }
  void set_output_raw_strided(int64_t idx, c10::IntArrayRef sizes, c10::IntArrayRef strides, at::TensorOptions options,
                              at::DimnameList names) override {
    set_output_strided(idx, sizes, strides, options, names);
  }
  const at::Tensor& maybe_get_output(int64_t idx) override { return *outputs_[idx]; }
  std::array<at::Tensor*, 2> outputs_;
};

at::Tensor log_softmax(const at::Tensor& self, int64_t dim, bool half_to_float) {
  const c10::DeviceGuard guard(self.device());
  FunctionalMeta<at::meta::structured__log_softmax> op;
  op.meta(self, dim, half_to_float);
  log_softmax_impl(self, dim, half_to_float, op.outputs_[0]);
  return std::move(op.outputs_[0]);
}
at::Tensor& log_softmax_out(const at::Tensor& self, int64_t dim, bool half_to_float, at::Tensor& out) {
  const c10::DeviceGuard guard(self.device());
  OutMeta<at::meta::structured__log_softmax> op(out, out);
  op.meta(self, dim, half_to_float);
  log_softmax_impl(self, dim, half_to_float, out);
  return out;
}
at::Tensor log_softmax_backward(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype) {
  const c10::DeviceGuard guard(output.device());
  FunctionalMeta<at::meta::structured__log_softmax_backward_data> op;
  op.meta(grad_output, output, dim, input_dtype);
  log_softmax_backward_impl(grad_output, output, dim, input_dtype, op.outputs_[0]);
  return std::move(op.outputs_[0]);
}
at::Tensor& log_softmax_backward_out(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim,
                                     at::ScalarType input_dtype, at::Tensor& out) {
  const c10::DeviceGuard guard(output.device());
  OutMeta<at::meta::structured__log_softmax_backward_data> op(out, out);
  op.meta(grad_output, output, dim, input_dtype);
  log_softmax_backward_impl(grad_output, output, dim, input_dtype, out);
  return out;
}

// ---- softmax: the same shells around the non-log kernels ---------------------------------------------------------
at::Tensor softmax(const at::Tensor& self, int64_t dim, bool half_to_float) {
  const c10::DeviceGuard guard(self.device());
  FunctionalMeta<at::meta::structured__softmax> op;
  op.meta(self, dim, half_to_float);
  log_softmax_impl(self, dim, half_to_float, op.outputs_[0], /*log=*/false);
  return std::move(op.outputs_[0]);
}
at::Tensor& softmax_out(const at::Tensor& self, int64_t dim, bool half_to_float, at::Tensor& out) {
  const c10::DeviceGuard guard(self.device());
  OutMeta<at::meta::structured__softmax> op(out, out);
  op.meta(self, dim, half_to_float);
  log_softmax_impl(self, dim, half_to_float, out, /*log=*/false);
  return out;
}
at::Tensor softmax_backward(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype) {
  const c10::DeviceGuard guard(output.device());
  FunctionalMeta<at::meta::structured__softmax_backward_data> op;
  op.meta(grad_output, output, dim, input_dtype);
  log_softmax_backward_impl(grad_output, output, dim, input_dtype, op.outputs_[0], /*log=*/false);
  return std::move(op.outputs_[0]);
}
at::Tensor& softmax_backward_out(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype,
                                 at::Tensor& out) {
  const c10::DeviceGuard guard(output.device());
  OutMeta<at::meta::structured__softmax_backward_data> op(out, out);
  op.meta(grad_output, output, dim, input_dtype);
  log_softmax_backward_impl(grad_output, output, dim, input_dtype, out, /*log=*/false);
  return out;
}

// ---- nll_loss --------------------------------------------------------------------------------------------------
sb_nll_args nll_args(const at::Tensor& self, const at::Tensor& target, const at::Tensor& weight, int64_t reduction,
                     int64_t ignore_index) {
  sb_nll_args a{};
  a.log_probs = self.const_data_ptr();
  a.dtype = dtype_code(self.scalar_type());
  TORCH_CHECK(target.scalar_type() == at::kLong || target.scalar_type() == at::kByte,
              "expected scalar type Long or Byte for target but found ", target.scalar_type());
  a.target_dtype = dtype_code(target.scalar_type());
  a.target = target.const_data_ptr();
  a.weight = weight.defined() ? weight.const_data_ptr() : nullptr;
  a.rows = self.dim() == 1 ? 1 : self.size(0);
  a.classes = self.size(-1);
  a.ignore_index = ignore_index;
  a.reduction = reduction_code(reduction);
  a.status = status_word(self.device().index());
  return a;
}

void nll_forward_impl(const at::Tensor& self, const at::Tensor& target, at::OptionalTensorRef weight_opt, int64_t reduction,
                      int64_t ignore_index, const at::Tensor& output, const at::Tensor& total_weight) {
  const at::Tensor input = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  at::Tensor weight;
  if (weight_opt.has_value() && weight_opt->defined()) weight = weight_opt->contiguous().to(input.scalar_type());
  const int red = reduction_code(reduction);
  if (red == SB_REDUCTION_NONE && input.dim() == 2) {
    if (input.size(0) == 0) {
      total_weight.zero_();
      return;
    }
  }
  TORCH_CHECK(output.is_contiguous() && total_weight.is_contiguous(), "nll_loss: outputs must be contiguous");
  const sb_nll_args a = nll_args(input, tgt, weight, reduction, ignore_index);
  // `none` never writes total_weight in the kernel; libtorch leaves it zero in that case
  if (red == SB_REDUCTION_NONE) total_weight.zero_();
  check_kernel(sb_nll_loss_forward(&a, output.data_ptr(), total_weight.data_ptr(), stream_of(input)), "supa nll_loss_forward");
}

void nll_backward_impl(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                       at::OptionalTensorRef weight_opt, int64_t reduction, int64_t ignore_index, const at::Tensor& total_weight,
                       const at::Tensor& grad_input) {
  if (self.numel() == 0) return;
  const at::Tensor input = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  at::Tensor weight;
  if (weight_opt.has_value() && weight_opt->defined()) weight = weight_opt->contiguous().to(input.scalar_type());
  at::Tensor go = grad_output.contiguous();
  if (go.scalar_type() != input.scalar_type()) go = go.to(input.scalar_type());
  at::Tensor tw = total_weight.scalar_type() == input.scalar_type() ? total_weight : total_weight.to(input.scalar_type());
  at::Tensor result = grad_input.is_contiguous() ? grad_input : at::empty(grad_input.sizes(), grad_input.options());
  const sb_nll_args a = nll_args(input, tgt, weight, reduction, ignore_index);
  check_kernel(sb_nll_loss_backward(&a, go.const_data_ptr(), tw.const_data_ptr(), result.data_ptr(), stream_of(input)),
               "supa nll_loss_backward");
  if (!result.is_same(grad_input)) grad_input.copy_(result);
}

at::OptionalTensorRef weight_ref(const c10::optional<at::Tensor>& weight) {
  return (weight.has_value() && weight->defined()) ? at::OptionalTensorRef(*weight) : at::OptionalTensorRef();
}

std::tuple<at::Tensor, at::Tensor> nll_loss_forward(const at::Tensor& self, const at::Tensor& target,
                                                    const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index) {
  const c10::DeviceGuard guard(self.device());
  FunctionalMeta<at::meta::structured_nll_loss_forward> op;
  op.meta(self, target, weight_ref(weight), reduction, ignore_index);
  nll_forward_impl(self, target, weight_ref(weight), reduction, ignore_index, op.outputs_[0], op.outputs_[1]);
  return std::make_tuple(std::move(op.outputs_[0]), std::move(op.outputs_[1]));
}
std::tuple<at::Tensor&, at::Tensor&> nll_loss_forward_out(const at::Tensor& self, const at::Tensor& target,
                                                          const c10::optional<at::Tensor>& weight, int64_t reduction,
                                                          int64_t ignore_index, at::Tensor& output, at::Tensor& total_weight) {
  const c10::DeviceGuard guard(self.device());
  OutMeta<at::meta::structured_nll_loss_forward> op(output, total_weight);
  op.meta(self, target, weight_ref(weight), reduction, ignore_index);
  nll_forward_impl(self, target, weight_ref(weight), reduction, ignore_index, output, total_weight);
  return std::forward_as_tuple(output, total_weight);
}
at::Tensor nll_loss_backward(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                             const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index,
                             const at::Tensor& total_weight) {
  const c10::DeviceGuard guard(self.device());
  FunctionalMeta<at::meta::structured_nll_loss_backward> op;
  op.meta(grad_output, self, target, weight_ref(weight), reduction, ignore_index, total_weight);
  nll_backward_impl(grad_output, self, target, weight_ref(weight), reduction, ignore_index, total_weight, op.outputs_[0]);
  return std::move(op.outputs_[0]);
}
at::Tensor& nll_loss_backward_out(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                                  const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index,
                                  const at::Tensor& total_weight, at::Tensor& grad_input) {
  const c10::DeviceGuard guard(self.device());
  OutMeta<at::meta::structured_nll_loss_backward> op(grad_input, grad_input);
  op.meta(grad_output, self, target, weight_ref(weight), reduction, ignore_index, total_weight);
  nll_backward_impl(grad_output, self, target, weight_ref(weight), reduction, ignore_index, total_weight, grad_input);
  return grad_input;
}

// ---- nll_loss2d ------------------------------------------------------------------------------------------------
// (N, C, H, W) log-probabilities, (N, H, W) targets.  Not a structured op upstream: shapes are checked and outputs
// resized here, with the messages of libtorch's CPU kernel.
void check_nll2d_inputs(const at::Tensor& self, const at::Tensor& target, const at::Tensor& weight) {
  TORCH_CHECK(target.dim() == 3, "only batches of spatial targets supported (3D tensors) but got targets of dimension: ", target.dim());
  TORCH_CHECK(self.dim() == 4, "only batches of spatial inputs supported (4D tensors), but got input of dimension: ", self.dim());
  TORCH_CHECK(!weight.defined() || weight.numel() == self.size(1), "weight tensor should be defined either for all or no classes");
  TORCH_CHECK(self.size(0) == target.size(0) && self.size(2) == target.size(1) && self.size(3) == target.size(2),
              "size mismatch (got input: ", self.sizes(), " , target: ", target.sizes());
}

sb_nll_nd_args nll2d_args(const at::Tensor& input, const at::Tensor& tgt, const at::Tensor& weight, int64_t reduction,
                          int64_t ignore_index) {
  sb_nll_nd_args a{};
  a.log_probs = input.const_data_ptr();
  a.dtype = dtype_code(input.scalar_type());
  TORCH_CHECK(tgt.scalar_type() == at::kLong || tgt.scalar_type() == at::kByte,
              "expected scalar type Long or Byte for target but found ", tgt.scalar_type());
  a.target_dtype = dtype_code(tgt.scalar_type());
  a.target = tgt.const_data_ptr();
  a.weight = weight.defined() ? weight.const_data_ptr() : nullptr;
  a.outer = input.size(0);
  a.classes = input.size(1);
  a.inner = input.size(2) * input.size(3);
  a.ignore_index = ignore_index;
  a.reduction = reduction_code(reduction);
  a.status = status_word(input.device().index());
  return a;
}

std::tuple<at::Tensor&, at::Tensor&> nll_loss2d_forward_out(const at::Tensor& self, const at::Tensor& target,
                                                            const c10::optional<at::Tensor>& weight_opt, int64_t reduction,
                                                            int64_t ignore_index, at::Tensor& output, at::Tensor& total_weight) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor weight;
  if (weight_opt.has_value() && weight_opt->defined()) weight = weight_opt->contiguous().to(self.scalar_type());
  check_nll2d_inputs(self, target, weight);
  const int red = reduction_code(reduction);
  total_weight.resize_({});
  if (red == SB_REDUCTION_NONE) output.resize_({self.size(0), self.size(2), self.size(3)});
  else output.resize_({});
  TORCH_CHECK(output.scalar_type() == self.scalar_type() && total_weight.scalar_type() == self.scalar_type(),
              "nll_loss2d: outputs must have the input's dtype");
  const at::Tensor input = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  at::Tensor result = output.is_contiguous() ? output : at::empty(output.sizes(), output.options());
  if (red == SB_REDUCTION_NONE) total_weight.zero_();  // not written by the kernel in this mode
  sb_nll_nd_args a = nll2d_args(input, tgt, weight, reduction, ignore_index);
  at::Tensor scratch;
  const size_t need = sb_nll_loss_nd_scratch_bytes(&a);
  if (need) {
    scratch = at::empty({static_cast<int64_t>(need)}, input.options().dtype(at::kByte));
    a.scratch = scratch.data_ptr();
    a.scratch_bytes = need;
  }
  check_kernel(sb_nll_loss_nd_forward(&a, result.data_ptr(), total_weight.data_ptr(), stream_of(input)), "supa nll_loss2d_forward");
  if (!result.is_same(output)) output.copy_(result);
  return std::forward_as_tuple(output, total_weight);
}

std::tuple<at::Tensor, at::Tensor> nll_loss2d_forward(const at::Tensor& self, const at::Tensor& target,
                                                      const c10::optional<at::Tensor>& weight, int64_t reduction,
                                                      int64_t ignore_index) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor output = at::empty({0}, self.options());
  at::Tensor total_weight = at::empty({0}, self.options());
  nll_loss2d_forward_out(self, target, weight, reduction, ignore_index, output, total_weight);
  return std::make_tuple(std::move(output), std::move(total_weight));
}

at::Tensor& nll_loss2d_backward_out(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                                    const c10::optional<at::Tensor>& weight_opt, int64_t reduction, int64_t ignore_index,
                                    const at::Tensor& total_weight, at::Tensor& grad_input) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor weight;
  if (weight_opt.has_value() && weight_opt->defined()) weight = weight_opt->contiguous().to(self.scalar_type());
  check_nll2d_inputs(self, target, weight);
  grad_input.resize_(self.sizes());
  TORCH_CHECK(total_weight.numel() == 1, "expected total_weight to be a single element tensor, got: ", total_weight.sizes(), " (",
              total_weight.numel(), " elements)");
  if (self.numel() == 0) return grad_input;
  const int red = reduction_code(reduction);
  if (red == SB_REDUCTION_NONE) {
    TORCH_CHECK(grad_output.dim() == 3 && grad_output.size(0) == self.size(0) && grad_output.size(1) == self.size(2) &&
                    grad_output.size(2) == self.size(3),
                "grad_output must have the shape of target for reduction none, got ", grad_output.sizes());
  } else {
    TORCH_CHECK(grad_output.numel() == 1, "Expected a single element grad_output tensor, but got: ", grad_output.sizes());
  }
  const at::Tensor input = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  at::Tensor go = grad_output.contiguous();
  if (go.scalar_type() != input.scalar_type()) go = go.to(input.scalar_type());
  at::Tensor tw = total_weight.scalar_type() == input.scalar_type() ? total_weight : total_weight.to(input.scalar_type());
  at::Tensor result = grad_input.is_contiguous() ? grad_input : at::empty(grad_input.sizes(), grad_input.options());
  const sb_nll_nd_args a = nll2d_args(input, tgt, weight, reduction, ignore_index);
  check_kernel(sb_nll_loss_nd_backward(&a, go.const_data_ptr(), tw.const_data_ptr(), result.data_ptr(), stream_of(input)),
               "supa nll_loss2d_backward");
  if (!result.is_same(grad_input)) grad_input.copy_(result);
  return grad_input;
}

at::Tensor nll_loss2d_backward(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                               const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index,
                               const at::Tensor& total_weight) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor grad_input = at::empty({0}, self.options());
  nll_loss2d_backward_out(grad_output, self, target, weight, reduction, ignore_index, total_weight, grad_input);
  return grad_input;
}

// ---- cross entropy ---------------------------------------------------------------------------------------------
// Which calls take the fused kernel.  Wider than the reference's predicate (CrossEntropyLoss.cpp:23-33: 2-D
// fp32, no smoothing): 16-bit logits, label smoothing, 1-D logits and class weights (without smoothing) are fused
// too; weights together with smoothing, probability targets, fp64 and K-dimensional inputs go to libtorch's composite (log_softmax + nll_loss ...),
// whose pieces are registered above.
bool fused_path(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, double label_smoothing) {
  // class weights are fused when there is no label smoothing (the smoothing term would weight every class of a row)
  bool has_weight = weight.has_value() && weight->defined();
  if (has_weight && label_smoothing == 0.0 && is_supa(*weight) && weight->dim() == 1 && weight->numel() == self.size(-1) &&
      c10::isFloatingType(weight->scalar_type()))
    has_weight = false;  // this one the kernel takes
  const at::ScalarType dt = self.scalar_type();
  const bool dtype_ok = dt == at::kFloat || dt == at::kBFloat16 || dt == at::kHalf;
  const bool shape_ok = (self.dim() == 2 && target.dim() == 1 && target.size(0) == self.size(0)) || (self.dim() == 1 && target.dim() == 0);
  return dtype_ok && shape_ok && !has_weight && target.scalar_type() == at::kLong && is_supa(target) && label_smoothing >= 0.0 &&
         label_smoothing <= 1.0 && self.size(-1) > 0;
}

// The class weights as the kernel wants them: fp32, contiguous; undefined when there are none.
at::Tensor fused_weight(const c10::optional<at::Tensor>& weight) {
  if (!weight.has_value() || !weight->defined()) return at::Tensor();
  return weight->to(at::kFloat).contiguous();
}

struct FusedResult {
  at::Tensor loss;      // 0-d in the logits' dtype (mean, sum) or [N] (none)
  at::Tensor grad;      // [N, C] logit gradient for an upstream gradient of 1 (mean, sum with want_grad)
  at::Tensor row_lse;   // [N] fp32 (none with want_grad)
  at::Tensor applied;   // two device floats used alternately: the upstream factor currently folded into `grad`
};

// The launch sequence of include/supa_b200_kernels.h: count -> [all-reduce] -> fused sweep -> loss sum ->
// [all-reduce] -> finish.  `comm` is null on a single GPU.
FusedResult fused_forward(const at::Tensor& self, const at::Tensor& target, const at::Tensor& class_weight, int64_t reduction,
                          int64_t ignore_index, double label_smoothing, bool want_grad, NcclComm* comm) {
  const c10::DeviceGuard guard(self.device());
  const at::Tensor logits = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  const int64_t rows = logits.dim() == 1 ? 1 : logits.size(0);
  const int64_t classes = logits.size(-1);
  const int red = reduction_code(reduction);
  sb_stream_t stream = stream_of(logits);
  FusedResult r;
  const auto f32 = logits.options().dtype(at::kFloat);
  at::Tensor row_loss = at::empty({std::max<int64_t>(rows, 1)}, f32);
  at::Tensor acc = at::empty({2}, logits.options().dtype(at::kDouble));

  sb_ce_args a{};
  a.logits = logits.const_data_ptr();
  a.dtype = dtype_code(logits.scalar_type());
  a.reduction = red;
  a.target = tgt.const_data_ptr<int64_t>();
  a.row_loss = row_loss.data_ptr<float>();
  a.acc = acc.data_ptr<double>();
  a.rows = rows;
  a.classes = classes;
  a.ignore_index = ignore_index;
  a.label_smoothing = static_cast<float>(label_smoothing);
  a.grad_scale = 1.f;
  a.status = status_word(logits.device().index());
  a.class_weight = class_weight.defined() ? class_weight.const_data_ptr<float>() : nullptr;  // fp32, contiguous (see fused_weight)

  if (red == SB_REDUCTION_NONE) {
    if (want_grad) {
      r.row_lse = at::empty({std::max<int64_t>(rows, 1)}, f32);
      a.row_lse = r.row_lse.data_ptr<float>();
    }
    check_kernel(sb_ce_forward_backward(&a, stream), "supa cross_entropy");
    at::Tensor out = logits.dim() == 1 ? row_loss.reshape({}) : row_loss.narrow(0, 0, rows);
    r.loss = out.scalar_type() == logits.scalar_type() ? out : out.to(logits.scalar_type());
    return r;
  }

  if (a.class_weight)
    check_kernel(sb_ce_count_weighted(tgt.const_data_ptr<int64_t>(), a.class_weight, rows, classes, ignore_index, acc.data_ptr<double>(),
                                      a.status, stream),
                 "supa cross_entropy weight sum");
  else
    check_kernel(sb_ce_count_valid(tgt.const_data_ptr<int64_t>(), rows, classes, ignore_index, acc.data_ptr<double>(), a.status, stream),
                 "supa cross_entropy count");
  if (comm) comm->all_reduce_sum_f64(acc.data_ptr<double>() + 1, 1, stream);
  if (want_grad) {
    r.grad = at::empty_like(logits);
    a.grad_logits = r.grad.data_ptr();
  }
  check_kernel(sb_ce_forward_backward(&a, stream), "supa cross_entropy");
  r.loss = at::empty({}, logits.options());
  if (!comm) {
    check_kernel(sb_ce_loss_sum_finish(row_loss.const_data_ptr<float>(), rows, acc.data_ptr<double>(), red, r.loss.data_ptr(),
                                       dtype_code(logits.scalar_type()), stream),
                 "supa cross_entropy loss sum");
  } else {
    check_kernel(sb_ce_loss_sum(row_loss.const_data_ptr<float>(), rows, acc.data_ptr<double>(), stream), "supa cross_entropy loss sum");
    comm->all_reduce_sum_f64(acc.data_ptr<double>(), 1, stream);
    check_kernel(sb_ce_loss_finish(acc.const_data_ptr<double>(), red, r.loss.data_ptr(), dtype_code(logits.scalar_type()), stream),
                 "supa cross_entropy loss finish");
  }
  if (want_grad) {
    r.applied = at::empty({2}, f32);  // written by the first rescale; until then the factor is 1 by construction
  }
  return r;
}

class CrossEntropyFunction : public torch::autograd::Function<CrossEntropyFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& self, const at::Tensor& target,
                            const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index, double label_smoothing,
                            int64_t comm_handle) {
    NcclComm* comm = comm_handle ? NcclComm::from_handle(comm_handle) : nullptr;
    const at::Tensor class_weight = fused_weight(weight);
    FusedResult r = fused_forward(self, target, class_weight, reduction, ignore_index, label_smoothing, /*want_grad=*/true, comm);
    ctx->saved_data["reduction"] = reduction;
    ctx->saved_data["ignore_index"] = ignore_index;
    ctx->saved_data["label_smoothing"] = label_smoothing;
    if (reduction == at::Reduction::None) ctx->save_for_backward({self, target, r.row_lse, class_weight});
    else ctx->save_for_backward({r.grad, r.applied});
    ctx->saved_data["applied_slot"] = static_cast<int64_t>(-1);  // which word of `applied` is valid; -1 = none (factor 1)
    ctx->saved_data["shape_1d"] = self.dim() == 1;
    return r.loss;
  }

  static std::vector<at::Tensor> backward(torch::autograd::AutogradContext* ctx, std::vector<at::Tensor> grad_outputs) {
    const auto saved = ctx->get_saved_variables();
    const int64_t reduction = ctx->saved_data["reduction"].toInt();
    const at::Tensor& go = grad_outputs[0];
    at::Tensor grad_self;
    if (!go.defined()) return {grad_self, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
    if (reduction == at::Reduction::None) {
      // per-row upstream gradients: one more fused sweep with the saved logits (1 read + 1 write)
      const at::Tensor logits = saved[0].contiguous();
      const at::Tensor tgt = saved[1].contiguous();
      const c10::DeviceGuard guard(logits.device());
      const int64_t rows = logits.dim() == 1 ? 1 : logits.size(0);
      at::Tensor row_go = go.reshape({rows}).to(at::kFloat).contiguous();
      at::Tensor row_loss = at::empty({std::max<int64_t>(rows, 1)}, row_go.options());
      grad_self = at::empty_like(logits);
      sb_ce_args a{};
      a.logits = logits.const_data_ptr();
      a.dtype = dtype_code(logits.scalar_type());
      a.reduction = SB_REDUCTION_NONE;
      a.target = tgt.const_data_ptr<int64_t>();
      a.grad_logits = grad_self.data_ptr();
      a.row_loss = row_loss.data_ptr<float>();
      a.row_grad_out = row_go.const_data_ptr<float>();
      a.rows = rows;
      a.classes = logits.size(-1);
      a.ignore_index = ctx->saved_data["ignore_index"].toInt();
      a.label_smoothing = static_cast<float>(ctx->saved_data["label_smoothing"].toDouble());
      a.grad_scale = 1.f;
      a.status = status_word(logits.device().index());
      a.class_weight = saved[3].defined() ? saved[3].const_data_ptr<float>() : nullptr;
      check_kernel(sb_ce_forward_backward(&a, stream_of(logits)), "supa cross_entropy backward");
      grad_self = grad_self.view(saved[0].sizes());
    } else {
      // The stored gradient carries the factor `applied` (1 after forward).  Fold in the new upstream value
      // on the device; the sweep is skipped there when nothing changes.
      grad_self = saved[0];
      const at::Tensor applied = saved[1];
      const c10::DeviceGuard guard(grad_self.device());
      at::Tensor scale = go.reshape({1});
      if (!is_supa(scale)) scale = scale.to(grad_self.device());
      const at::ScalarType st = scale.scalar_type();
      if (st != at::kFloat && st != at::kBFloat16 && st != at::kHalf && st != at::kDouble) scale = scale.to(at::kFloat);
      scale = scale.contiguous();
      const int64_t slot = ctx->saved_data["applied_slot"].toInt();
      const int64_t next = slot < 0 ? 0 : 1 - slot;
      check_kernel(sb_ce_rescale_grad(grad_self.data_ptr(), dtype_code(grad_self.scalar_type()), grad_self.numel(),
                                      scale.const_data_ptr(), dtype_code(scale.scalar_type()),
                                      slot < 0 ? nullptr : applied.const_data_ptr<float>() + slot, applied.data_ptr<float>() + next,
                                      stream_of(grad_self)),
                   "supa cross_entropy rescale");
      ctx->saved_data["applied_slot"] = next;
      if (ctx->saved_data["shape_1d"].toBool()) grad_self = grad_self.reshape({grad_self.size(-1)});
    }
    return {grad_self, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

at::Tensor cross_entropy_fused(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                               int64_t reduction, int64_t ignore_index, double label_smoothing, int64_t comm_handle) {
  const bool has_weight = weight.has_value() && weight->defined();
  if (at::GradMode::is_enabled() && self.requires_grad())
    return CrossEntropyFunction::apply(self, target, has_weight ? weight : c10::nullopt, reduction, ignore_index, label_smoothing,
                                       comm_handle);
  NcclComm* comm = comm_handle ? NcclComm::from_handle(comm_handle) : nullptr;
  return fused_forward(self, target, fused_weight(weight), reduction, ignore_index, label_smoothing, /*want_grad=*/false, comm).loss;
}

at::Tensor cross_entropy_loss(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                              int64_t reduction, int64_t ignore_index, double label_smoothing) {
  if (!fused_path(self, target, weight, label_smoothing))
    return at::native::cross_entropy_loss_symint(self, target, weight, reduction, c10::SymInt(ignore_index), label_smoothing);
  return cross_entropy_fused(self, target, weight, reduction, ignore_index, label_smoothing, 0);
}

// supa_b200::sharded_cross_entropy: the same fused path with the two scalar all-reduces of the row-sharded
// multi-GPU protocol (valid-row count before the sweep, loss sum after it) on the communicator `comm`.
at::Tensor sharded_cross_entropy(const at::Tensor& self, const at::Tensor& target, int64_t reduction, int64_t ignore_index,
                                 double label_smoothing, int64_t comm) {
  TORCH_CHECK(fused_path(self, target, c10::nullopt, label_smoothing),
              "sharded_cross_entropy: expected [rows, classes] fp32/bf16/fp16 logits and int64 class targets on a supa device");
  return cross_entropy_fused(self, target, c10::nullopt, reduction, ignore_index, label_smoothing, reduction == at::Reduction::None ? 0 : comm);
}

}  // namespace
}  // namespace supa

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_log_softmax", TORCH_FN(supa::log_softmax));
  m.impl("_log_softmax.out", TORCH_FN(supa::log_softmax_out));
  m.impl("_log_softmax_backward_data", TORCH_FN(supa::log_softmax_backward));
  m.impl("_log_softmax_backward_data.out", TORCH_FN(supa::log_softmax_backward_out));
  m.impl("_softmax", TORCH_FN(supa::softmax));
  m.impl("_softmax.out", TORCH_FN(supa::softmax_out));
  m.impl("_softmax_backward_data", TORCH_FN(supa::softmax_backward));
  m.impl("_softmax_backward_data.out", TORCH_FN(supa::softmax_backward_out));
  m.impl("nll_loss_forward", TORCH_FN(supa::nll_loss_forward));
  m.impl("nll_loss_forward.output", TORCH_FN(supa::nll_loss_forward_out));
  m.impl("nll_loss_backward", TORCH_FN(supa::nll_loss_backward));
  m.impl("nll_loss_backward.grad_input", TORCH_FN(supa::nll_loss_backward_out));
  m.impl("nll_loss2d_forward", TORCH_FN(supa::nll_loss2d_forward));
  m.impl("nll_loss2d_forward.output", TORCH_FN(supa::nll_loss2d_forward_out));
  m.impl("nll_loss2d_backward", TORCH_FN(supa::nll_loss2d_backward));
  m.impl("nll_loss2d_backward.grad_input", TORCH_FN(supa::nll_loss2d_backward_out));
  m.impl("cross_entropy_loss", TORCH_FN(supa::cross_entropy_loss));
}

// With a backend kernel registered for a CompositeImplicitAutograd operator, the Autograd key of the
// backend must fall through to it (VariableFallbackKernel.cpp:31-33 of the reference).
TORCH_LIBRARY_IMPL(_, AutogradPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

TORCH_LIBRARY(supa_b200, m) {
  m.def("sharded_cross_entropy(Tensor self, Tensor target, int reduction, int ignore_index, float label_smoothing, int comm) -> Tensor");
}
TORCH_LIBRARY_IMPL(supa_b200, PrivateUse1, m) { m.impl("sharded_cross_entropy", TORCH_FN(supa::sharded_cross_entropy)); }

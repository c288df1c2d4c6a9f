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
#include "dist/PeerExchange.h"

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
// fp32, no smoothing): 16-bit logits, label smoothing, 1-D logits and class weights (with or without smoothing) are
// fused too; probability targets, fp64 and K-dimensional inputs go to libtorch's composite (log_softmax + nll_loss ...),
// whose pieces are registered above.
bool fused_path(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, double label_smoothing) {
  bool has_weight = weight.has_value() && weight->defined();
  if (has_weight && is_supa(*weight) && weight->dim() == 1 && weight->numel() == self.size(-1) && c10::isFloatingType(weight->scalar_type()))
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

// How the ranks of a row-sharded job exchange the two scalars: through peer memory inside the bookkeeping kernels
// (preferred), else through two NCCL all-reduces; neither on a single GPU.
struct Exchange {
  NcclComm* nccl = nullptr;
  PeerExchange* peer = nullptr;
  bool any() const { return nccl || peer; }
};

struct FusedResult {
  at::Tensor loss;      // 0-d in the logits' dtype (mean, sum) or [N] (none)
  at::Tensor grad;      // [N, C] logit gradient for an upstream gradient of 1 (mean, sum with want_grad)
  at::Tensor row_lse;   // [N] fp32 (none with want_grad)
  at::Tensor applied;   // two device floats used alternately: the upstream factor currently folded into `grad`
  at::Tensor acc;       // {loss sum, denominator} as two doubles (kept for a backward that runs the sweep again)
};

sb_ce_args ce_args(const at::Tensor& logits, const at::Tensor& tgt, const at::Tensor& class_weight, int red, int64_t ignore_index,
                   double label_smoothing) {
  sb_ce_args a{};
  a.logits = logits.const_data_ptr();
  a.dtype = dtype_code(logits.scalar_type());
  a.reduction = red;
  a.target = tgt.const_data_ptr<int64_t>();
  a.rows = logits.dim() == 1 ? 1 : logits.size(0);
  a.classes = logits.size(-1);
  a.ignore_index = ignore_index;
  a.label_smoothing = static_cast<float>(label_smoothing);
  a.grad_scale = 1.f;
  a.status = status_word(logits.device().index());
  a.class_weight = class_weight.defined() ? class_weight.const_data_ptr<float>() : nullptr;  // fp32, contiguous (see fused_weight)
  return a;
}

// The launch sequence of include/supa_b200_kernels.h: count [+ exchange] -> fused sweep -> loss sum [+ exchange] + finish.
// want_grad: the sweep also writes the logit gradient, scaled for an upstream gradient of 1.
FusedResult fused_forward(const at::Tensor& self, const at::Tensor& target, const at::Tensor& class_weight, int64_t reduction,
                          int64_t ignore_index, double label_smoothing, bool want_grad, bool want_lse, Exchange ex) {
  const c10::DeviceGuard guard(self.device());
  const at::Tensor logits = self.contiguous();
  const at::Tensor tgt = target.contiguous();
  const int red = reduction_code(reduction);
  sb_stream_t stream = stream_of(logits);
  FusedResult r;
  const auto f32 = logits.options().dtype(at::kFloat);
  sb_ce_args a = ce_args(logits, tgt, class_weight, red, ignore_index, label_smoothing);
  const int64_t rows = a.rows;
  at::Tensor row_loss = at::empty({std::max<int64_t>(rows, 1)}, f32);
  a.row_loss = row_loss.data_ptr<float>();

  if (red == SB_REDUCTION_NONE) {
    if (want_lse) {
      r.row_lse = at::empty({std::max<int64_t>(rows, 1)}, f32);
      a.row_lse = r.row_lse.data_ptr<float>();
    }
    check_kernel(sb_ce_forward_backward(&a, stream), "supa cross_entropy");
    at::Tensor out = logits.dim() == 1 ? row_loss.reshape({}) : row_loss.narrow(0, 0, rows);
    r.loss = out.scalar_type() == logits.scalar_type() ? out : out.to(logits.scalar_type());
    return r;
  }

  r.acc = at::empty({2}, logits.options().dtype(at::kDouble));
  a.acc = r.acc.data_ptr<double>();
  if (want_grad) {  // allocated before the count so that nothing sits between the count and the sweep on the stream
    r.grad = at::empty_like(logits);
    a.grad_logits = r.grad.data_ptr();
  }
  r.loss = at::empty({}, logits.options());
  if (ex.peer) {
    const sb_xchg x = ex.peer->next();
    check_kernel(sb_ce_count_exchange(a.target, a.class_weight, rows, a.classes, ignore_index, r.acc.data_ptr<double>(), a.status, &x, stream),
                 "supa cross_entropy count");
    a.flags = SB_CE_FLAG_AFTER_COUNT;
  } else {
    check_kernel(sb_ce_count_exchange(a.target, a.class_weight, rows, a.classes, ignore_index, r.acc.data_ptr<double>(), a.status, nullptr, stream),
                 "supa cross_entropy count");
    if (ex.nccl) ex.nccl->all_reduce_sum_f64(r.acc.data_ptr<double>() + 1, 1, stream);
    else a.flags = SB_CE_FLAG_AFTER_COUNT;
  }
  check_kernel(sb_ce_forward_backward(&a, stream), "supa cross_entropy");
  const int out_dtype = dtype_code(logits.scalar_type());
  if (ex.peer) {
    const sb_xchg x = ex.peer->next();
    check_kernel(sb_ce_loss_exchange(row_loss.const_data_ptr<float>(), rows, r.acc.data_ptr<double>(), red, r.loss.data_ptr(), out_dtype, a.status,
                                     &x, stream),
                 "supa cross_entropy loss sum");
  } else if (ex.nccl) {
    check_kernel(sb_ce_loss_sum(row_loss.const_data_ptr<float>(), rows, r.acc.data_ptr<double>(), stream), "supa cross_entropy loss sum");
    ex.nccl->all_reduce_sum_f64(r.acc.data_ptr<double>(), 1, stream);
    check_kernel(sb_ce_loss_finish(r.acc.const_data_ptr<double>(), red, r.loss.data_ptr(), out_dtype, stream), "supa cross_entropy loss finish");
  } else {
    check_kernel(sb_ce_loss_exchange(row_loss.const_data_ptr<float>(), rows, r.acc.data_ptr<double>(), red, r.loss.data_ptr(), out_dtype, a.status,
                                     nullptr, stream),
                 "supa cross_entropy loss sum");
  }
  if (want_grad) r.applied = at::empty({2}, f32);  // written by the first rescale; until then the factor is 1 by construction
  return r;
}

// The gradient a mean / sum forward stored carries the factor `applied` (1 after forward).  The first backward folds the
// upstream value in on the device, in place (the sweep is skipped there when it is 1), and hands the buffer out; later
// backward calls on a retained graph write into a fresh tensor, so no tensor handed out earlier changes under its holder.
at::Tensor apply_upstream(torch::autograd::AutogradContext* ctx, const at::Tensor& stored, const at::Tensor& applied, const at::Tensor& go) {
  const c10::DeviceGuard guard(stored.device());
  at::Tensor scale = go.reshape({1});
  if (!is_supa(scale)) scale = scale.to(stored.device());
  const at::ScalarType st = scale.scalar_type();
  if (st != at::kFloat && st != at::kBFloat16 && st != at::kHalf && st != at::kDouble) scale = scale.to(at::kFloat);
  scale = scale.contiguous();
  const int64_t slot = ctx->saved_data["applied_slot"].toInt();
  int32_t* status = status_word(stored.device().index());
  if (slot < 0) {
    check_kernel(sb_ce_rescale_grad(stored.const_data_ptr(), stored.data_ptr(), dtype_code(stored.scalar_type()), stored.numel(),
                                    scale.const_data_ptr(), dtype_code(scale.scalar_type()), nullptr, applied.data_ptr<float>(), status,
                                    stream_of(stored)),
                 "supa cross_entropy rescale");
    ctx->saved_data["applied_slot"] = static_cast<int64_t>(0);
    return stored;
  }
  at::Tensor fresh = at::empty_like(stored);
  check_kernel(sb_ce_rescale_grad(stored.const_data_ptr(), fresh.data_ptr(), dtype_code(stored.scalar_type()), stored.numel(),
                                  scale.const_data_ptr(), dtype_code(scale.scalar_type()), applied.const_data_ptr<float>() + slot, nullptr,
                                  status, stream_of(stored)),
               "supa cross_entropy rescale");
  return fresh;
}

// Autograd node.  Three ways to the logit gradient:
//  * mean / sum on fp32 and bf16 logits: the forward sweep already wrote it, scaled for an upstream gradient of 1;
//    the first backward folds the real upstream value into that buffer in place (skipped on the device when it is 1)
//    and hands the buffer out; later backward calls on a retained graph write into a fresh tensor, so no tensor handed
//    out earlier changes under its holder;
//  * fp16 logits: a gradient stored before the upstream factor is known would flush to zero (p / |V| < 6e-8 for most
//    classes) and a loss scale applied afterwards could not bring it back, so forward keeps the logits and backward
//    runs the sweep with the upstream value folded in before anything is rounded to fp16;
//  * reduction none: per-row upstream values, same second sweep.
class CrossEntropyFunction : public torch::autograd::Function<CrossEntropyFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& self, const at::Tensor& target,
                            const c10::optional<at::Tensor>& weight, int64_t reduction, int64_t ignore_index, double label_smoothing,
                            int64_t comm_handle, int64_t peer_handle) {
    Exchange ex;
    if (comm_handle) ex.nccl = NcclComm::from_handle(comm_handle);
    if (peer_handle) ex.peer = PeerExchange::from_handle(peer_handle);
    const at::Tensor class_weight = fused_weight(weight);
    const bool recompute = reduction == at::Reduction::None || self.scalar_type() == at::kHalf;
    FusedResult r = fused_forward(self, target, class_weight, reduction, ignore_index, label_smoothing, /*want_grad=*/!recompute,
                                  /*want_lse=*/false, ex);
    ctx->saved_data["reduction"] = reduction;
    ctx->saved_data["ignore_index"] = ignore_index;
    ctx->saved_data["label_smoothing"] = label_smoothing;
    ctx->saved_data["recompute"] = recompute;
    if (recompute) ctx->save_for_backward({self, target, class_weight, r.acc});
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
    const auto result = [&] { return std::vector<at::Tensor>{grad_self, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()}; };
    if (!go.defined()) return result();
    if (ctx->saved_data["recompute"].toBool()) {
      // one more fused sweep with the saved logits (1 read + 1 write), the upstream values folded in per row
      const at::Tensor logits = saved[0].contiguous();
      const at::Tensor tgt = saved[1].contiguous();
      const c10::DeviceGuard guard(logits.device());
      const int red = reduction_code(reduction);
      sb_ce_args a = ce_args(logits, tgt, saved[2], red, ctx->saved_data["ignore_index"].toInt(), ctx->saved_data["label_smoothing"].toDouble());
      at::Tensor upstream = go;
      if (!is_supa(upstream)) upstream = upstream.to(logits.device());
      at::Tensor row_go = upstream.to(at::kFloat).reshape({-1}).expand({a.rows}).contiguous();
      at::Tensor row_loss = at::empty({std::max<int64_t>(a.rows, 1)}, row_go.options());
      grad_self = at::empty_like(logits);
      a.grad_logits = grad_self.data_ptr();
      a.row_loss = row_loss.data_ptr<float>();
      a.row_grad_out = row_go.const_data_ptr<float>();
      if (red != SB_REDUCTION_NONE) a.acc = saved[3].const_data_ptr<double>();  // the (global) denominator of `mean`
      check_kernel(sb_ce_forward_backward(&a, stream_of(logits)), "supa cross_entropy backward");
      grad_self = grad_self.view(saved[0].sizes());
      return result();
    }
    grad_self = apply_upstream(ctx, saved[0], saved[1], go);
    if (ctx->saved_data["shape_1d"].toBool()) grad_self = grad_self.reshape({grad_self.size(-1)});
    return result();
  }
};

at::Tensor cross_entropy_fused(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                               int64_t reduction, int64_t ignore_index, double label_smoothing, int64_t comm_handle, int64_t peer_handle) {
  const bool has_weight = weight.has_value() && weight->defined();
  if (at::GradMode::is_enabled() && self.requires_grad())
    return CrossEntropyFunction::apply(self, target, has_weight ? weight : c10::nullopt, reduction, ignore_index, label_smoothing,
                                       comm_handle, peer_handle);
  Exchange ex;
  if (comm_handle) ex.nccl = NcclComm::from_handle(comm_handle);
  if (peer_handle) ex.peer = PeerExchange::from_handle(peer_handle);
  return fused_forward(self, target, fused_weight(weight), reduction, ignore_index, label_smoothing, /*want_grad=*/false, /*want_lse=*/false, ex)
      .loss;
}

// ---- class-probability targets ---------------------------------------------------------------------------------------
// Float targets of the logits' shape (CrossEntropyLoss.cpp:43-45 and cross_entropy_prob_kernel of the reference).
bool prob_path(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, double label_smoothing) {
  const at::ScalarType dt = self.scalar_type();
  if (!(dt == at::kFloat || dt == at::kBFloat16 || dt == at::kHalf)) return false;
  if (!c10::isFloatingType(target.scalar_type()) || !is_supa(target) || target.sizes() != self.sizes()) return false;
  if (!(self.dim() == 2 || self.dim() == 1) || self.size(-1) == 0) return false;
  if (weight.has_value() && weight->defined() &&
      !(is_supa(*weight) && weight->dim() == 1 && weight->numel() == self.size(-1) && c10::isFloatingType(weight->scalar_type())))
    return false;
  if (at::GradMode::is_enabled() && target.requires_grad()) return false;  // a gradient for the targets: the composite has it
  return label_smoothing >= 0.0 && label_smoothing <= 1.0;
}

struct ProbResult {
  at::Tensor loss, grad;
};

// One launch of the fused kernel (+ the fixed-order sum for mean / sum).  row_go: per-row upstream values (reduction none
// in backward), undefined for 1.
ProbResult prob_forward(const at::Tensor& self, const at::Tensor& target, const at::Tensor& class_weight, int64_t reduction,
                        double label_smoothing, bool want_grad, const at::Tensor& row_go, bool want_loss) {
  const c10::DeviceGuard guard(self.device());
  const at::Tensor logits = self.contiguous();
  at::Tensor tgt = target.contiguous();
  if (tgt.scalar_type() != logits.scalar_type()) tgt = tgt.to(logits.scalar_type());
  const int red = reduction_code(reduction);
  const int64_t rows = logits.dim() == 1 ? 1 : logits.size(0);
  const auto f32 = logits.options().dtype(at::kFloat);
  at::Tensor row_loss = at::empty({std::max<int64_t>(rows, 1)}, f32);
  ProbResult r;
  sb_ce_prob_args a{};
  a.logits = logits.const_data_ptr();
  a.target = tgt.const_data_ptr();
  a.dtype = dtype_code(logits.scalar_type());
  a.row_loss = row_loss.data_ptr<float>();
  a.class_weight = class_weight.defined() ? class_weight.const_data_ptr<float>() : nullptr;
  a.rows = rows;
  a.classes = logits.size(-1);
  a.label_smoothing = static_cast<float>(label_smoothing);
  const float inv = (red == SB_REDUCTION_MEAN && rows > 0) ? static_cast<float>(1.0 / static_cast<double>(rows)) : 1.f;
  a.grad_scale = inv;
  a.loss_scale = inv;
  if (row_go.defined()) a.row_grad_out = row_go.const_data_ptr<float>();
  if (want_grad) {
    r.grad = at::empty_like(logits);
    a.grad_logits = r.grad.data_ptr();
  }
  sb_stream_t stream = stream_of(logits);
  check_kernel(sb_ce_prob_forward_backward(&a, stream), "supa cross_entropy (probability targets)");
  if (!want_loss) return r;
  if (red == SB_REDUCTION_NONE) {
    at::Tensor out = logits.dim() == 1 ? row_loss.reshape({}) : row_loss.narrow(0, 0, rows);
    r.loss = out.scalar_type() == logits.scalar_type() ? out : out.to(logits.scalar_type());
    return r;
  }
  r.loss = at::empty({}, logits.options());
  if (rows == 0) {  // mean of nothing: NaN, sum: 0 (the CPU's results)
    r.loss.fill_(red == SB_REDUCTION_MEAN ? std::numeric_limits<double>::quiet_NaN() : 0.0);
    return r;
  }
  at::Tensor acc = at::empty({2}, logits.options().dtype(at::kDouble));
  check_kernel(sb_ce_loss_sum_finish(row_loss.const_data_ptr<float>(), rows, acc.data_ptr<double>(), SB_REDUCTION_SUM, r.loss.data_ptr(),
                                     dtype_code(logits.scalar_type()), stream),
               "supa cross_entropy loss sum");
  return r;
}

class CrossEntropyProbFunction : public torch::autograd::Function<CrossEntropyProbFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& self, const at::Tensor& target,
                            const c10::optional<at::Tensor>& weight, int64_t reduction, double label_smoothing) {
    const at::Tensor class_weight = fused_weight(weight);
    // fp16 and reduction none form the gradient in backward, with the upstream values folded in before rounding
    const bool recompute = reduction == at::Reduction::None || self.scalar_type() == at::kHalf;
    ProbResult r = prob_forward(self, target, class_weight, reduction, label_smoothing, !recompute, at::Tensor(), true);
    ctx->saved_data["reduction"] = reduction;
    ctx->saved_data["label_smoothing"] = label_smoothing;
    ctx->saved_data["recompute"] = recompute;
    ctx->saved_data["applied_slot"] = static_cast<int64_t>(-1);
    if (recompute) ctx->save_for_backward({self, target, class_weight});
    else ctx->save_for_backward({r.grad, at::empty({2}, self.options().dtype(at::kFloat))});
    return r.loss;
  }
  static std::vector<at::Tensor> backward(torch::autograd::AutogradContext* ctx, std::vector<at::Tensor> grad_outputs) {
    const auto saved = ctx->get_saved_variables();
    const at::Tensor& go = grad_outputs[0];
    at::Tensor grad_self;
    if (go.defined()) {
      if (ctx->saved_data["recompute"].toBool()) {
        const at::Tensor& self = saved[0];
        const int64_t rows = self.dim() == 1 ? 1 : self.size(0);
        at::Tensor upstream = is_supa(go) ? go : go.to(self.device());
        at::Tensor row_go = upstream.to(at::kFloat).reshape({-1}).expand({rows}).contiguous();
        grad_self = prob_forward(self, saved[1], saved[2], ctx->saved_data["reduction"].toInt(), ctx->saved_data["label_smoothing"].toDouble(),
                                 true, row_go, false)
                        .grad.view(self.sizes());
      } else {
        grad_self = apply_upstream(ctx, saved[0], saved[1], go).view(saved[0].sizes());
      }
    }
    return {grad_self, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

at::Tensor cross_entropy_prob(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, int64_t reduction,
                              int64_t ignore_index, double label_smoothing) {
  TORCH_CHECK(ignore_index < 0, "ignore_index is not supported for floating point target");
  const bool has_weight = weight.has_value() && weight->defined();
  if (at::GradMode::is_enabled() && self.requires_grad())
    return CrossEntropyProbFunction::apply(self, target, has_weight ? weight : c10::nullopt, reduction, label_smoothing);
  return prob_forward(self, target, fused_weight(weight), reduction, label_smoothing, false, at::Tensor(), true).loss;
}

at::Tensor cross_entropy_loss(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                              int64_t reduction, int64_t ignore_index, double label_smoothing) {
  if (prob_path(self, target, weight, label_smoothing)) return cross_entropy_prob(self, target, weight, reduction, ignore_index, label_smoothing);
  if (!fused_path(self, target, weight, label_smoothing))
    return at::native::cross_entropy_loss_symint(self, target, weight, reduction, c10::SymInt(ignore_index), label_smoothing);
  return cross_entropy_fused(self, target, weight, reduction, ignore_index, label_smoothing, 0, 0);
}

// supa_b200::sharded_cross_entropy: the same fused path with the two scalar exchanges of the row-sharded
// multi-GPU protocol (valid-row count before the sweep, loss sum after it): through the peer-memory exchange `peer`
// when given, else through the NCCL communicator `comm`.
at::Tensor sharded_cross_entropy(const at::Tensor& self, const at::Tensor& target, int64_t reduction, int64_t ignore_index,
                                 double label_smoothing, int64_t comm, int64_t peer) {
  TORCH_CHECK(fused_path(self, target, c10::nullopt, label_smoothing),
              "sharded_cross_entropy: expected [rows, classes] fp32/bf16/fp16 logits and int64 class targets on a supa device");
  const bool none = reduction == at::Reduction::None;
  return cross_entropy_fused(self, target, c10::nullopt, reduction, ignore_index, label_smoothing, (none || peer) ? 0 : comm, none ? 0 : peer);
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
  m.def("sharded_cross_entropy(Tensor self, Tensor target, int reduction, int ignore_index, float label_smoothing, int comm, int peer=0) -> Tensor");
}
TORCH_LIBRARY_IMPL(supa_b200, PrivateUse1, m) { m.impl("sharded_cross_entropy", TORCH_FN(supa::sharded_cross_entropy)); }

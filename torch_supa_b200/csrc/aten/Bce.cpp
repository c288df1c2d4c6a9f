// binary_cross_entropy_with_logits on the supa device.
//
// The reference computes the unreduced loss with one TensorIterator kernel and reduces it with mean() / sum()
// (torch_supa/csrc/aten/ops/BinaryCrossEntropyWithLogits.cpp:22-73, kernels/elementwise/
// BinaryCrossEntropyWithLogitsKernel.cu:16-113); its backward is libtorch's formula, a chain of elementwise
// operators.  Here the forward is the same single kernel (operands broadcast by TensorIterator) and the backward
// is one kernel as well: the autograd node is ours, registered on AutogradPrivateUse1.
#include <ATen/core/Reduction.h>
#include <torch/csrc/autograd/custom_function.h>
#include <torch/library.h>

#include "aten/Common.h"

namespace supa {
namespace {

at::Tensor defined_or_empty(const c10::optional<at::Tensor>& t) { return (t.has_value() && t->defined()) ? *t : at::Tensor(); }

// loss (unreduced), contiguous, in the input's dtype
at::Tensor bce_logits_unreduced(const at::Tensor& self, const at::Tensor& target, const at::Tensor& weight, const at::Tensor& pos_weight) {
  at::Tensor loss = at::empty_like(self, at::MemoryFormat::Contiguous);
  at::TensorIteratorConfig config;
  config.add_output(loss).add_const_input(self).add_const_input(target);
  if (pos_weight.defined()) config.add_const_input(pos_weight);
  config.check_all_same_dtype(false).promote_inputs_to_common_dtype(true).cast_common_dtype_to_outputs(true).enforce_safe_casting_to_output(true);
  auto iter = config.build();
  if (iter.numel() > 0) launch_elementwise(iter, pos_weight.defined() ? SB_EW_BCE_LOGITS_PW : SB_EW_BCE_LOGITS, iter.common_dtype());
  if (weight.defined()) loss.mul_(weight);
  return loss;
}

// mean / sum in one pass: everything contiguous, of one dtype and of the input's shape; pos_weight along the last dimension
bool fused_reduce_applies(const at::Tensor& self, const at::Tensor& target, const at::Tensor& weight, const at::Tensor& pos_weight) {
  const at::ScalarType dt = self.scalar_type();
  if (self.numel() == 0 || !self.is_contiguous() || !target.is_contiguous() || target.scalar_type() != dt) return false;
  if (weight.defined() && (weight.scalar_type() != dt || !weight.is_contiguous() || weight.sizes() != self.sizes())) return false;
  if (pos_weight.defined()) {
    if (pos_weight.scalar_type() != dt || !pos_weight.is_contiguous() || pos_weight.dim() != 1 || self.dim() < 1 ||
        pos_weight.size(0) != self.size(-1))
      return false;
  }
  return true;
}

at::Tensor bce_logits_forward(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight_opt,
                              const c10::optional<at::Tensor>& pos_weight_opt, int64_t reduction) {
  TORCH_CHECK(self.sizes() == target.sizes(), "Target size (", target.sizes(), ") must be the same as input size (", self.sizes(), ")");
  TORCH_CHECK(at::isFloatingType(self.scalar_type()), "binary_cross_entropy_with_logits is only implemented for floating dtypes");
  const at::Tensor weight = defined_or_empty(weight_opt), pos_weight = defined_or_empty(pos_weight_opt);
  check_same_device("binary_cross_entropy_with_logits", {self, target, weight, pos_weight});
  const c10::DeviceGuard guard(self.device());
  if (reduction != at::Reduction::None && fused_reduce_applies(self, target, weight, pos_weight)) {
    at::Tensor out = at::empty({}, self.options());
    const size_t need = sb_bce_logits_scratch_bytes(self.numel());
    at::Tensor scratch = at::empty({static_cast<int64_t>(need)}, self.options().dtype(at::kByte));
    check_kernel(sb_bce_logits_reduce(self.const_data_ptr(), target.const_data_ptr(), pos_weight.defined() ? pos_weight.const_data_ptr() : nullptr,
                                      pos_weight.defined() ? pos_weight.numel() : 0, weight.defined() ? weight.const_data_ptr() : nullptr,
                                      dtype_code(self.scalar_type()), self.numel(),
                                      reduction == at::Reduction::Mean ? SB_REDUCTION_MEAN : SB_REDUCTION_SUM, out.data_ptr(),
                                      scratch.data_ptr(), need, stream_of(self)),
                 "supa binary_cross_entropy_with_logits");
    return out;
  }
  at::Tensor loss = bce_logits_unreduced(self, target, weight, pos_weight);
  if (reduction == at::Reduction::None) return loss;
  if (reduction == at::Reduction::Mean) return loss.mean();
  if (reduction == at::Reduction::Sum) return loss.sum();
  TORCH_CHECK(false, "invalid reduction enum: ", reduction);
}

// d loss / d x times the upstream gradient: (lw sigmoid(x) - pw t) * g * w [/ numel for mean]
at::Tensor bce_logits_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, const at::Tensor& weight,
                               const at::Tensor& pos_weight, int64_t reduction) {
  const c10::DeviceGuard guard(self.device());
  at::Tensor grad_input = at::empty_like(self, at::MemoryFormat::Contiguous);
  if (self.numel() == 0) return grad_input;
  const double alpha = reduction == at::Reduction::Mean ? 1.0 / static_cast<double>(self.numel()) : 1.0;
  at::Tensor g = grad;
  if (!is_supa(g)) g = g.to(self.device());
  if (g.scalar_type() != self.scalar_type()) g = g.to(self.scalar_type());
  at::TensorIteratorConfig config;
  config.add_output(grad_input).add_const_input(self).add_const_input(target).add_const_input(pos_weight.defined() ? pos_weight : g);
  config.check_all_same_dtype(false).promote_inputs_to_common_dtype(true).cast_common_dtype_to_outputs(true).resize_outputs(false);
  auto iter = config.build();
  launch_elementwise(iter, pos_weight.defined() ? SB_EW_BCE_LOGITS_PW_BWD : SB_EW_BCE_LOGITS_BWD, iter.common_dtype(), alpha);
  if (pos_weight.defined()) grad_input.mul_(g);
  if (weight.defined()) grad_input.mul_(weight);
  return grad_input;
}

class BceLogitsFunction : public torch::autograd::Function<BceLogitsFunction> {
 public:
  // optional inputs stay optionals: the autograd machinery records the layout and device of every Tensor argument
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& self, const at::Tensor& target,
                            const c10::optional<at::Tensor>& weight, const c10::optional<at::Tensor>& pos_weight, int64_t reduction) {
    at::AutoDispatchBelowADInplaceOrView below;
    ctx->save_for_backward({self, target, defined_or_empty(weight), defined_or_empty(pos_weight)});
    ctx->saved_data["reduction"] = reduction;
    return bce_logits_forward(self, target, weight, pos_weight, reduction);
  }
  static std::vector<at::Tensor> backward(torch::autograd::AutogradContext* ctx, std::vector<at::Tensor> grad_outputs) {
    const auto saved = ctx->get_saved_variables();
    at::Tensor grad_self;
    if (grad_outputs[0].defined())
      grad_self = bce_logits_backward(grad_outputs[0], saved[0], saved[1], saved[2], saved[3], ctx->saved_data["reduction"].toInt());
    return {grad_self, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

at::Tensor bce_logits_autograd(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                               const c10::optional<at::Tensor>& pos_weight, int64_t reduction) {
  TORCH_CHECK(!(at::GradMode::is_enabled() && target.requires_grad()),
              "binary_cross_entropy_with_logits on the supa device does not differentiate with respect to the target");
  if (at::GradMode::is_enabled() && self.requires_grad())
    return BceLogitsFunction::apply(self, target, (weight.has_value() && weight->defined()) ? weight : c10::nullopt,
                                    (pos_weight.has_value() && pos_weight->defined()) ? pos_weight : c10::nullopt, reduction);
  at::AutoDispatchBelowADInplaceOrView below;
  return bce_logits_forward(self, target, weight, pos_weight, reduction);
}

}  // namespace
}  // namespace supa

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) { m.impl("binary_cross_entropy_with_logits", TORCH_FN(supa::bce_logits_forward)); }
TORCH_LIBRARY_IMPL(aten, AutogradPrivateUse1, m) { m.impl("binary_cross_entropy_with_logits", TORCH_FN(supa::bce_logits_autograd)); }

// Helpers shared by the ATen operator wrappers of the supa backend.
#pragma once

#include <ATen/ATen.h>
#include <ATen/TensorIterator.h>
#include <c10/core/DeviceGuard.h>

#include "runtime/Runtime.h"
#include "supa_b200_kernels.h"

namespace supa {

inline int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kBool: return SB_BOOL;
    case at::kByte: return SB_U8;
    case at::kChar: return SB_I8;
    case at::kShort: return SB_I16;
    case at::kInt: return SB_I32;
    case at::kLong: return SB_I64;
    case at::kHalf: return SB_F16;
    case at::kBFloat16: return SB_BF16;
    case at::kFloat: return SB_F32;
    case at::kDouble: return SB_F64;
    default:
      TORCH_CHECK_NOT_IMPLEMENTED(false, "supa backend: dtype ", c10::toString(t), " is not supported by the kernel library");
  }
}

inline bool is_supa(const at::Tensor& t) { return t.defined() && t.device().type() == c10::DeviceType::PrivateUse1; }

// The calling thread's current stream on the tensor's device, as the handle the C ABI takes.
inline sb_stream_t stream_of(const at::Tensor& t) { return static_cast<sb_stream_t>(current_cuda_stream(t.device().index())); }

// All defined tensors must live on the same supa device (the common-device check of the reference's
// generated wrappers, script/codegen_supa/dest/register_dispatch_key.py:324-360).
inline void check_same_device(const char* op, std::initializer_list<std::reference_wrapper<const at::Tensor>> tensors) {
  c10::optional<c10::Device> dev;
  for (const at::Tensor& t : tensors) {
    if (!t.defined()) continue;
    TORCH_CHECK(is_supa(t), op, ": expected a supa tensor but got a tensor on ", t.device());
    if (!dev) dev = t.device();
    TORCH_CHECK(*dev == t.device(), op, ": expected all tensors on ", *dev, " but found one on ", t.device());
  }
}

// Elementwise launch from a TensorIterator whose operand 0 is the output.  `common` is the dtype the
// arithmetic is defined on.  CPU scalar operands must have been removed or lifted by the caller.
void launch_elementwise(at::TensorIteratorBase& iter, int op, at::ScalarType common, double alpha = 1.0, int64_t ialpha = 1,
                        double scalar = 0.0, int64_t iscalar = 0);
// dst = cast(src) for two supa tensors on one device, any strides, src broadcastable to dst.
void copy_device_to_device(const at::Tensor& dst, const at::Tensor& src);
// Reduction launch from a reduce TensorIterator (operand 0 output, operand 1 input).
void launch_reduce(at::TensorIterator& iter, int op);

}  // namespace supa

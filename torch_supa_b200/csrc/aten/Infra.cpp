// Tensor factories, copies and view plumbing of the supa backend.
//
// Counterparts in the reference: empty_supa / empty_strided_supa (torch_supa/csrc/aten/common/EmptyTensor.cpp:10-55),
// SUPANativeFunctions::empty (TensorFactories.cpp:18-34), copy_ (Copy.cpp:154-255: H2D / D2H with optional
// non_blocking, D2D memcpy or cast kernel, temporaries for non-contiguous transfers) and the view ops of
// supa_native_functions.yaml:5-54.
#include <ATen/EmptyTensor.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorIterator.h>
#include <ATen/ops/_copy_from_and_resize_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/view_native.h>
#include <ATen/ops/_reshape_alias_native.h>
#include <ATen/ops/unfold_native.h>
#include <torch/library.h>

#include "Common.h"

namespace supa {

namespace {

c10::Device resolve_device(c10::optional<c10::Device> device_opt) {
  c10::Device dev = device_opt.value_or(c10::Device(c10::DeviceType::PrivateUse1));
  TORCH_CHECK(dev.is_privateuseone(), "expected a supa device, got ", dev);
  if (!dev.has_index()) dev = c10::Device(c10::DeviceType::PrivateUse1, current_device());
  return dev;
}

at::Tensor empty_memory_format(c10::IntArrayRef size, c10::optional<at::ScalarType> dtype_opt,
                               c10::optional<at::Layout> layout_opt, c10::optional<c10::Device> device_opt,
                               c10::optional<bool> pin_memory_opt, c10::optional<at::MemoryFormat> memory_format_opt) {
  TORCH_CHECK(!pin_memory_opt.value_or(false), "Only dense CPU tensors can be pinned");
  TORCH_CHECK(layout_opt.value_or(at::kStrided) == at::kStrided, "supa tensors are strided");
  const c10::Device dev = resolve_device(device_opt);
  const c10::DeviceGuard guard(dev);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_generic(size, device_allocator(), ks, c10::dtype_or_default(dtype_opt), memory_format_opt);
}

at::Tensor empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride, c10::optional<at::ScalarType> dtype_opt,
                         c10::optional<at::Layout> layout_opt, c10::optional<c10::Device> device_opt,
                         c10::optional<bool> pin_memory_opt) {
  TORCH_CHECK(!pin_memory_opt.value_or(false), "Only dense CPU tensors can be pinned");
  TORCH_CHECK(layout_opt.value_or(at::kStrided) == at::kStrided, "supa tensors are strided");
  const c10::Device dev = resolve_device(device_opt);
  const c10::DeviceGuard guard(dev);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_strided_generic(size, stride, device_allocator(), ks, c10::dtype_or_default(dtype_opt));
}

// ---- copies ------------------------------------------------------------------------------------------------
bool same_dense_layout(const at::Tensor& a, const at::Tensor& b) {
  return a.sizes() == b.sizes() && a.strides() == b.strides() && a.is_non_overlapping_and_dense();
}

void copy_host_to_device(const at::Tensor& dst, const at::Tensor& src, bool non_blocking) {
  const c10::DeviceGuard guard(dst.device());
  cudaStream_t stream = current_cuda_stream(dst.device().index());
  at::Tensor host = src;
  if (host.dtype() != dst.dtype()) host = host.to(dst.scalar_type());
  if (host.sizes() != dst.sizes()) host = host.expand(dst.sizes());
  if (same_dense_layout(dst, host)) {
    const size_t nbytes = dst.numel() * dst.element_size();
    if (nbytes == 0) return;
    SUPA_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), host.const_data_ptr(), nbytes, cudaMemcpyHostToDevice, stream));
    // A pageable source has been staged by the driver when the call returns; a pinned one is read later,
    // so a blocking copy waits and a non-blocking one relies on the caller keeping the buffer alive.
    if (!non_blocking || !host.is_pinned()) SUPA_CUDA_CHECK(cudaStreamSynchronize(stream));
    else record_pinned_use(host.const_data_ptr(), stream);  // the block is not recycled while the copy reads it
    return;
  }
  // General layouts: contiguous host staging -> contiguous device temporary -> strided device copy.
  host = host.contiguous();
  at::Tensor staged = at::empty(dst.sizes(), dst.options());
  const size_t nbytes = staged.numel() * staged.element_size();
  if (nbytes) {
    SUPA_CUDA_CHECK(cudaMemcpyAsync(staged.data_ptr(), host.const_data_ptr(), nbytes, cudaMemcpyHostToDevice, stream));
    SUPA_CUDA_CHECK(cudaStreamSynchronize(stream));
    copy_device_to_device(dst, staged);
  }
}

void copy_device_to_host(const at::Tensor& dst, const at::Tensor& src, bool non_blocking) {
  const c10::DeviceGuard guard(src.device());
  cudaStream_t stream = current_cuda_stream(src.device().index());
  at::Tensor dev = src;
  if (dev.sizes() != dst.sizes()) dev = dev.expand(dst.sizes());
  if (dev.dtype() != dst.dtype() || !same_dense_layout(dst, dev)) {
    // cast / gather on the device into a contiguous temporary of the destination's dtype
    at::Tensor tmp = at::empty(dst.sizes(), dev.options().dtype(dst.scalar_type()));
    copy_device_to_device(tmp, dev);
    dev = tmp;
  }
  const size_t nbytes = dst.numel() * dst.element_size();
  if (same_dense_layout(dst, dev)) {
    if (nbytes) SUPA_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), dev.const_data_ptr(), nbytes, cudaMemcpyDeviceToHost, stream));
    if (!non_blocking || !dst.is_pinned()) check_status_word(src.device().index(), stream);  // synchronises the stream
    else record_pinned_use(dst.data_ptr(), stream);  // the block is not recycled while the copy writes it
    return;
  }
  at::Tensor host = at::empty(dst.sizes(), dst.options().memory_format(at::MemoryFormat::Contiguous));
  if (nbytes) SUPA_CUDA_CHECK(cudaMemcpyAsync(host.data_ptr(), dev.const_data_ptr(), nbytes, cudaMemcpyDeviceToHost, stream));
  check_status_word(src.device().index(), stream);
  dst.copy_(host);
}

void copy_across_devices(const at::Tensor& dst, const at::Tensor& src) {
  // contiguous temporaries on both sides, one peer copy between them
  at::Tensor s = src.dtype() == dst.dtype() ? src : src.to(dst.scalar_type());
  s = s.expand(dst.sizes()).contiguous();
  at::Tensor d;
  {
    const c10::DeviceGuard guard(dst.device());
    d = dst.is_contiguous() ? dst : at::empty(dst.sizes(), dst.options());
  }
  const size_t nbytes = d.numel() * d.element_size();
  if (nbytes) {
    // The copy runs on the source device's current stream.  Work queued on the destination's current stream that still
    // reads or writes `dst` must come first: an event recorded there holds the copy back.
    cudaStream_t dst_stream = current_cuda_stream(dst.device().index());
    cudaEvent_t before = nullptr;
    {
      const c10::DeviceGuard guard(dst.device());
      SUPA_CUDA_CHECK(cudaEventCreateWithFlags(&before, cudaEventDisableTiming));
      SUPA_CUDA_CHECK(cudaEventRecord(before, dst_stream));
    }
    const c10::DeviceGuard guard(src.device());
    cudaStream_t stream = current_cuda_stream(src.device().index());
    cudaError_t err = cudaStreamWaitEvent(stream, before, 0);
    if (err == cudaSuccess)
      err = cudaMemcpyPeerAsync(d.data_ptr(), dst.device().index(), s.const_data_ptr(), src.device().index(), nbytes, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);  // the destination's streams may use the data from here on
    cudaEventDestroy(before);
    SUPA_CUDA_CHECK(err);
  }
  if (!d.is_same(dst)) {
    const c10::DeviceGuard guard(dst.device());  // the strided copy-back is a kernel on the destination device
    copy_device_to_device(dst, d);
  }
}

// aten::_copy_from(self = source, dst, non_blocking): what Tensor.copy_ reaches for a backend outside the
// built-in list.  Returns dst.
at::Tensor copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  TORCH_CHECK(self.defined() && dst.defined(), "copy_: undefined tensor");
  TORCH_CHECK(!self.is_complex() && !dst.is_complex(), "supa backend: complex copies are not supported");
  if (dst.numel() == 0) return dst;
  if (is_supa(dst) && self.device().is_cpu()) {
    copy_host_to_device(dst, self, non_blocking);
  } else if (dst.device().is_cpu() && is_supa(self)) {
    copy_device_to_host(dst, self, non_blocking);
  } else if (is_supa(dst) && is_supa(self)) {
    if (dst.device() == self.device()) {
      const c10::DeviceGuard guard(dst.device());
      copy_device_to_device(dst, self);
    } else {
      copy_across_devices(dst, self);
    }
  } else {
    TORCH_CHECK(false, "copy_ between ", self.device(), " and ", dst.device(), " is not supported by the supa backend");
  }
  return dst;
}

at::Tensor copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  at::native::resize_output(dst, self.sizes());
  return copy_from(self, dst, false);
}

// ---- cat ---------------------------------------------------------------------------------------------------------
// Concatenation as narrow + copy per input (each copy is one launch of the elementwise engine or a memcpy).  Needed by
// callers that flatten tensors into one buffer, such as the parameter broadcast of DistributedDataParallel.
at::Tensor& cat_out(const at::ITensorListRef& tensors, int64_t dim, at::Tensor& out) {
  std::vector<at::Tensor> parts;
  for (const at::Tensor& t : tensors) {
    if (t.dim() == 1 && t.numel() == 0) continue;  // legacy: empty 1-D tensors are skipped whatever their shape
    parts.push_back(t);
  }
  TORCH_CHECK(!tensors.materialize().empty(), "torch.cat(): expected a non-empty list of Tensors");
  if (parts.empty()) {
    at::native::resize_output(out, {0});
    return out;
  }
  const int64_t d = at::maybe_wrap_dim(dim, parts[0].dim());
  std::vector<int64_t> shape = parts[0].sizes().vec();
  int64_t total = 0;
  for (const at::Tensor& t : parts) {
    TORCH_CHECK(is_supa(t) && t.device() == parts[0].device(), "torch.cat(): expected all tensors on ", parts[0].device());
    TORCH_CHECK(t.dim() == parts[0].dim(), "Tensors must have same number of dimensions: got ", parts[0].dim(), " and ", t.dim());
    for (int64_t i = 0; i < t.dim(); ++i)
      TORCH_CHECK(i == d || t.size(i) == shape[i], "Sizes of tensors must match except in dimension ", d, ". Expected size ", shape[i],
                  " but got size ", t.size(i), " in the list.");
    total += t.size(d);
  }
  shape[d] = total;
  const c10::DeviceGuard guard(parts[0].device());
  at::native::resize_output(out, shape);
  int64_t at_ = 0;
  for (const at::Tensor& t : parts) {
    if (t.size(d) == 0) continue;
    copy_device_to_device(out.narrow(d, at_, t.size(d)), t);
    at_ += t.size(d);
  }
  return out;
}
at::Tensor cat(const at::ITensorListRef& tensors, int64_t dim) {
  at::ScalarType dtype = at::kFloat;
  bool first = true;
  c10::optional<c10::Device> dev;
  for (const at::Tensor& t : tensors) {
    dtype = first ? t.scalar_type() : c10::promoteTypes(dtype, t.scalar_type());
    first = false;
    if (!dev && is_supa(t)) dev = t.device();
  }
  TORCH_CHECK(dev.has_value(), "torch.cat(): expected a non-empty list of supa Tensors");
  const c10::DeviceGuard guard(*dev);
  at::Tensor out = at::empty({0}, at::TensorOptions().dtype(dtype).device(*dev));
  return cat_out(tensors, dim, out);
}

// ---- resize / set ------------------------------------------------------------------------------------------
void grow_storage(const at::Tensor& self, size_t nbytes) {
  const c10::Storage& storage = self.storage();
  if (nbytes > storage.nbytes()) at::detail::getPrivateUse1Hooks().resizePrivateUse1Bytes(storage, nbytes);
}

const at::Tensor& resize_(const at::Tensor& self, c10::IntArrayRef size, c10::optional<at::MemoryFormat> memory_format) {
  TORCH_CHECK(!self.has_names(), "resize_ of named tensors is not supported on supa");
  c10::TensorImpl* impl = self.unsafeGetTensorImpl();
  if (impl->sizes() != size) {
    impl->set_sizes_contiguous(size);
    const size_t need = (static_cast<size_t>(impl->numel()) + impl->storage_offset()) * self.element_size();
    const c10::DeviceGuard guard(self.device());
    grow_storage(self, need);
  }
  if (memory_format.has_value() && *memory_format != at::MemoryFormat::Preserve) impl->empty_tensor_restride(*memory_format);
  return self;
}

at::Tensor& set_storage_offset(at::Tensor& result, at::Storage storage, int64_t storage_offset, c10::IntArrayRef size,
                               c10::IntArrayRef stride) {
  at::native::checkSetStorage(result, storage, storage_offset, size, stride);
  c10::TensorImpl* impl = result.unsafeGetTensorImpl();
  impl->set_storage_offset(storage_offset);
  if (stride.data()) impl->set_sizes_and_strides(size, stride);
  else impl->set_sizes_contiguous(size);
  // grow the storage if the view reaches past its end
  const size_t need = at::detail::computeStorageNbytes(impl->sizes(), impl->strides(), result.element_size(), storage_offset);
  const c10::DeviceGuard guard(result.device());
  grow_storage(result, need);
  return result;
}

at::Tensor& set_storage(at::Tensor& result, at::Storage source) {
  const int64_t numel = static_cast<int64_t>(source.nbytes() / result.element_size());
  return set_storage_offset(result, source, 0, {numel}, {});
}

at::Tensor& set_tensor(at::Tensor& result, const at::Tensor& source) {
  if (result.unsafeGetTensorImpl() != source.unsafeGetTensorImpl())
    return set_storage_offset(result, source.storage(), source.storage_offset(), source.sizes(), source.strides());
  return result;
}

// ---- fill / scalar -----------------------------------------------------------------------------------------
at::Tensor& fill_scalar(at::Tensor& self, const at::Scalar& value) {
  if (self.numel() == 0) return self;
  const c10::DeviceGuard guard(self.device());
  auto iter = at::TensorIteratorConfig()
                  .set_check_mem_overlap(false)  // fill is fine on internally overlapping (expanded) outputs
                  .check_all_same_dtype(false)
                  .add_output(self)
                  .resize_outputs(false)
                  .build();
  const at::ScalarType dt = self.scalar_type();
  double d = 0.0;
  int64_t i = 0;
  if (c10::isFloatingType(dt)) d = value.to<double>();
  else if (dt == at::kBool) i = value.to<bool>() ? 1 : 0;
  else i = value.to<int64_t>();
  launch_elementwise(iter, SB_EW_FILL, dt, 1.0, 1, d, i);
  return self;
}

at::Tensor& fill_tensor(at::Tensor& self, const at::Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "fill_ only supports 0-dimension value tensor but got tensor with ", value.dim(), " dimensions.");
  if (value.device().is_cpu()) return fill_scalar(self, value.item());
  if (self.numel() == 0) return self;
  const c10::DeviceGuard guard(self.device());
  copy_device_to_device(self, value);  // broadcast copy
  return self;
}

at::Tensor& zero_(at::Tensor& self) {
  if (self.numel() == 0) return self;
  if (self.is_non_overlapping_and_dense()) {
    const c10::DeviceGuard guard(self.device());
    SUPA_CUDA_CHECK(cudaMemsetAsync(self.data_ptr(), 0, self.numel() * self.element_size(), current_cuda_stream(self.device().index())));
    return self;
  }
  return fill_scalar(self, 0);
}

// Tensor.record_stream: the allocator must not reuse the memory before work queued on `s` has finished.
void record_stream_op(at::Tensor& self, c10::Stream s) { record_stream(self.storage().data_ptr(), s); }

at::Scalar local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  at::Tensor host = at::empty({}, self.options().device(at::kCPU));
  copy_device_to_host(host, self.reshape({}), false);
  return host.item();
}

}  // namespace

// dst = cast(src) on one device through the elementwise engine (COPY), or a plain memcpy when the layouts
// and dtypes agree.
void copy_device_to_device(const at::Tensor& dst, const at::Tensor& src) {
  if (dst.numel() == 0) return;
  cudaStream_t stream = current_cuda_stream(dst.device().index());
  if (dst.dtype() == src.dtype() && same_dense_layout(dst, src)) {
    if (dst.data_ptr() == src.const_data_ptr()) return;
    SUPA_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), src.const_data_ptr(), dst.numel() * dst.element_size(),
                                    cudaMemcpyDeviceToDevice, stream));
    return;
  }
  auto iter = at::TensorIteratorConfig()
                  .add_output(dst)
                  .add_const_input(src)
                  .resize_outputs(false)
                  .check_all_same_dtype(false)
                  .check_all_same_device(true)
                  .build();
  launch_elementwise(iter, SB_EW_COPY, src.scalar_type());
}

}  // namespace supa

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", TORCH_FN(supa::empty_memory_format));
  m.impl("empty_strided", TORCH_FN(supa::empty_strided));
  m.impl("_copy_from", TORCH_FN(supa::copy_from));
  m.impl("_copy_from_and_resize", TORCH_FN(supa::copy_from_and_resize));
  m.impl("as_strided", TORCH_FN(at::native::as_strided_tensorimpl));
  m.impl("view", TORCH_FN(at::native::view));
  m.impl("_reshape_alias", TORCH_FN(at::native::_reshape_alias));
  m.impl("unfold", TORCH_FN(at::native::unfold));
  m.impl("resize_", TORCH_FN(supa::resize_));
  m.impl("set_.source_Storage_storage_offset", TORCH_FN(supa::set_storage_offset));
  m.impl("set_.source_Storage", TORCH_FN(supa::set_storage));
  m.impl("set_.source_Tensor", TORCH_FN(supa::set_tensor));
  m.impl("fill_.Scalar", TORCH_FN(supa::fill_scalar));
  m.impl("fill_.Tensor", TORCH_FN(supa::fill_tensor));
  m.impl("zero_", TORCH_FN(supa::zero_));
  m.impl("_local_scalar_dense", TORCH_FN(supa::local_scalar_dense));
  m.impl("record_stream", TORCH_FN(supa::record_stream_op));
  m.impl("cat", TORCH_FN(supa::cat));
  m.impl("cat.out", TORCH_FN(supa::cat_out));
}

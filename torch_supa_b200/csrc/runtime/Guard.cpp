// DeviceGuardImplInterface, allocator and hooks registration for the PrivateUse1 ("supa") device.
//
// Counterpart of SUPAGuardImpl (torch_supa/csrc/core/supa/impl/SUPAGuardImpl.h:15-59, .cpp:254-265) and of
// REGISTER_ALLOCATOR(PrivateUse1, ...) (SUPACachingAllocator.cpp:3556): the dispatcher, the autograd engine
// (which switches device and stream through this interface on its worker threads) and torch.Stream /
// torch.Event all reach the CUDA runtime through here.
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/core/impl/alloc_cpu.h>

#include "Generator.h"
#include "Runtime.h"

namespace supa {

namespace {

struct SupaGuardImpl final : public c10::impl::DeviceGuardImplInterface {
  static constexpr c10::DeviceType static_type = c10::DeviceType::PrivateUse1;

  SupaGuardImpl() = default;
  explicit SupaGuardImpl(c10::DeviceType t) { TORCH_INTERNAL_ASSERT(t == c10::DeviceType::PrivateUse1); }

  c10::DeviceType type() const override { return c10::DeviceType::PrivateUse1; }

  c10::Device exchangeDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.is_privateuseone());
    return c10::Device(c10::DeviceType::PrivateUse1, exchange_device(d.index()));
  }
  c10::Device getDevice() const override { return c10::Device(c10::DeviceType::PrivateUse1, current_device()); }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.is_privateuseone());
    set_device(d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    if (cudaSetDevice(d.index()) != cudaSuccess) cudaGetLastError();
  }

  c10::Stream getStream(c10::Device d) const override { return current_stream(d.index()); }
  c10::Stream getDefaultStream(c10::Device d) const override { return default_stream(d.index()); }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool high = false) const override {
    return stream_from_pool(d.index(), high);
  }
  c10::Stream getNewStream(c10::Device d, int priority = 0) const override { return stream_from_pool(d.index(), priority < 0); }
  c10::Stream exchangeStream(c10::Stream s) const override { return exchange_current_stream(s); }
  void* getStreamNativeHandle(const c10::Stream s) const override { return cuda_stream(s); }

  c10::DeviceIndex deviceCount() const noexcept override { return device_count(); }

  // ---- events ----
  void destroyEvent(void* event, const c10::DeviceIndex device_index) const noexcept override {
    if (!event) return;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != device_index) cudaSetDevice(device_index);
    cudaEventDestroy(static_cast<cudaEvent_t>(event));
    if (prev != device_index && prev >= 0) cudaSetDevice(prev);
    cudaGetLastError();
  }

  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag flag) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ",
                static_cast<int>(device_index), " does not match recording stream's device index ",
                static_cast<int>(stream.device_index()), ".");
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    cudaEvent_t ev = static_cast<cudaEvent_t>(*event);
    if (!ev) {
      unsigned int flags = cudaEventDefault;
      switch (flag) {
        case c10::EventFlag::PYTORCH_DEFAULT: flags = cudaEventDisableTiming; break;
        case c10::EventFlag::BACKEND_DEFAULT: flags = cudaEventDefault; break;
        default: TORCH_CHECK(false, "supa event received unknown flag");
      }
      SUPA_CUDA_CHECK(cudaEventCreateWithFlags(&ev, flags));
    }
    SUPA_CUDA_CHECK(cudaEventRecord(ev, cuda_stream(stream)));
    *event = ev;
    if (prev != stream.device_index()) set_device(prev);
  }

  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    SUPA_CUDA_CHECK(cudaStreamWaitEvent(cuda_stream(stream), static_cast<cudaEvent_t>(event), 0));
    if (prev != stream.device_index()) set_device(prev);
  }

  bool queryEvent(void* event) const override {
    if (!event) return true;
    const cudaError_t err = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (err == cudaErrorNotReady) {
      cudaGetLastError();
      return false;
    }
    SUPA_CUDA_CHECK(err);
    return true;
  }

  void synchronizeEvent(void* event) const override {
    if (!event) return;
    SUPA_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  }

  double elapsedTime(void* event1, void* event2, const c10::DeviceIndex device_index) const override {
    TORCH_CHECK(event1 && event2, "Both events must be recorded before calculating elapsed time.");
    const c10::DeviceIndex prev = exchange_device(device_index);
    float ms = 0.f;
    const cudaError_t err = cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(event1), static_cast<cudaEvent_t>(event2));
    if (prev != device_index) set_device(prev);
    SUPA_CUDA_CHECK(err);
    return static_cast<double>(ms);
  }

  // ---- streams ----
  bool queryStream(const c10::Stream& stream) const override {
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    const cudaError_t err = cudaStreamQuery(cuda_stream(stream));
    if (prev != stream.device_index()) set_device(prev);
    if (err == cudaErrorNotReady) {
      cudaGetLastError();
      return false;
    }
    SUPA_CUDA_CHECK(err);
    return true;
  }

  void synchronizeStream(const c10::Stream& stream) const override {
    const c10::DeviceIndex prev = exchange_device(stream.device_index());
    const cudaError_t err = cudaStreamSynchronize(cuda_stream(stream));
    if (prev != stream.device_index()) set_device(prev);
    SUPA_CUDA_CHECK(err);
    check_status_word(stream.device_index(), cuda_stream(stream));
  }

  void synchronizeDevice(const c10::DeviceIndex device_index) const override { synchronize_device(device_index); }

  void recordDataPtrOnStream(const c10::DataPtr& data_ptr, const c10::Stream& stream) const override {
    record_stream(data_ptr, stream);
  }
};

struct SupaHooks final : public at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return device_count() > 0; }
  bool hasPrimaryContext(c10::DeviceIndex device_index) const override {
    unsigned int flags = 0;
    int active = 0;
    if (cuDevicePrimaryCtxGetStateCompat(device_index, &flags, &active)) return active != 0;
    return true;
  }
  c10::DeviceIndex deviceCount() const override { return device_count(); }
  void setCurrentDevice(c10::DeviceIndex device) const override { set_device(device); }
  c10::DeviceIndex getCurrentDevice() const override { return current_device(); }
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex device) const override { return exchange_device(device); }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex device) const override { return exchange_device(device); }
  bool isPinnedPtr(const void* data) const override {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, data) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    return attr.type == cudaMemoryTypeHost;
  }
  c10::Allocator* getPinnedMemoryAllocator() const override { return pinned_allocator(); }
  const at::Generator& getDefaultGenerator(c10::DeviceIndex device_index) const override { return default_generator(device_index); }
  at::Generator getNewGenerator(c10::DeviceIndex device_index = -1) const override { return new_generator(device_index); }
  at::Device getDeviceFromPtr(void* data) const override {
    cudaPointerAttributes attr{};
    SUPA_CUDA_CHECK(cudaPointerGetAttributes(&attr, data));
    TORCH_CHECK(attr.type == cudaMemoryTypeDevice, "The specified pointer resides on host memory and is not registered with any supa device.");
    return at::Device(c10::DeviceType::PrivateUse1, static_cast<c10::DeviceIndex>(attr.device));
  }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t new_bytes) const override {
    // Grow (or shrink) a storage, keeping the old contents, on the current stream.
    c10::StorageImpl* impl = storage.unsafeGetStorageImpl();
    TORCH_CHECK(impl->resizable(), "Trying to resize storage that is not resizable");
    const c10::DeviceIndex prev = exchange_device(storage.device().index());
    c10::DataPtr fresh = new_bytes ? device_allocator()->allocate(new_bytes) : c10::DataPtr(nullptr, storage.device());
    const size_t keep = std::min(new_bytes, impl->nbytes());
    if (keep && impl->data()) {
      SUPA_CUDA_CHECK(cudaMemcpyAsync(fresh.get(), impl->data(), keep, cudaMemcpyDeviceToDevice, current_cuda_stream()));
    }
    impl->set_data_ptr_noswap(std::move(fresh));
    impl->set_nbytes(new_bytes);
    if (prev != storage.device().index()) set_device(prev);
  }

 private:
  // cuDevicePrimaryCtxGetState lives in the driver library; the runtime offers no equivalent, so report
  // "active" once this process has created a context through the runtime (any earlier cudaSetDevice).
  static bool cuDevicePrimaryCtxGetStateCompat(c10::DeviceIndex, unsigned int*, int*) { return false; }
};

}  // namespace

}  // namespace supa

// ---- static registration ------------------------------------------------------------------------------------
namespace c10::impl {
C10_REGISTER_GUARD_IMPL(PrivateUse1, supa::SupaGuardImpl);
}

namespace {
struct RegisterBackend {
  RegisterBackend() {
    c10::register_privateuse1_backend("supa");
    c10::SetAllocator(c10::DeviceType::PrivateUse1, supa::device_allocator());
    at::RegisterPrivateUse1HooksInterface(new supa::SupaHooks());
  }
} g_register_backend;
}  // namespace

// Device selection, stream pool and the per-device status word.
#include <array>
#include <atomic>
#include <mutex>
#include <sstream>

#include "Runtime.h"
#include "supa_b200_kernels.h"

namespace supa {

namespace {
constexpr int kMaxDevices = 16;
}

void check_cuda(cudaError_t err, const char* what, const char* file, int line) {
  if (err == cudaSuccess) return;
  cudaGetLastError();  // clear the sticky-less error state so that later calls report their own errors
  std::ostringstream os;
  os << "CUDA error: " << cudaGetErrorString(err) << " (" << cudaGetErrorName(err) << ") in `" << what << "` at " << file
     << ":" << line;
  TORCH_CHECK(false, os.str());
}

void check_kernel(int status, const char* what) {
  if (status == SB_OK) return;
  if (status == SB_ERR_UNSUPPORTED) {
    TORCH_CHECK_NOT_IMPLEMENTED(false, what, ": ", sb_status_string(status), " (the supa backend has no CPU fallback)");
  }
  TORCH_CHECK(false, what, " failed: ", sb_status_string(status));
}

// ---- devices -------------------------------------------------------------------------------------------------
c10::DeviceIndex device_count() noexcept {
  static const int count = [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    return n > kMaxDevices ? kMaxDevices : n;
  }();
  return static_cast<c10::DeviceIndex>(count);
}

c10::DeviceIndex current_device() {
  int dev = 0;
  SUPA_CUDA_CHECK(cudaGetDevice(&dev));
  return static_cast<c10::DeviceIndex>(dev);
}

void set_device(c10::DeviceIndex device) {
  TORCH_CHECK(device >= 0 && device < device_count(), "invalid supa device index ", static_cast<int>(device), " (",
              static_cast<int>(device_count()), " device(s) present)");
  int cur = -1;
  SUPA_CUDA_CHECK(cudaGetDevice(&cur));
  if (cur != device) SUPA_CUDA_CHECK(cudaSetDevice(device));
}

c10::DeviceIndex exchange_device(c10::DeviceIndex device) {
  const c10::DeviceIndex prev = current_device();
  if (device >= 0 && device != prev) set_device(device);
  return prev;
}

void synchronize_device(c10::DeviceIndex device) {
  const c10::DeviceIndex prev = exchange_device(device);
  const cudaError_t err = cudaDeviceSynchronize();
  if (prev != device) cudaSetDevice(prev);
  SUPA_CUDA_CHECK(err);
  check_status_word(device, nullptr);
}

// ---- streams -------------------------------------------------------------------------------------------------
namespace {

struct DeviceStreams {
  std::once_flag once;
  std::array<cudaStream_t, 2 * kStreamsPerPool> pool{};
  std::atomic<uint32_t> next_normal{0};
  std::atomic<uint32_t> next_high{0};
};

DeviceStreams g_streams[kMaxDevices];
thread_local c10::StreamId tl_current[kMaxDevices] = {};  // 0 = default stream

void check_device_index(c10::DeviceIndex device) {
  TORCH_CHECK(device >= 0 && device < device_count(), "invalid supa device index ", static_cast<int>(device));
}

void init_pool(c10::DeviceIndex device) {
  std::call_once(g_streams[device].once, [device] {
    const c10::DeviceIndex prev = exchange_device(device);
    int least = 0, greatest = 0;
    SUPA_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    for (int i = 0; i < kStreamsPerPool; ++i) {
      SUPA_CUDA_CHECK(cudaStreamCreateWithPriority(&g_streams[device].pool[i], cudaStreamNonBlocking, least));
      SUPA_CUDA_CHECK(
          cudaStreamCreateWithPriority(&g_streams[device].pool[kStreamsPerPool + i], cudaStreamNonBlocking, greatest));
    }
    if (prev != device) cudaSetDevice(prev);
  });
}

c10::Stream make_stream(c10::DeviceIndex device, c10::StreamId id) {
  return c10::Stream(c10::Stream::UNSAFE, c10::Device(c10::DeviceType::PrivateUse1, device), id);
}

}  // namespace

c10::Stream default_stream(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  check_device_index(device);
  return make_stream(device, 0);
}

c10::Stream current_stream(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  check_device_index(device);
  return make_stream(device, tl_current[device]);
}

c10::Stream stream_from_pool(c10::DeviceIndex device, bool high_priority) {
  if (device < 0) device = current_device();
  check_device_index(device);
  init_pool(device);
  auto& ds = g_streams[device];
  const uint32_t slot = (high_priority ? ds.next_high : ds.next_normal).fetch_add(1) % kStreamsPerPool;
  return make_stream(device, 1 + (high_priority ? kStreamsPerPool : 0) + slot);
}

c10::Stream exchange_current_stream(c10::Stream stream) {
  TORCH_CHECK(stream.device_type() == c10::DeviceType::PrivateUse1, "expected a supa stream");
  const c10::DeviceIndex device = stream.device_index();
  check_device_index(device);
  TORCH_CHECK(stream.id() >= 0 && stream.id() <= 2 * kStreamsPerPool, "invalid supa stream id ", stream.id());
  const c10::Stream prev = make_stream(device, tl_current[device]);
  tl_current[device] = stream.id();
  return prev;
}

cudaStream_t cuda_stream(c10::Stream stream) {
  TORCH_CHECK(stream.device_type() == c10::DeviceType::PrivateUse1, "expected a supa stream");
  const c10::StreamId id = stream.id();
  if (id == 0) return nullptr;
  const c10::DeviceIndex device = stream.device_index();
  check_device_index(device);
  TORCH_CHECK(id > 0 && id <= 2 * kStreamsPerPool, "invalid supa stream id ", id);
  init_pool(device);
  return g_streams[device].pool[id - 1];
}

cudaStream_t current_cuda_stream(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  return cuda_stream(current_stream(device));
}

// ---- status word ---------------------------------------------------------------------------------------------
namespace {
struct StatusWord {
  std::once_flag once;
  int32_t* device_ptr = nullptr;
  int32_t* host_pinned = nullptr;
};
StatusWord g_status[kMaxDevices];
}  // namespace

int32_t* status_word(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  check_device_index(device);
  std::call_once(g_status[device].once, [device] {
    const c10::DeviceIndex prev = exchange_device(device);
    SUPA_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&g_status[device].device_ptr), sizeof(int32_t)));
    SUPA_CUDA_CHECK(cudaMemset(g_status[device].device_ptr, 0, sizeof(int32_t)));
    SUPA_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&g_status[device].host_pinned), sizeof(int32_t), cudaHostAllocDefault));
    *g_status[device].host_pinned = 0;
    if (prev != device) cudaSetDevice(prev);
  });
  return g_status[device].device_ptr;
}

void check_status_word(c10::DeviceIndex device, cudaStream_t stream) {
  if (device < 0) device = current_device();
  if (g_status[device].device_ptr == nullptr) return;  // no kernel that can report has run on this device
  const c10::DeviceIndex prev = exchange_device(device);
  cudaError_t err = cudaMemcpyAsync(g_status[device].host_pinned, g_status[device].device_ptr, sizeof(int32_t),
                                    cudaMemcpyDeviceToHost, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  int32_t word = 0;
  if (err == cudaSuccess) {
    word = *g_status[device].host_pinned;
    if (word != 0) err = cudaMemsetAsync(g_status[device].device_ptr, 0, sizeof(int32_t), stream);
  }
  if (prev != device) cudaSetDevice(prev);
  SUPA_CUDA_CHECK(err);
  if (word & SB_STATUS_KERNEL_TIMEOUT)
    TORCH_CHECK(false, "a supa kernel gave up on a bounded wait; its results are invalid");
  if (word & SB_STATUS_GRADIENT_LOST)
    TORCH_CHECK(false, "cross_entropy: backward through a retained graph after a backward with a zero upstream gradient, which wiped "
                       "the stored gradient; run the forward again");
  if (word & SB_STATUS_TARGET_OUT_OF_RANGE) TORCH_CHECK_INDEX(false, "Target is out of bounds.");
}

}  // namespace supa

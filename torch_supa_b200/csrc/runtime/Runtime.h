// Core runtime of the "supa" (PrivateUse1) device on CUDA: device selection, stream pool, stream-ordered
// allocator, status word.  It plays the role of the reference's c10::supa layer
// (torch_supa/csrc/core/supa/SUPAFunctions.cpp:209-290, SUPAStream.cpp:26-342,
// SUPACachingAllocator.h:276-408) on top of the CUDA runtime; nothing here depends on libtorch_cuda.
#pragma once

#include <c10/core/Allocator.h>
#include <c10/core/Device.h>
#include <c10/core/Stream.h>
#include <c10/util/Exception.h>
#include <cuda_runtime.h>

#include <cstdint>

#define SUPA_EXPORT __attribute__((visibility("default")))

namespace supa {

// Throws c10::Error with the CUDA error text.
void check_cuda(cudaError_t err, const char* what, const char* file, int line);
#define SUPA_CUDA_CHECK(expr) ::supa::check_cuda((expr), #expr, __FILE__, __LINE__)

// Throws when a kernel-library launcher returned a negative status.
void check_kernel(int status, const char* what);

// ---- devices -----------------------------------------------------------------------------------------------
// Number of CUDA devices; 0 when the driver is absent (never throws).
c10::DeviceIndex device_count() noexcept;
// Current device of the calling thread.
c10::DeviceIndex current_device();
void set_device(c10::DeviceIndex device);
c10::DeviceIndex exchange_device(c10::DeviceIndex device);
void synchronize_device(c10::DeviceIndex device);

// ---- streams -----------------------------------------------------------------------------------------------
// Stream ids: 0 is the legacy default stream (handle 0), 1..kStreamsPerPool the normal-priority pool,
// kStreamsPerPool+1..2*kStreamsPerPool the high-priority pool.  Pool streams are non-blocking and created
// lazily per device; the current stream is thread-local per device.
constexpr int kStreamsPerPool = 32;

c10::Stream default_stream(c10::DeviceIndex device);
c10::Stream current_stream(c10::DeviceIndex device);
c10::Stream stream_from_pool(c10::DeviceIndex device, bool high_priority);
// Sets the thread-local current stream of the stream's device; returns the previous one.
c10::Stream exchange_current_stream(c10::Stream stream);
cudaStream_t cuda_stream(c10::Stream stream);
// The calling thread's current CUDA stream on `device` (-1: current device).
cudaStream_t current_cuda_stream(c10::DeviceIndex device = -1);

// ---- allocator --------------------------------------------------------------------------------------------
struct MemoryStats {
  int64_t allocated_bytes;       // live bytes handed out
  int64_t peak_allocated_bytes;
  int64_t reserved_bytes;        // bytes the pool holds from the driver
  int64_t num_allocs;
  int64_t num_frees;
  int64_t num_ooms;
};

c10::Allocator* device_allocator();
MemoryStats memory_stats(c10::DeviceIndex device);
void reset_peak_memory_stats(c10::DeviceIndex device);
// Returns cached memory to the driver.
void empty_cache();
// Caps live bytes per device (0 = no cap); allocations beyond the cap raise OutOfMemoryError without
// touching the GPU.  Used to exercise the out-of-memory path on the host.
void set_memory_limit(c10::DeviceIndex device, int64_t bytes);
// Marks `ptr` (an allocation of this allocator) as used on `stream`: its memory is not reused before the
// work queued on that stream so far has finished.
void record_stream(const c10::DataPtr& ptr, c10::Stream stream);

// ---- pinned host memory -------------------------------------------------------------------------------------
struct HostMemoryStats {
  int64_t allocated_bytes;  // bytes in blocks handed out
  int64_t reserved_bytes;   // bytes obtained from cudaHostAlloc and not given back
  int64_t host_allocs;      // cudaHostAlloc calls
  int64_t hits;             // allocations served from the cache
};
// Caching allocator of page-locked host memory (tensor.pin_memory(), non-blocking copies).
c10::Allocator* pinned_allocator();
// Marks the pinned block that holds `ptr` as used by asynchronous work on `stream`: after it is freed it is not handed
// out again before that work has finished.  False when `ptr` is not in a block of this allocator.
bool record_pinned_use(const void* ptr, cudaStream_t stream);
bool is_cached_pinned(const void* ptr);
// Returns cached pinned blocks to the driver.
void empty_pinned_cache();
HostMemoryStats host_memory_stats();

// ---- status word ------------------------------------------------------------------------------------------
// One int32 per device in device memory that kernels OR error bits into (an out-of-range class index).
int32_t* status_word(c10::DeviceIndex device);
// Reads the word after the given stream has drained and throws c10::IndexError if an error bit is set
// (the word is cleared first).  Called at the host's natural synchronisation points.
void check_status_word(c10::DeviceIndex device, cudaStream_t stream);

}  // namespace supa

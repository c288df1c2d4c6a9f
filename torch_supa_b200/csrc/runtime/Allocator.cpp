// Stream-ordered device allocator: c10::Allocator on cudaMallocAsync with one explicit memory pool per
// device.
//
// The reference caches blocks itself, keyed by stream, and defers frees of blocks used on other streams
// with events (torch_supa/csrc/core/supa/SUPACachingAllocator.cpp:959-1107, 1332, 2843-2930).  Here the
// CUDA memory pool does the caching (release threshold = unlimited, so freed memory stays in the pool like
// in the reference) and stream ordering does the rest: an allocation belongs to the stream it was made
// on; a free is queued on that stream after it has been made to wait for every other stream the block was
// used on (record_stream), so no host-side deferred-free list is needed.
//
// Two pools per device, as the reference keeps a small-block and a large-block pool (kSmallSize = 1 MiB,
// torch_supa/csrc/core/supa/SUPAAllocatorConfig.h:18-23): requests up to 1 MiB come from their own pool.  With one pool
// the few-hundred-byte scratch tensors of an operator were carved out of a freed half-gigabyte block, the next large
// request no longer fitted there, and the driver re-stitched physical memory for it: 2.7 ms per allocation measured on
// B200, against microseconds when the large blocks are only ever reused whole.
#include <atomic>
#include <mutex>
#include <vector>

#include "Runtime.h"

namespace supa {

namespace {

constexpr int kMaxDevices = 16;
constexpr size_t kRoundTo = 512;  // allocation granularity, as the reference's kMinBlockSize
constexpr size_t kSmallSize = 1 << 20;  // requests up to this size come from the small pool

struct DevicePool {
  std::once_flag once;
  cudaMemPool_t pool = nullptr;        // large requests
  cudaMemPool_t small_pool = nullptr;  // requests of at most kSmallSize bytes
  std::atomic<int64_t> allocated{0};
  std::atomic<int64_t> peak{0};
  std::atomic<int64_t> num_allocs{0};
  std::atomic<int64_t> num_frees{0};
  std::atomic<int64_t> num_ooms{0};
  std::atomic<int64_t> limit{0};
};

DevicePool g_pools[kMaxDevices];

struct Block {
  void* ptr;
  size_t size;
  c10::DeviceIndex device;
  cudaStream_t alloc_stream;
  std::mutex mu;
  std::vector<cudaStream_t> other_streams;  // streams recorded with record_stream
};

void init_pool(c10::DeviceIndex device) {
  std::call_once(g_pools[device].once, [device] {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    SUPA_CUDA_CHECK(cudaMemPoolCreate(&g_pools[device].pool, &props));
    SUPA_CUDA_CHECK(cudaMemPoolCreate(&g_pools[device].small_pool, &props));
    uint64_t threshold = UINT64_MAX;  // keep freed memory cached in the pools
    SUPA_CUDA_CHECK(cudaMemPoolSetAttribute(g_pools[device].pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    SUPA_CUDA_CHECK(cudaMemPoolSetAttribute(g_pools[device].small_pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    if (const char* env = std::getenv("TORCH_SUPA_B200_MEMORY_LIMIT_BYTES")) g_pools[device].limit = std::atoll(env);
  });
}

void update_peak(DevicePool& dp, int64_t now) {
  int64_t peak = dp.peak.load(std::memory_order_relaxed);
  while (now > peak && !dp.peak.compare_exchange_weak(peak, now, std::memory_order_relaxed)) {
  }
}

void free_block(void* ctx) {
  Block* b = static_cast<Block*>(ctx);
  if (!b) return;
  DevicePool& dp = g_pools[b->device];
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != b->device) cudaSetDevice(b->device);
  // Make the owning stream wait for the work queued so far on every other stream that used the block,
  // then free in stream order.
  for (cudaStream_t other : b->other_streams) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
      cudaEventRecord(ev, other);
      cudaStreamWaitEvent(b->alloc_stream, ev, 0);
      cudaEventDestroy(ev);  // released by the driver once the wait has been satisfied
    }
  }
  cudaFreeAsync(b->ptr, b->alloc_stream);
  cudaGetLastError();  // a deleter must not throw (it may run during interpreter shutdown)
  if (prev != b->device && prev >= 0) cudaSetDevice(prev);
  dp.allocated.fetch_sub(static_cast<int64_t>(b->size), std::memory_order_relaxed);
  dp.num_frees.fetch_add(1, std::memory_order_relaxed);
  delete b;
}

class SupaAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t nbytes) override {
    const c10::DeviceIndex device = current_device();
    const c10::Device dev(c10::DeviceType::PrivateUse1, device);
    if (nbytes == 0) return c10::DataPtr(nullptr, nullptr, &free_block, dev);
    init_pool(device);
    DevicePool& dp = g_pools[device];
    const size_t size = (nbytes + kRoundTo - 1) / kRoundTo * kRoundTo;
    const int64_t limit = dp.limit.load(std::memory_order_relaxed);
    if (limit > 0 && dp.allocated.load(std::memory_order_relaxed) + static_cast<int64_t>(size) > limit) {
      dp.num_ooms.fetch_add(1, std::memory_order_relaxed);
      TORCH_CHECK_WITH(OutOfMemoryError, false, "supa out of memory: tried to allocate ", size, " bytes with ",
                       dp.allocated.load(), " bytes allocated and a limit of ", limit, " bytes on device ",
                       static_cast<int>(device));
    }
    cudaStream_t stream = current_cuda_stream(device);
    void* ptr = nullptr;
    cudaMemPool_t pool = size <= kSmallSize ? dp.small_pool : dp.pool;
    cudaError_t err = cudaMallocFromPoolAsync(&ptr, size, pool, stream);
    if (err == cudaErrorMemoryAllocation) {
      // Give cached memory back to the driver and try once more, as the reference does before reporting OOM.
      cudaGetLastError();
      cudaDeviceSynchronize();
      cudaMemPoolTrimTo(dp.pool, 0);
      cudaMemPoolTrimTo(dp.small_pool, 0);
      err = cudaMallocFromPoolAsync(&ptr, size, pool, stream);
    }
    if (err == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      dp.num_ooms.fetch_add(1, std::memory_order_relaxed);
      size_t free_b = 0, total_b = 0;
      cudaMemGetInfo(&free_b, &total_b);
      TORCH_CHECK_WITH(OutOfMemoryError, false, "supa out of memory: tried to allocate ", size, " bytes; device ",
                       static_cast<int>(device), " has ", free_b, " of ", total_b, " bytes free, ", dp.allocated.load(),
                       " bytes are allocated by tensors");
    }
    SUPA_CUDA_CHECK(err);
    Block* b = new Block{ptr, size, device, stream, {}, {}};
    const int64_t now = dp.allocated.fetch_add(static_cast<int64_t>(size), std::memory_order_relaxed) + static_cast<int64_t>(size);
    update_peak(dp, now);
    dp.num_allocs.fetch_add(1, std::memory_order_relaxed);
    return c10::DataPtr(ptr, b, &free_block, dev);
  }

  c10::DeleterFnPtr raw_deleter() const override { return nullptr; }  // contexts are Blocks, not raw pointers

  void copy_data(void* dest, const void* src, std::size_t count) const override {
    SUPA_CUDA_CHECK(cudaMemcpyAsync(dest, src, count, cudaMemcpyDeviceToDevice, current_cuda_stream()));
  }
};

SupaAllocator g_allocator;

}  // namespace

c10::Allocator* device_allocator() { return &g_allocator; }

MemoryStats memory_stats(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  TORCH_CHECK(device < device_count(), "invalid supa device index");
  DevicePool& dp = g_pools[device];
  MemoryStats s{};
  s.allocated_bytes = dp.allocated.load();
  s.peak_allocated_bytes = dp.peak.load();
  s.num_allocs = dp.num_allocs.load();
  s.num_frees = dp.num_frees.load();
  s.num_ooms = dp.num_ooms.load();
  s.reserved_bytes = 0;
  for (cudaMemPool_t pool : {dp.pool, dp.small_pool}) {
    if (!pool) continue;
    uint64_t reserved = 0;
    if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved) == cudaSuccess)
      s.reserved_bytes += static_cast<int64_t>(reserved);
    else
      cudaGetLastError();
  }
  return s;
}

void reset_peak_memory_stats(c10::DeviceIndex device) {
  if (device < 0) device = current_device();
  g_pools[device].peak = g_pools[device].allocated.load();
}

void empty_cache() {
  for (c10::DeviceIndex d = 0; d < device_count(); ++d) {
    if (!g_pools[d].pool) continue;
    const c10::DeviceIndex prev = exchange_device(d);
    cudaDeviceSynchronize();
    cudaMemPoolTrimTo(g_pools[d].pool, 0);
    cudaMemPoolTrimTo(g_pools[d].small_pool, 0);
    cudaGetLastError();
    if (prev != d) cudaSetDevice(prev);
  }
}

void set_memory_limit(c10::DeviceIndex device, int64_t bytes) {
  if (device < 0) device = current_device();
  TORCH_CHECK(device < device_count(), "invalid supa device index");
  g_pools[device].limit = bytes;
}

void record_stream(const c10::DataPtr& ptr, c10::Stream stream) {
  if (!ptr.get() || ptr.get_deleter() != &free_block) return;  // not ours, or empty
  Block* b = static_cast<Block*>(ptr.get_context());
  if (!b) return;
  cudaStream_t s = cuda_stream(stream);
  if (s == b->alloc_stream) return;
  std::lock_guard<std::mutex> lock(b->mu);
  for (cudaStream_t o : b->other_streams)
    if (o == s) return;
  b->other_streams.push_back(s);
}

}  // namespace supa

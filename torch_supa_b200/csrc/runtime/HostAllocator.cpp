// Caching allocator for pinned (page-locked) host memory, the memory behind tensor.pin_memory() and non-blocking copies.
//
// cudaHostAlloc and cudaFreeHost are expensive and synchronise the device, so blocks are kept: freed blocks go to a free
// list per size class (powers of two from 512 bytes) and are handed out again.  A block that a non-blocking copy still
// reads or writes must not be reused early: every such copy records an event on its stream for the block
// (record_pinned_use), and a freed block with events outstanding waits in a pending list until they have all
// completed.  The same scheme as the reference's host allocator (torch_supa/csrc/core/supa/CachingHostAllocator.cpp:119-121,
// which instantiates libtorch's CachingHostAllocatorImpl for its runtime); written out here on the CUDA runtime.
#include <deque>
#include <map>
#include <mutex>
#include <vector>

#include "Runtime.h"

namespace supa {

namespace {

struct HostBlock {
  void* ptr = nullptr;
  size_t size = 0;
  bool allocated = false;
  std::vector<cudaEvent_t> events;  // uses by asynchronous copies that may still be running
};

class HostCache {
 public:
  void* allocate(size_t nbytes) {
    const size_t size = size_class(nbytes);
    {
      std::lock_guard<std::mutex> lock(mu_);
      retire_pending();
      auto& list = free_[size];
      if (!list.empty()) {
        HostBlock* b = list.back();
        list.pop_back();
        b->allocated = true;
        ++stats_.hits;
        stats_.allocated_bytes += static_cast<int64_t>(b->size);
        return b->ptr;
      }
    }
    void* ptr = nullptr;
    cudaError_t err = cudaHostAlloc(&ptr, size, cudaHostAllocDefault);
    if (err != cudaSuccess) {  // give cached blocks back and try once more
      cudaGetLastError();
      empty();
      err = cudaHostAlloc(&ptr, size, cudaHostAllocDefault);
    }
    SUPA_CUDA_CHECK(err);
    std::lock_guard<std::mutex> lock(mu_);
    HostBlock* b = new HostBlock{ptr, size, true, {}};
    blocks_[ptr] = b;
    ++stats_.host_allocs;
    stats_.reserved_bytes += static_cast<int64_t>(size);
    stats_.allocated_bytes += static_cast<int64_t>(size);
    return ptr;
  }

  void free(void* ptr) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lock(mu_);
    auto it = blocks_.find(ptr);
    if (it == blocks_.end()) return;
    HostBlock* b = it->second;
    b->allocated = false;
    stats_.allocated_bytes -= static_cast<int64_t>(b->size);
    if (b->events.empty()) free_[b->size].push_back(b);
    else pending_.push_back(b);
  }

  // `ptr` may point anywhere inside a block (a view of a pinned tensor).
  bool record(const void* ptr, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(mu_);
    HostBlock* b = find_containing(ptr);
    if (!b) return false;
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (cudaEventRecord(ev, stream) != cudaSuccess) {
      cudaGetLastError();
      cudaEventDestroy(ev);
      return false;
    }
    b->events.push_back(ev);
    return true;
  }

  bool owns(const void* ptr) {
    std::lock_guard<std::mutex> lock(mu_);
    return find_containing(ptr) != nullptr;
  }

  void empty() {
    std::lock_guard<std::mutex> lock(mu_);
    retire_pending();
    for (auto& kv : free_) {
      for (HostBlock* b : kv.second) {
        cudaFreeHost(b->ptr);
        cudaGetLastError();
        stats_.reserved_bytes -= static_cast<int64_t>(b->size);
        blocks_.erase(b->ptr);
        delete b;
      }
      kv.second.clear();
    }
  }

  HostMemoryStats stats() {
    std::lock_guard<std::mutex> lock(mu_);
    return stats_;
  }

 private:
  static size_t size_class(size_t nbytes) {
    size_t s = 512;
    while (s < nbytes) s <<= 1;
    return s;
  }
  HostBlock* find_containing(const void* ptr) {
    auto it = blocks_.upper_bound(const_cast<void*>(ptr));
    if (it == blocks_.begin()) return nullptr;
    --it;
    HostBlock* b = it->second;
    const char* base = static_cast<const char*>(b->ptr);
    return (static_cast<const char*>(ptr) < base + b->size) ? b : nullptr;
  }
  // Moves freed blocks whose recorded copies have all finished to the free lists.  Called with the lock held.
  void retire_pending() {
    for (size_t i = 0; i < pending_.size();) {
      HostBlock* b = pending_[i];
      while (!b->events.empty()) {
        const cudaError_t q = cudaEventQuery(b->events.back());
        if (q == cudaErrorNotReady) break;
        cudaGetLastError();
        cudaEventDestroy(b->events.back());
        b->events.pop_back();
      }
      if (b->events.empty()) {
        free_[b->size].push_back(b);
        pending_[i] = pending_.back();
        pending_.pop_back();
      } else {
        ++i;
      }
    }
  }

  std::mutex mu_;
  std::map<void*, HostBlock*> blocks_;               // every block, by base address
  std::map<size_t, std::vector<HostBlock*>> free_;   // reusable blocks per size class
  std::deque<HostBlock*> pending_;                   // freed, with copies still in flight
  HostMemoryStats stats_{};
};

HostCache& cache() {
  static HostCache* c = new HostCache();  // never destroyed: tensors may outlive static destruction
  return *c;
}

void free_pinned(void* ptr) { cache().free(ptr); }

struct PinnedAllocator final : public c10::Allocator {
  c10::DataPtr allocate(size_t nbytes) override {
    void* ptr = nbytes ? cache().allocate(nbytes) : nullptr;
    return c10::DataPtr(ptr, ptr, &free_pinned, c10::Device(c10::DeviceType::CPU));
  }
  c10::DeleterFnPtr raw_deleter() const override { return &free_pinned; }
  void copy_data(void* dest, const void* src, std::size_t count) const override { default_copy_data(dest, src, count); }
};
PinnedAllocator g_pinned;

}  // namespace

c10::Allocator* pinned_allocator() { return &g_pinned; }
bool record_pinned_use(const void* ptr, cudaStream_t stream) { return cache().record(ptr, stream); }
bool is_cached_pinned(const void* ptr) { return cache().owns(ptr); }
void empty_pinned_cache() { cache().empty(); }
HostMemoryStats host_memory_stats() { return cache().stats(); }

}  // namespace supa

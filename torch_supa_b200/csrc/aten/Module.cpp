// C entry points the Python package binds with ctypes (device control, memory statistics, the NCCL
// communicator), and the all-reduce operator for supa tensors.  Errors travel as a thread-local message
// (supa_last_error) plus a non-zero return code, since C++ exceptions cannot cross a ctypes call.
#include <torch/library.h>

#include <cstring>
#include <string>

#include "Common.h"
#include "dist/NcclComm.h"
#include "dist/PeerExchange.h"
#include "runtime/Generator.h"

namespace {

thread_local std::string g_last_error;

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const c10::Error& e) {
    g_last_error = e.what_without_backtrace();
  } catch (const std::exception& e) {
    g_last_error = e.what();
  }
  return -1;
}

}  // namespace

extern "C" {

SUPA_EXPORT const char* supa_last_error() { return g_last_error.c_str(); }
SUPA_EXPORT int supa_device_count() { return supa::device_count(); }
SUPA_EXPORT int supa_current_device(int* out) {
  return guarded([&] { *out = supa::current_device(); });
}
SUPA_EXPORT int supa_set_device(int device) {
  return guarded([&] { supa::set_device(static_cast<c10::DeviceIndex>(device)); });
}
SUPA_EXPORT int supa_synchronize(int device) {
  return guarded([&] { supa::synchronize_device(static_cast<c10::DeviceIndex>(device < 0 ? supa::current_device() : device)); });
}
SUPA_EXPORT int supa_current_stream(int device, void** out) {
  return guarded([&] { *out = supa::current_cuda_stream(static_cast<c10::DeviceIndex>(device)); });
}
SUPA_EXPORT int supa_memory_stats(int device, int64_t* out6) {
  return guarded([&] {
    const supa::MemoryStats s = supa::memory_stats(static_cast<c10::DeviceIndex>(device));
    out6[0] = s.allocated_bytes;
    out6[1] = s.peak_allocated_bytes;
    out6[2] = s.reserved_bytes;
    out6[3] = s.num_allocs;
    out6[4] = s.num_frees;
    out6[5] = s.num_ooms;
  });
}
SUPA_EXPORT int supa_reset_peak_memory_stats(int device) {
  return guarded([&] { supa::reset_peak_memory_stats(static_cast<c10::DeviceIndex>(device)); });
}
SUPA_EXPORT int supa_empty_cache() {
  return guarded([&] { supa::empty_cache(); });
}
SUPA_EXPORT int supa_host_memory_stats(int64_t* out4) {
  return guarded([&] {
    const supa::HostMemoryStats s = supa::host_memory_stats();
    out4[0] = s.allocated_bytes;
    out4[1] = s.reserved_bytes;
    out4[2] = s.host_allocs;
    out4[3] = s.hits;
  });
}
SUPA_EXPORT int supa_empty_pinned_cache() {
  return guarded([&] { supa::empty_pinned_cache(); });
}
// The default generator of `device` (-1: the current device).  op 0: manual_seed(value); 1: seed() -> *out; 2: initial_seed
// -> *out; 3: offset -> *out; 4: set offset(value).
SUPA_EXPORT int supa_generator_control(int device, int op, uint64_t value, uint64_t* out) {
  return guarded([&] {
    auto* gen = supa::generator_or_default(c10::nullopt, static_cast<c10::DeviceIndex>(device));
    std::lock_guard<std::mutex> lock(gen->mutex_);
    switch (op) {
      case 0: gen->set_current_seed(value); break;
      case 1: *out = gen->seed(); break;
      case 2: *out = gen->current_seed(); break;
      case 3: *out = gen->get_offset(); break;
      case 4: gen->set_offset(value); break;
      default: TORCH_CHECK(false, "supa_generator_control: unknown op ", op);
    }
  });
}
// The 16-byte state (seed, offset) of the default generator of `device`.
SUPA_EXPORT int supa_get_rng_state(int device, uint8_t* out16) {
  return guarded([&] {
    auto* gen = supa::generator_or_default(c10::nullopt, static_cast<c10::DeviceIndex>(device));
    std::lock_guard<std::mutex> lock(gen->mutex_);
    const auto state = gen->get_state();
    std::memcpy(out16, state->data(), 16);
  });
}
SUPA_EXPORT int supa_set_rng_state(int device, const uint8_t* state, int64_t nbytes) {
  return guarded([&] {
    auto* gen = supa::generator_or_default(c10::nullopt, static_cast<c10::DeviceIndex>(device));
    at::Tensor t = at::empty({nbytes}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
    std::memcpy(t.data_ptr(), state, static_cast<size_t>(nbytes));
    std::lock_guard<std::mutex> lock(gen->mutex_);
    gen->set_state(*t.unsafeGetTensorImpl());
  });
}
SUPA_EXPORT int supa_set_memory_limit(int device, int64_t bytes) {
  return guarded([&] { supa::set_memory_limit(static_cast<c10::DeviceIndex>(device), bytes); });
}
// Reads and clears the device status word after draining the current stream; a set error bit comes back
// as a non-zero return code with the message in supa_last_error().
SUPA_EXPORT int supa_check_status(int device) {
  return guarded([&] {
    const c10::DeviceIndex d = static_cast<c10::DeviceIndex>(device < 0 ? supa::current_device() : device);
    supa::check_status_word(d, supa::current_cuda_stream(d));
  });
}

// Raw copy between any two addresses the CUDA runtime knows (device, pinned or pageable host), queued on the
// calling thread's current stream of `device`.
SUPA_EXPORT int supa_memcpy_async(int device, void* dst, const void* src, int64_t nbytes) {
  return guarded([&] {
    const c10::DeviceIndex d = static_cast<c10::DeviceIndex>(device < 0 ? supa::current_device() : device);
    const c10::DeviceIndex prev = supa::exchange_device(d);
    const cudaError_t err = cudaMemcpyAsync(dst, src, static_cast<size_t>(nbytes), cudaMemcpyDefault, supa::current_cuda_stream(d));
    if (prev != d) supa::set_device(prev);
    SUPA_CUDA_CHECK(err);
  });
}

// ---- NCCL communicator --------------------------------------------------------------------------------------
SUPA_EXPORT int supa_nccl_unique_id(char* out128) {
  return guarded([&] { supa::NcclComm::unique_id(out128); });
}
SUPA_EXPORT int supa_nccl_init(int nranks, const char* id128, int rank, int device, int64_t* handle) {
  return guarded([&] { *handle = (new supa::NcclComm(nranks, id128, rank, device))->handle(); });
}
SUPA_EXPORT int supa_nccl_destroy(int64_t handle) {
  return guarded([&] { delete supa::NcclComm::from_handle(handle); });
}
SUPA_EXPORT int supa_nccl_abort(int64_t handle) {
  return guarded([&] { supa::NcclComm::from_handle(handle)->abort(); });
}
SUPA_EXPORT int supa_nccl_all_reduce(int64_t handle, void* data, int64_t count, int dtype, int op, void* stream) {
  return guarded([&] { supa::NcclComm::from_handle(handle)->all_reduce(data, count, dtype, op, stream); });
}


// ---- peer-memory exchange of the loss scalars (see dist/PeerExchange.h) -----------------------------------------
SUPA_EXPORT int supa_peer_create(int nranks, int rank, int device, int64_t* handle) {
  return guarded([&] { *handle = (new supa::PeerExchange(nranks, rank, device))->handle(); });
}
SUPA_EXPORT int supa_peer_export(int64_t handle, char* out64) {
  return guarded([&] { supa::PeerExchange::from_handle(handle)->export_handle(out64); });
}
SUPA_EXPORT int supa_peer_open(int64_t handle, const char* handles) {
  return guarded([&] { supa::PeerExchange::from_handle(handle)->open_peers(handles); });
}
SUPA_EXPORT int supa_peer_destroy(int64_t handle) {
  return guarded([&] { delete supa::PeerExchange::from_handle(handle); });
}

}  // extern "C"

namespace supa {
namespace {

// supa_b200::all_reduce_(Tensor(a!) self, int comm, int op) -> Tensor(a!): in place, on the current stream.
at::Tensor& all_reduce_(at::Tensor& self, int64_t comm, int64_t op) {
  TORCH_CHECK(is_supa(self) && self.is_contiguous(), "all_reduce_: expected a contiguous supa tensor");
  const c10::DeviceGuard guard(self.device());
  NcclComm::from_handle(comm)->all_reduce(self.data_ptr(), self.numel(), dtype_code(self.scalar_type()), static_cast<int>(op),
                                          stream_of(self));
  return self;
}

}  // namespace
}  // namespace supa

TORCH_LIBRARY_FRAGMENT(supa_b200, m) { m.def("all_reduce_(Tensor(a!) self, int comm, int op) -> Tensor(a!)"); }
TORCH_LIBRARY_IMPL(supa_b200, PrivateUse1, m) { m.impl("all_reduce_", TORCH_FN(supa::all_reduce_)); }

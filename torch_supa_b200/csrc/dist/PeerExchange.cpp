#include "PeerExchange.h"

#include <c10/util/Exception.h>

#include <cstring>
#include <mutex>
#include <set>

#include "runtime/Runtime.h"

namespace supa {

namespace {
std::mutex g_mu;
std::set<PeerExchange*> g_live;

struct DeviceScope {
  explicit DeviceScope(int device) {
    cudaGetDevice(&prev_);
    if (prev_ != device) cudaSetDevice(device);
    device_ = device;
  }
  ~DeviceScope() {
    if (prev_ >= 0 && prev_ != device_) cudaSetDevice(prev_);
  }
  int prev_ = -1, device_ = -1;
};
}  // namespace

PeerExchange::PeerExchange(int nranks, int rank, int device) : nranks_(nranks), rank_(rank), device_(device) {
  static_assert(sizeof(cudaIpcMemHandle_t) == kHandleBytes, "IPC handle size");
  TORCH_CHECK(nranks >= 1 && nranks <= SB_XCHG_MAX_RANKS, "supa: the peer exchange serves 1..", SB_XCHG_MAX_RANKS, " ranks, got ", nranks);
  TORCH_CHECK(rank >= 0 && rank < nranks, "supa: invalid rank ", rank, " of ", nranks);
  const DeviceScope scope(device);
  // cudaMalloc, not the stream-ordered pool: only plain allocations can be exported through CUDA IPC
  SUPA_CUDA_CHECK(cudaMalloc(&slots_[rank], SB_XCHG_SLOT_BYTES));
  SUPA_CUDA_CHECK(cudaMemset(slots_[rank], 0, SB_XCHG_SLOT_BYTES));
  SUPA_CUDA_CHECK(cudaDeviceSynchronize());
  if (nranks == 1) ready_ = true;
  std::lock_guard<std::mutex> lock(g_mu);
  g_live.insert(this);
}

PeerExchange::~PeerExchange() {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_live.erase(this);
  }
  const DeviceScope scope(device_);
  cudaDeviceSynchronize();  // no kernel of this rank may still be writing into a peer's array
  for (int r = 0; r < nranks_; ++r) {
    if (!slots_[r]) continue;
    if (r == rank_) cudaFree(slots_[r]);
    else cudaIpcCloseMemHandle(slots_[r]);
  }
}

void PeerExchange::export_handle(char* out) const {
  const DeviceScope scope(device_);
  cudaIpcMemHandle_t h;
  SUPA_CUDA_CHECK(cudaIpcGetMemHandle(&h, slots_[rank_]));
  std::memcpy(out, &h, kHandleBytes);
}

void PeerExchange::open_peers(const char* handles) {
  const DeviceScope scope(device_);
  for (int r = 0; r < nranks_; ++r) {
    if (r == rank_ || slots_[r]) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handles + static_cast<size_t>(r) * kHandleBytes, kHandleBytes);
    SUPA_CUDA_CHECK(cudaIpcOpenMemHandle(&slots_[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  ready_ = true;
}

sb_xchg PeerExchange::next() {
  TORCH_CHECK(ready_, "supa: the peer exchange has not mapped its peers yet");
  sb_xchg x{};
  for (int r = 0; r < nranks_; ++r) x.slots[r] = slots_[r];
  x.rank = rank_;
  x.nranks = nranks_;
  x.seq = ++seq_;
  return x;
}

PeerExchange* PeerExchange::from_handle(int64_t h) {
  PeerExchange* p = reinterpret_cast<PeerExchange*>(h);
  std::lock_guard<std::mutex> lock(g_mu);
  TORCH_CHECK(g_live.count(p), "supa: invalid peer-exchange handle");
  return p;
}

}  // namespace supa

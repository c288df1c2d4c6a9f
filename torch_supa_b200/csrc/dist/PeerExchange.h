// Slot arrays in peer device memory for the two scalar exchanges of row-sharded cross entropy (the sb_xchg part of
// include/supa_b200_kernels.h).  One process per GPU: every rank allocates a small zeroed slot array, publishes its
// CUDA IPC handle, and maps the arrays of all other ranks, which must be GPUs of the same node with peer access
// (NVLink / NVSwitch).  The bookkeeping kernels then store their partials straight into the peers' arrays, so the
// loss path launches no collective between the count, the sweep and the loss.  It stands where the reference would
// call ProcessGroupBCCL::allreduce twice (torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3723-3790); the NCCL
// communicator remains the route when the arrays cannot be mapped.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "supa_b200_kernels.h"

namespace supa {

class PeerExchange {
 public:
  static constexpr int kHandleBytes = 64;  // sizeof(cudaIpcMemHandle_t)

  // Allocates and zeroes this rank's slot array on `device`.
  PeerExchange(int nranks, int rank, int device);
  ~PeerExchange();
  PeerExchange(const PeerExchange&) = delete;
  PeerExchange& operator=(const PeerExchange&) = delete;

  // The IPC handle of this rank's array (kHandleBytes) for the other ranks.
  void export_handle(char* out) const;
  // Maps every other rank's array; `handles` holds nranks * kHandleBytes bytes in rank order.
  void open_peers(const char* handles);

  // Descriptor of the next exchange (every rank must ask in the same order).
  sb_xchg next();
  bool ready() const { return ready_; }
  int nranks() const { return nranks_; }

  int64_t handle() const { return reinterpret_cast<int64_t>(this); }
  static PeerExchange* from_handle(int64_t h);

 private:
  int nranks_, rank_, device_;
  void* slots_[SB_XCHG_MAX_RANKS] = {};
  uint64_t seq_ = 0;
  bool ready_ = false;
};

}  // namespace supa

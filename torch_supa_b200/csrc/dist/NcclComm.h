// NCCL communicator on raw device pointers: the all-reduce of (loss sum, valid-row count) that joins
// row-sharded cross entropy across GPUs.  It replaces the BCCL path of the reference
// (torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3723-3790, BCCLUtils.hpp:262-285) for the one collective the
// hot path needs; ProcessGroupNCCL cannot be used because it only accepts CUDA-typed tensors.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "supa_b200_kernels.h"

namespace supa {

class NcclComm {
 public:
  static constexpr int kUniqueIdBytes = 128;

  // Fills `out` (kUniqueIdBytes) with a fresh unique id; rank 0 calls this and shares the bytes.
  static void unique_id(char* out);
  // Collective over all ranks of the group: creates the communicator for `rank` on `device`.
  NcclComm(int nranks, const char* id_bytes, int rank, int device);
  ~NcclComm();
  NcclComm(const NcclComm&) = delete;
  NcclComm& operator=(const NcclComm&) = delete;

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  int device() const { return device_; }

  // In-place sum of `count` doubles across ranks, queued on `stream`.
  void all_reduce_sum_f64(double* data, int64_t count, sb_stream_t stream);
  // In-place all-reduce of any dtype the kernel library knows; op: 0 sum, 1 max, 2 min, 3 product, 4 average.
  void all_reduce(void* data, int64_t count, int dtype, int op, sb_stream_t stream);
  // In place: every rank ends up with the `count` elements of rank `root`.
  void broadcast(void* data, int64_t count, int dtype, int root, sb_stream_t stream);
  // recv holds nranks * count elements: rank r's `count` elements at offset r * count.
  void all_gather(const void* send, void* recv, int64_t count, int dtype, sb_stream_t stream);
  // send holds nranks * count elements; rank r receives the reduction of everyone's r-th block.
  void reduce_scatter(const void* send, void* recv, int64_t count, int dtype, int op, sb_stream_t stream);
  // Tears the communicator down without waiting for outstanding work (after a failed rank).
  void abort();

  int64_t handle() const { return reinterpret_cast<int64_t>(this); }
  static NcclComm* from_handle(int64_t h);

 private:
  void* comm_ = nullptr;
  int rank_, nranks_, device_;
};

}  // namespace supa

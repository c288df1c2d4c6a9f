// c10d backend for tensors on the supa device: torch.distributed.all_reduce / broadcast / all_gather / reduce_scatter /
// barrier, and with them DistributedDataParallel, on PrivateUse1 tensors.  It is the counterpart of the reference's
// ProcessGroupBCCL (torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3723-3790 for allreduce) registered from Python for
// the device (torch_supa/distributed/distributed_c10d.py:65-102), over the NCCL communicator of NcclComm.h.
//
// Collectives are queued on the calling thread's current stream of the device, so they are ordered with the kernels
// around them without events; a Work object only remembers an event recorded behind the collective.  Deadlines are
// enforced on the host: wait(timeout) polls that event and, when the time is up, aborts the communicator and throws,
// which is how a rank learns that a peer is gone (BCCLUtils.hpp:389-434 of the reference does the same from a watchdog).
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <chrono>
#include <memory>

#include "NcclComm.h"

namespace supa {

class SupaBackend final : public c10d::Backend {
 public:
  SupaBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout);
  ~SupaBackend() override;

  const std::string getBackendName() const override { return "supa_nccl"; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input, const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override;
  void setTimeout(std::chrono::milliseconds timeout) override { timeout_ = timeout; }
  void abort() override;
  void shutdown() override;

 private:
  NcclComm& comm(const at::Tensor& like);
  c10::intrusive_ptr<c10d::Work> finish(std::vector<at::Tensor> outputs, c10d::OpType op, const at::Tensor& like);

  c10::intrusive_ptr<c10d::Store> store_;
  std::chrono::milliseconds timeout_;
  std::unique_ptr<NcclComm> comm_;  // created with the first collective, on the device of its tensor
  int device_ = -1;
};

// Creator registered with torch.distributed.Backend.register_backend.
c10::intrusive_ptr<c10d::Backend> create_supa_backend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                      std::chrono::milliseconds timeout);

}  // namespace supa

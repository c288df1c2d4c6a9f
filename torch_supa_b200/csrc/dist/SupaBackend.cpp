#include "SupaBackend.h"

#include <ATen/ATen.h>
#include <c10/core/DeviceGuard.h>

#include <thread>

#include "aten/Common.h"

namespace supa {

namespace {

// An event recorded behind the collective on the stream it was queued on.
class SupaWork final : public c10d::Work {
 public:
  SupaWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, int device, cudaStream_t stream, std::chrono::milliseconds timeout,
           NcclComm* comm)
      : c10d::Work(rank, op), outputs_(std::move(outputs)), device_(device), timeout_(timeout), comm_(comm) {
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != device) cudaSetDevice(device);
    SUPA_CUDA_CHECK(cudaEventCreateWithFlags(&event_, cudaEventDisableTiming));
    SUPA_CUDA_CHECK(cudaEventRecord(event_, stream));
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                      std::vector<c10::Device>{c10::Device(c10::DeviceType::PrivateUse1, static_cast<c10::DeviceIndex>(device))});
    // the collective is ordered on the stream its consumers use: the value can be handed out now
    future_->markCompleted(c10::IValue(outputs_));
  }
  ~SupaWork() override {
    if (event_) cudaEventDestroy(event_);
  }
  bool isCompleted() override { return cudaEventQuery(event_) == cudaSuccess; }
  bool isSuccess() const override { return true; }
  // Stream semantics, as ProcessGroupNCCL's: the collective sits on the caller's stream, later kernels follow it there,
  // so nothing blocks unless a deadline is asked for.
  bool wait(std::chrono::milliseconds timeout) override {
    if (timeout == kNoTimeout) return true;
    return wait_on_host(timeout);
  }
  void synchronize() override {}
  // Host-side deadline: polls the event; when the time is up the communicator is torn down and the caller gets an error.
  bool wait_on_host(std::chrono::milliseconds timeout) {
    const auto limit = timeout.count() > 0 ? timeout : timeout_;
    const auto start = std::chrono::steady_clock::now();
    while (cudaEventQuery(event_) == cudaErrorNotReady) {
      if (limit.count() > 0 && std::chrono::steady_clock::now() - start > limit) {
        if (comm_) comm_->abort();
        TORCH_CHECK(false, "supa_nccl: a collective did not finish within ", limit.count(), " ms; the communicator was aborted");
      }
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    cudaGetLastError();
    return true;
  }
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
  std::vector<at::Tensor> outputs_;
  int device_;
  std::chrono::milliseconds timeout_;
  NcclComm* comm_;
  cudaEvent_t event_ = nullptr;
  c10::intrusive_ptr<at::ivalue::Future> future_;
};

int reduce_code(const c10d::ReduceOp& op) {
  switch (op) {
    case c10d::ReduceOp::SUM: return 0;
    case c10d::ReduceOp::MAX: return 1;
    case c10d::ReduceOp::MIN: return 2;
    case c10d::ReduceOp::PRODUCT: return 3;
    case c10d::ReduceOp::AVG: return 4;
    default: TORCH_CHECK(false, "supa_nccl: unsupported reduce op");
  }
}

void check_tensor(const at::Tensor& t, const char* what) {
  TORCH_CHECK(is_supa(t), "supa_nccl ", what, ": expected a tensor on a supa device, got ", t.device());
  TORCH_CHECK(t.is_contiguous(), "supa_nccl ", what, ": tensors must be contiguous");
}

}  // namespace

SupaBackend::SupaBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout)
    : c10d::Backend(rank, size), store_(store), timeout_(timeout) {}

SupaBackend::~SupaBackend() = default;

// The communicator is created by the first collective (every rank issues the same one), on the device of its tensor: the
// unique id travels through the store of the process group.
NcclComm& SupaBackend::comm(const at::Tensor& like) {
  const int device = like.device().index();
  if (!comm_) {
    const std::string key = "supa_nccl/unique_id";
    std::vector<uint8_t> id(NcclComm::kUniqueIdBytes);
    if (getRank() == 0) {
      NcclComm::unique_id(reinterpret_cast<char*>(id.data()));
      store_->set(key, id);
    } else {
      id = store_->get(key);
      TORCH_CHECK(id.size() == NcclComm::kUniqueIdBytes, "supa_nccl: malformed unique id in the store");
    }
    comm_ = std::make_unique<NcclComm>(getSize(), reinterpret_cast<const char*>(id.data()), getRank(), device);
    device_ = device;
  }
  TORCH_CHECK(device == device_, "supa_nccl: this process group is bound to supa:", device_, ", got a tensor on supa:", device);
  return *comm_;
}

c10::intrusive_ptr<c10d::Work> SupaBackend::finish(std::vector<at::Tensor> outputs, c10d::OpType op, const at::Tensor& like) {
  return c10::make_intrusive<SupaWork>(getRank(), op, std::move(outputs), device_, static_cast<cudaStream_t>(stream_of(like)), timeout_,
                                       comm_.get());
}

c10::intrusive_ptr<c10d::Work> SupaBackend::allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) {
  TORCH_CHECK(!tensors.empty(), "supa_nccl allreduce: no tensors");
  const int op = reduce_code(opts.reduceOp);
  for (at::Tensor& t : tensors) {
    check_tensor(t, "allreduce");
    const c10::DeviceGuard guard(t.device());
    comm(t).all_reduce(t.data_ptr(), t.numel(), dtype_code(t.scalar_type()), op, stream_of(t));
  }
  return finish(tensors, c10d::OpType::ALLREDUCE, tensors[0]);
}

c10::intrusive_ptr<c10d::Work> SupaBackend::allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) {
  c10d::AllreduceOptions o;
  o.reduceOp = opts.reduceOp;
  o.timeout = opts.timeout;
  return allreduce(tensors, o);
}

c10::intrusive_ptr<c10d::Work> SupaBackend::broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) {
  TORCH_CHECK(!tensors.empty(), "supa_nccl broadcast: no tensors");
  for (at::Tensor& t : tensors) {
    check_tensor(t, "broadcast");
    const c10::DeviceGuard guard(t.device());
    comm(t).broadcast(t.data_ptr(), t.numel(), dtype_code(t.scalar_type()), static_cast<int>(opts.rootRank), stream_of(t));
  }
  return finish(tensors, c10d::OpType::BROADCAST, tensors[0]);
}

c10::intrusive_ptr<c10d::Work> SupaBackend::_allgather_base(at::Tensor& output, at::Tensor& input, const c10d::AllgatherOptions&) {
  check_tensor(output, "all_gather_into_tensor");
  check_tensor(input, "all_gather_into_tensor");
  TORCH_CHECK(output.scalar_type() == input.scalar_type() && output.numel() == input.numel() * getSize(),
              "supa_nccl all_gather_into_tensor: the output must hold world_size times the input");
  const c10::DeviceGuard guard(input.device());
  comm(input).all_gather(input.const_data_ptr(), output.data_ptr(), input.numel(), dtype_code(input.scalar_type()), stream_of(input));
  return finish({output}, c10d::OpType::_ALLGATHER_BASE, input);
}

c10::intrusive_ptr<c10d::Work> SupaBackend::allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                                      const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "supa_nccl allgather: one input tensor per rank");
  at::Tensor& input = inputs[0];
  check_tensor(input, "allgather");
  TORCH_CHECK(static_cast<int>(outputs[0].size()) == getSize(), "supa_nccl allgather: expected world_size output tensors");
  const c10::DeviceGuard guard(input.device());
  at::Tensor flat = at::empty({getSize(), input.numel()}, input.options());
  comm(input).all_gather(input.const_data_ptr(), flat.data_ptr(), input.numel(), dtype_code(input.scalar_type()), stream_of(input));
  for (int r = 0; r < getSize(); ++r) {
    TORCH_CHECK(outputs[0][r].numel() == input.numel(), "supa_nccl allgather: output ", r, " has another size than the input");
    outputs[0][r].copy_(flat[r].view_as(outputs[0][r]));
  }
  return finish(outputs[0], c10d::OpType::ALLGATHER, input);
}

c10::intrusive_ptr<c10d::Work> SupaBackend::_reduce_scatter_base(at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) {
  check_tensor(output, "reduce_scatter_tensor");
  check_tensor(input, "reduce_scatter_tensor");
  TORCH_CHECK(output.scalar_type() == input.scalar_type() && input.numel() == output.numel() * getSize(),
              "supa_nccl reduce_scatter_tensor: the input must hold world_size times the output");
  const c10::DeviceGuard guard(input.device());
  comm(input).reduce_scatter(input.const_data_ptr(), output.data_ptr(), output.numel(), dtype_code(input.scalar_type()),
                             reduce_code(opts.reduceOp), stream_of(input));
  return finish({output}, c10d::OpType::_REDUCE_SCATTER_BASE, input);
}

// An all-reduce of one element, then the host waits for it (with the group's deadline).
c10::intrusive_ptr<c10d::Work> SupaBackend::barrier(const c10d::BarrierOptions& opts) {
  int device = device_;
  if (device < 0) device = !opts.device_ids.empty() ? static_cast<int>(opts.device_ids[0]) : static_cast<int>(current_device());
  const c10::Device dev(c10::DeviceType::PrivateUse1, static_cast<c10::DeviceIndex>(device));
  const c10::DeviceGuard guard(dev);
  at::Tensor token = at::zeros({1}, at::TensorOptions().dtype(at::kFloat).device(dev));
  comm(token).all_reduce(token.data_ptr(), 1, SB_F32, 0, stream_of(token));
  auto work = c10::make_intrusive<SupaWork>(getRank(), c10d::OpType::BARRIER, std::vector<at::Tensor>{token}, device_,
                                            static_cast<cudaStream_t>(stream_of(token)), timeout_, comm_.get());
  work->wait_on_host(std::chrono::milliseconds(0));
  return work;
}

void SupaBackend::abort() {
  if (comm_) comm_->abort();
}

void SupaBackend::shutdown() { comm_.reset(); }

c10::intrusive_ptr<c10d::Backend> create_supa_backend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                      std::chrono::milliseconds timeout) {
  return c10::make_intrusive<SupaBackend>(store, rank, size, timeout);
}

}  // namespace supa

// NCCL bindings resolved at run time from the libnccl.so.2 that is already mapped into the process (the one
// libtorch_cuda links), so that a single NCCL copy serves torch.distributed and this communicator.
#include "NcclComm.h"

#include <c10/util/Exception.h>
#include <dlfcn.h>

#include <cstring>

#include <mutex>
#include <set>

namespace supa {

namespace {

struct ncclUniqueIdRaw {
  char internal[NcclComm::kUniqueIdBytes];
};
using ncclComm_t = void*;
// Values of ncclDataType_t / ncclRedOp_t / ncclResult_t from the public nccl.h.
enum { kNcclInt8 = 0, kNcclUint8 = 1, kNcclInt32 = 2, kNcclInt64 = 4, kNcclHalf = 6, kNcclFloat = 7, kNcclDouble = 8, kNcclBfloat16 = 9 };
enum { kNcclSum = 0, kNcclProd = 1, kNcclMax = 2, kNcclMin = 3, kNcclAvg = 4 };

struct Api {
  int (*GetUniqueId)(ncclUniqueIdRaw*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueIdRaw, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

const Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    TORCH_CHECK(h, "supa: libnccl.so.2 could not be loaded: ", dlerror());
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(dlsym(h, "ncclCommAbort"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    a.Broadcast = reinterpret_cast<decltype(a.Broadcast)>(dlsym(h, "ncclBroadcast"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.ReduceScatter = reinterpret_cast<decltype(a.ReduceScatter)>(dlsym(h, "ncclReduceScatter"));
    TORCH_CHECK(a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.AllReduce && a.GetErrorString && a.Broadcast &&
                    a.AllGather && a.ReduceScatter,
                "supa: libnccl.so.2 lacks an expected symbol");
  });
  return a;
}

void check_nccl(int rc, const char* what) { TORCH_CHECK(rc == 0, "NCCL error in ", what, ": ", api().GetErrorString(rc)); }

std::mutex g_mu;
std::set<NcclComm*> g_live;

int nccl_dtype(int dtype) {
  switch (dtype) {
    case SB_I8: return kNcclInt8;
    case SB_U8: case SB_BOOL: return kNcclUint8;
    case SB_I32: return kNcclInt32;
    case SB_I64: return kNcclInt64;
    case SB_F16: return kNcclHalf;
    case SB_BF16: return kNcclBfloat16;
    case SB_F32: return kNcclFloat;
    case SB_F64: return kNcclDouble;
    default: TORCH_CHECK(false, "supa: dtype has no NCCL equivalent");
  }
}

int nccl_op(int op) {
  switch (op) {
    case 0: return kNcclSum;
    case 1: return kNcclMax;
    case 2: return kNcclMin;
    case 3: return kNcclProd;
    case 4: return kNcclAvg;
    default: TORCH_CHECK(false, "supa: unknown reduction op ", op);
  }
}

}  // namespace

void NcclComm::unique_id(char* out) {
  ncclUniqueIdRaw id;
  check_nccl(api().GetUniqueId(&id), "ncclGetUniqueId");
  std::memcpy(out, id.internal, kUniqueIdBytes);
}

NcclComm::NcclComm(int nranks, const char* id_bytes, int rank, int device) : rank_(rank), nranks_(nranks), device_(device) {
  TORCH_CHECK(nranks >= 1 && rank >= 0 && rank < nranks, "supa: invalid rank ", rank, " of ", nranks);
  ncclUniqueIdRaw id;
  std::memcpy(id.internal, id_bytes, kUniqueIdBytes);
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  const int rc = api().CommInitRank(&comm_, nranks, id, rank);
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  check_nccl(rc, "ncclCommInitRank");
  std::lock_guard<std::mutex> lock(g_mu);
  g_live.insert(this);
}

NcclComm::~NcclComm() {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_live.erase(this);
  }
  if (comm_) api().CommDestroy(comm_);
}

void NcclComm::abort() {
  if (comm_) api().CommAbort(comm_);
  comm_ = nullptr;
}

void NcclComm::all_reduce(void* data, int64_t count, int dtype, int op, sb_stream_t stream) {
  TORCH_CHECK(comm_, "supa: communicator has been aborted");
  TORCH_CHECK(count >= 0 && (count == 0 || data), "supa: invalid all_reduce buffer");
  if (count == 0) return;
  check_nccl(api().AllReduce(data, data, static_cast<size_t>(count), nccl_dtype(dtype), nccl_op(op), comm_, static_cast<cudaStream_t>(stream)),
             "ncclAllReduce");
}

void NcclComm::broadcast(void* data, int64_t count, int dtype, int root, sb_stream_t stream) {
  TORCH_CHECK(comm_, "supa: communicator has been aborted");
  TORCH_CHECK(count >= 0 && (count == 0 || data) && root >= 0 && root < nranks_, "supa: invalid broadcast arguments");
  if (count == 0) return;
  check_nccl(api().Broadcast(data, data, static_cast<size_t>(count), nccl_dtype(dtype), root, comm_, static_cast<cudaStream_t>(stream)),
             "ncclBroadcast");
}

void NcclComm::all_gather(const void* send, void* recv, int64_t count, int dtype, sb_stream_t stream) {
  TORCH_CHECK(comm_, "supa: communicator has been aborted");
  TORCH_CHECK(count >= 0 && (count == 0 || (send && recv)), "supa: invalid all_gather buffers");
  if (count == 0) return;
  check_nccl(api().AllGather(send, recv, static_cast<size_t>(count), nccl_dtype(dtype), comm_, static_cast<cudaStream_t>(stream)),
             "ncclAllGather");
}

void NcclComm::reduce_scatter(const void* send, void* recv, int64_t count, int dtype, int op, sb_stream_t stream) {
  TORCH_CHECK(comm_, "supa: communicator has been aborted");
  TORCH_CHECK(count >= 0 && (count == 0 || (send && recv)), "supa: invalid reduce_scatter buffers");
  if (count == 0) return;
  check_nccl(api().ReduceScatter(send, recv, static_cast<size_t>(count), nccl_dtype(dtype), nccl_op(op), comm_,
                                 static_cast<cudaStream_t>(stream)),
             "ncclReduceScatter");
}

void NcclComm::all_reduce_sum_f64(double* data, int64_t count, sb_stream_t stream) { all_reduce(data, count, SB_F64, 0, stream); }

NcclComm* NcclComm::from_handle(int64_t h) {
  NcclComm* c = reinterpret_cast<NcclComm*>(h);
  std::lock_guard<std::mutex> lock(g_mu);
  TORCH_CHECK(g_live.count(c), "supa: invalid communicator handle");
  return c;
}

}  // namespace supa

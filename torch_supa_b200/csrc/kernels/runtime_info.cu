// Device queries, status strings and other host-only helpers of the kernel library.
#include "common.cuh"

namespace sb {

namespace {
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
int g_smem_optin[kMaxDevices];
}  // namespace

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kDefaultSmCount;
  int v = g_sm_count[dev];  // benign race: every thread computes the same value
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = kDefaultSmCount;
    g_sm_count[dev] = v;
  }
  return v;
}

int max_smem_optin() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 48 * 1024;
  int v = g_smem_optin[dev];
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || v <= 0) v = 48 * 1024;
    g_smem_optin[dev] = v;
  }
  return v;
}

int launch_status() { return cudaGetLastError() == cudaSuccess ? SB_OK : SB_ERR_CUDA; }

}  // namespace sb

extern "C" {

const char* sb_version(void) { return "supa_b200_kernels 0.1 (sm_100a)"; }

int sb_built_for_sm(void) { return 100; }

const char* sb_status_string(int status) {
  switch (status) {
    case SB_OK: return "ok";
    case SB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SB_ERR_UNSUPPORTED: return "unsupported dtype or operation";
    case SB_ERR_CUDA: return "CUDA launch failed";
    case SB_ERR_TOO_LARGE: return "size beyond the documented maximum";
    case SB_ERR_MISALIGNED: return "pointer not aligned to its element size";
    default: return "unknown status";
  }
}

size_t sb_dtype_size(int dtype) { return static_cast<size_t>(sb::dtype_size(dtype)); }

}  // extern "C"

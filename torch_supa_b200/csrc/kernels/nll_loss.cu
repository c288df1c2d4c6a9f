// nll_loss forward / backward for [rows, classes] log-probabilities and class-index targets.
//
// forward:  out_i = -w[t_i] * x[i, t_i] (0 when t_i == ignore_index); `none` stores out_i, `sum` and
//           `mean` reduce it in a fixed order (one CTA, or a cluster of eight for 16384 rows and more: per-thread
//           strided partial sums with four gathers in flight, a tree per CTA, the CTAs' sums added in rank order
//           through distributed shared memory, so the result is bit-reproducible); total_weight = sum of w[t_i]
//           over rows that count.
// backward: grad_input is zero except [i, t_i] = -w[t_i] * g, with g = grad_output_i for `none`,
//           grad_output for `sum`, grad_output / total_weight for `mean`.
// An index outside [0, classes) that is not ignore_index sets SB_STATUS_TARGET_OUT_OF_RANGE and the row
// is skipped; nothing traps.
#include <cooperative_groups.h>

#include "io.cuh"

namespace sb {

namespace {

struct NllParams {
  const void* x;
  const void* target;
  const void* weight;
  int64_t rows, classes, ignore_index;
  int reduction;
  int target_dtype;
  int32_t* status;
};

__device__ __forceinline__ int64_t load_target(const NllParams& p, int64_t i) {
  return p.target_dtype == SB_U8 ? static_cast<int64_t>(static_cast<const uint8_t*>(p.target)[i])
                                 : static_cast<const int64_t*>(p.target)[i];
}

// Returns true when row i counts; fills t.
__device__ __forceinline__ bool row_counts(const NllParams& p, int64_t i, int64_t& t) {
  t = load_target(p, i);
  if (t == p.ignore_index) return false;
  if (t < 0 || t >= p.classes) {
    if (p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    return false;
  }
  return true;
}

template <typename T, typename A>
__global__ void __launch_bounds__(256) nll_fwd_none_kernel(NllParams p, T* __restrict__ out) {
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.weight);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < p.rows;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t t;
    A v = 0;
    if (row_counts(p, i, t)) {
      const A wt = w ? convert<A, T>(w[t]) : A(1);
      v = -wt * convert<A, T>(x[i * p.classes + t]);
    }
    out[i] = convert<T, A>(v);
  }
}

// Whether a target counts (an index outside [0, classes) that is not ignore_index is reported and skipped).
__device__ __forceinline__ bool target_counts(const NllParams& p, int64_t t) {
  if (t == p.ignore_index) return false;
  if (t < 0 || t >= p.classes) {
    if (p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    return false;
  }
  return true;
}

constexpr int kNllClusterMax = 8;

template <typename T, typename A>
__global__ void __launch_bounds__(1024) nll_fwd_reduce_kernel(NllParams p, T* __restrict__ out, T* __restrict__ total_weight) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned nranks = cluster.num_blocks(), rank = cluster.block_rank();
  __shared__ double s_v[32];
  __shared__ double s_w[32];
  __shared__ double c_v[kNllClusterMax];  // the copy of rank 0 collects the CTAs' sums
  __shared__ double c_w[kNllClusterMax];
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.weight);
  double av = 0.0, aw = 0.0;
  const int64_t stride = static_cast<int64_t>(nranks) * 1024;
  int64_t i = static_cast<int64_t>(rank) * 1024 + threadIdx.x;
  // four rows per thread at a time: the four targets, then the four elements they name, are in flight together
  // (a row that does not count reads class 0 instead and is left out of the sums; rows exist, so classes > 0 here
  // whenever a target can count)
  for (; i + 3 * stride < p.rows; i += 4 * stride) {
    int64_t t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] = load_target(p, i + u * stride);
    bool ok[4];
    A xv[4], wt[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      ok[u] = target_counts(p, t[u]);
      const int64_t tt = ok[u] ? t[u] : 0;
      xv[u] = p.classes > 0 ? convert<A, T>(x[(i + u * stride) * p.classes + tt]) : A(0);
      wt[u] = (w && p.classes > 0) ? convert<A, T>(w[tt]) : A(1);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (ok[u]) {
        av -= static_cast<double>(wt[u]) * static_cast<double>(xv[u]);
        aw += static_cast<double>(wt[u]);
      }
    }
  }
  for (; i < p.rows; i += stride) {
    int64_t t;
    if (row_counts(p, i, t)) {
      const double wt = w ? static_cast<double>(convert<A, T>(w[t])) : 1.0;
      av -= wt * static_cast<double>(convert<A, T>(x[i * p.classes + t]));
      aw += wt;
    }
  }
  av = warp_sum(av);
  aw = warp_sum(aw);
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = av;
    s_w[threadIdx.x >> 5] = aw;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    av = warp_sum(s_v[threadIdx.x]);
    aw = warp_sum(s_w[threadIdx.x]);
    if (threadIdx.x == 0) {
      cluster.map_shared_rank(c_v, 0)[rank] = av;
      cluster.map_shared_rank(c_w, 0)[rank] = aw;
    }
  }
  cluster.sync();  // every CTA's pair is in rank 0's shared memory; no CTA leaves before
  if (rank == 0 && threadIdx.x == 0) {
    double tv = c_v[0], tw = c_w[0];
    for (unsigned r = 1; r < nranks; ++r) {
      tv += c_v[r];
      tw += c_w[r];
    }
    double r = tv;
    if (p.reduction == SB_REDUCTION_MEAN) r = tv / tw;  // 0/0 = NaN when every row is ignored
    *out = convert<T, A>(static_cast<A>(r));
    *total_weight = convert<T, A>(static_cast<A>(tw));
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(256) nll_bwd_scatter_kernel(NllParams p, const T* __restrict__ grad_output,
                                                              const T* __restrict__ total_weight, T* __restrict__ grad_input) {
  const T* w = static_cast<const T*>(p.weight);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < p.rows;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t t;
    if (!row_counts(p, i, t)) continue;
    const A wt = w ? convert<A, T>(w[t]) : A(1);
    A g = convert<A, T>(p.reduction == SB_REDUCTION_NONE ? grad_output[i] : grad_output[0]);
    if (p.reduction == SB_REDUCTION_MEAN) g = g / convert<A, T>(*total_weight);
    grad_input[i * p.classes + t] = convert<T, A>(-wt * g);
  }
}

NllParams to_params(const sb_nll_args* a) {
  NllParams p;
  p.x = a->log_probs;
  p.target = a->target;
  p.weight = a->weight;
  p.rows = a->rows;
  p.classes = a->classes;
  p.ignore_index = a->ignore_index;
  p.reduction = a->reduction;
  p.target_dtype = a->target_dtype;
  p.status = a->status;
  return p;
}

int validate(const sb_nll_args* a) {
  if (!a || a->rows < 0 || a->classes < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->reduction < SB_REDUCTION_NONE || a->reduction > SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  if (a->target_dtype != SB_I64 && a->target_dtype != SB_U8) return SB_ERR_UNSUPPORTED;
  if (a->dtype != SB_F32 && a->dtype != SB_BF16 && a->dtype != SB_F16 && a->dtype != SB_F64) return SB_ERR_UNSUPPORTED;
  if (a->rows > 0 && (!a->log_probs || !a->target)) return SB_ERR_INVALID_ARGUMENT;
  return SB_OK;
}

template <typename T, typename A>
int launch_fwd(const sb_nll_args* a, void* output, void* total_weight, cudaStream_t st) {
  NllParams p = to_params(a);
  if (a->reduction == SB_REDUCTION_NONE) {
    if (a->rows == 0) return SB_OK;
    const int64_t ctas = (a->rows + 255) / 256;
    const int grid = static_cast<int>(ctas < 8LL * sm_count() ? ctas : 8LL * sm_count());
    nll_fwd_none_kernel<T, A><<<grid, 256, 0, st>>>(p, static_cast<T*>(output));
    return launch_status();
  }
  cudaLaunchConfig_t cfg{};
  const unsigned ranks = a->rows >= 16384 ? kNllClusterMax : 1;
  cfg.gridDim = dim3(ranks);
  cfg.blockDim = dim3(1024);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ranks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, nll_fwd_reduce_kernel<T, A>, p, static_cast<T*>(output), static_cast<T*>(total_weight)) != cudaSuccess) {
    cudaGetLastError();
    return SB_ERR_CUDA;
  }
  return launch_status();
}

template <typename T, typename A>
int launch_bwd(const sb_nll_args* a, const void* grad_output, const void* total_weight, void* grad_input, cudaStream_t st) {
  NllParams p = to_params(a);
  const size_t bytes = static_cast<size_t>(a->rows) * static_cast<size_t>(a->classes) * sizeof(T);
  if (bytes == 0) return SB_OK;
  if (cudaMemsetAsync(grad_input, 0, bytes, st) != cudaSuccess) return SB_ERR_CUDA;
  const int64_t ctas = (a->rows + 255) / 256;
  const int grid = static_cast<int>(ctas < 8LL * sm_count() ? ctas : 8LL * sm_count());
  nll_bwd_scatter_kernel<T, A><<<grid, 256, 0, st>>>(p, static_cast<const T*>(grad_output),
                                                     static_cast<const T*>(total_weight), static_cast<T*>(grad_input));
  return launch_status();
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

int sb_nll_loss_forward(const sb_nll_args* a, void* output, void* total_weight, sb_stream_t stream) {
  int rc = validate(a);
  if (rc != SB_OK) return rc;
  if (!output || (a->reduction != SB_REDUCTION_NONE && !total_weight)) return SB_ERR_INVALID_ARGUMENT;
  cudaStream_t st = as_stream(stream);
  switch (a->dtype) {
    case SB_F32: return launch_fwd<float, float>(a, output, total_weight, st);
    case SB_BF16: return launch_fwd<__nv_bfloat16, float>(a, output, total_weight, st);
    case SB_F16: return launch_fwd<__half, float>(a, output, total_weight, st);
    default: return launch_fwd<double, double>(a, output, total_weight, st);
  }
}

int sb_nll_loss_backward(const sb_nll_args* a, const void* grad_output, const void* total_weight, void* grad_input,
                         sb_stream_t stream) {
  int rc = validate(a);
  if (rc != SB_OK) return rc;
  if (a->rows > 0 && a->classes > 0 && (!grad_output || !grad_input)) return SB_ERR_INVALID_ARGUMENT;
  if (a->reduction == SB_REDUCTION_MEAN && !total_weight) return SB_ERR_INVALID_ARGUMENT;
  cudaStream_t st = as_stream(stream);
  switch (a->dtype) {
    case SB_F32: return launch_bwd<float, float>(a, grad_output, total_weight, grad_input, st);
    case SB_BF16: return launch_bwd<__nv_bfloat16, float>(a, grad_output, total_weight, grad_input, st);
    case SB_F16: return launch_bwd<__half, float>(a, grad_output, total_weight, grad_input, st);
    default: return launch_bwd<double, double>(a, grad_output, total_weight, grad_input, st);
  }
}

}  // extern "C"

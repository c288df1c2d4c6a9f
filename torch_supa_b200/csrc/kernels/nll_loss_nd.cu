// nll_loss for log-probabilities laid out [outer, classes, inner] with targets [outer, inner]: the 4-D
// (N, C, H, W) form behind nll_loss2d (inner = H * W) and, with inner = 1, the plain [rows, classes] form.
//
// forward:  sample s = (n, i): out_s = -w[t_s] * x[n, t_s, i] (0 when t_s == ignore_index).  `none` stores
//           out_s; `sum` / `mean` reduce in two fixed-order stages (per-CTA partials in caller scratch, then
//           one CTA), so the result is bit-reproducible; total_weight = sum of w[t_s] over samples that count.
// backward: grad_input[n, c, i] = (c == t_s) ? -w[c] * g : 0, written plane by plane so that every store is
//           coalesced along i and the tensor is written exactly once (no zero-fill pass); g = grad_output_s
//           for `none`, grad_output for `sum`, grad_output / total_weight for `mean`.
// An index outside [0, classes) that is not ignore_index sets SB_STATUS_TARGET_OUT_OF_RANGE and the sample is
// skipped; nothing traps.
#include "io.cuh"

namespace sb {

namespace {

constexpr int kMaxPartials = 2048;

struct NdParams {
  const void* x;
  const void* target;
  const void* weight;
  int64_t outer, classes, inner, samples, ignore_index;
  int reduction;
  int target_dtype;
  int32_t* status;
};

__device__ __forceinline__ int64_t nd_target(const NdParams& p, int64_t s) {
  return p.target_dtype == SB_U8 ? static_cast<int64_t>(static_cast<const uint8_t*>(p.target)[s])
                                 : static_cast<const int64_t*>(p.target)[s];
}

__device__ __forceinline__ bool nd_counts(const NdParams& p, int64_t s, int64_t& t) {
  t = nd_target(p, s);
  if (t == p.ignore_index) return false;
  if (t < 0 || t >= p.classes) {
    if (p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    return false;
  }
  return true;
}

// sample index -> (outer row, position inside it); 32-bit division whenever the sample count allows it (a 64-bit
// division costs more than the gather it addresses)
__device__ __forceinline__ void nd_split(const NdParams& p, int64_t s, int64_t& n, int64_t& i) {
  if (p.samples <= 0xffffffffLL) {
    const uint32_t s32 = static_cast<uint32_t>(s), in32 = static_cast<uint32_t>(p.inner);
    const uint32_t n32 = s32 / in32;
    n = n32;
    i = s32 - n32 * in32;
  } else {
    n = s / p.inner;
    i = s - n * p.inner;
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(256) nd_fwd_none_kernel(NdParams p, T* __restrict__ out) {
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.weight);
  for (int64_t s = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; s < p.samples; s += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t t;
    A v = 0;
    if (nd_counts(p, s, t)) {
      int64_t n, i;
      nd_split(p, s, n, i);
      const A wt = w ? convert<A, T>(w[t]) : A(1);
      v = -wt * convert<A, T>(x[(n * p.classes + t) * p.inner + i]);
    }
    out[s] = convert<T, A>(v);
  }
}

// Stage 1: CTA b sums the samples b * 256 + tid, + gridDim * 256, ... and writes {sum, weight} to partial[b].
template <typename T, typename A>
__global__ void __launch_bounds__(256) nd_fwd_partial_kernel(NdParams p, double2* __restrict__ partial) {
  __shared__ double s_v[8];
  __shared__ double s_w[8];
  const T* x = static_cast<const T*>(p.x);
  const T* w = static_cast<const T*>(p.weight);
  double av = 0.0, aw = 0.0;
  // four samples per thread and pass: the targets, then the four gathers they name, are in flight together
  constexpr int kU = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  for (int64_t s0 = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; s0 < p.samples; s0 += stride * kU) {
    int64_t t[kU];
    bool ok[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t s = s0 + u * stride;
      ok[u] = s < p.samples && nd_counts(p, s, t[u]);
    }
    A xv[kU], wv[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      xv[u] = A(0);
      wv[u] = A(0);
      if (ok[u]) {
        int64_t n, i;
        nd_split(p, s0 + u * stride, n, i);
        wv[u] = w ? convert<A, T>(w[t[u]]) : A(1);
        xv[u] = convert<A, T>(x[(n * p.classes + t[u]) * p.inner + i]);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      av -= static_cast<double>(wv[u]) * static_cast<double>(xv[u]);
      aw += static_cast<double>(wv[u]);
    }
  }
  av = warp_sum(av);
  aw = warp_sum(aw);
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = av;
    s_w[threadIdx.x >> 5] = aw;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double v = 0.0, ww = 0.0;
    for (int k = 0; k < 8; ++k) {
      v += s_v[k];
      ww += s_w[k];
    }
    partial[blockIdx.x] = make_double2(v, ww);
  }
}

// Stage 2: one CTA; thread k adds the partials k, k + 256, ..., then a fixed tree (the order never depends on timing).
template <typename T, typename A>
__global__ void __launch_bounds__(256) nd_fwd_final_kernel(const double2* __restrict__ partial, int count, int reduction,
                                                           T* __restrict__ out, T* __restrict__ total_weight) {
  __shared__ double s_v[8];
  __shared__ double s_w[8];
  double v = 0.0, w = 0.0;
  for (int k = threadIdx.x; k < count; k += 256) {
    v += partial[k].x;
    w += partial[k].y;
  }
  v = warp_sum(v);
  w = warp_sum(w);
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = v;
    s_w[threadIdx.x >> 5] = w;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double rv = 0.0, rw = 0.0;
    for (int k = 0; k < 8; ++k) {
      rv += s_v[k];
      rw += s_w[k];
    }
    if (reduction == SB_REDUCTION_MEAN) rv = rv / rw;  // 0/0 = NaN when every sample is ignored
    *out = convert<T, A>(static_cast<A>(rv));
    *total_weight = convert<T, A>(static_cast<A>(rw));
  }
}

// Backward: a CTA owns a tile of 256 * VEC * kBwdUnroll consecutive samples of one outer row; a thread owns kBwdUnroll
// vectors of it, 256 vectors apart, and writes their values in every class plane, so that the CTA writes 16 KB (fp32)
// of contiguous memory per plane.
constexpr int kBwdUnroll = 4;
template <typename T, typename A, int VEC>
__global__ void __launch_bounds__(256) nd_bwd_kernel(NdParams p, const T* __restrict__ grad_output, const T* __restrict__ total_weight,
                                                     T* __restrict__ grad_input, uint32_t tiles_per_row) {
  const T* w = static_cast<const T*>(p.weight);
  A gscale = A(1);
  if (p.reduction != SB_REDUCTION_NONE) {
    gscale = convert<A, T>(grad_output[0]);
    if (p.reduction == SB_REDUCTION_MEAN) gscale = gscale / convert<A, T>(*total_weight);
  }
  const int64_t n = blockIdx.x / tiles_per_row;
  const int64_t tile0 = static_cast<int64_t>(blockIdx.x % tiles_per_row) * (256 * VEC * kBwdUnroll);
  int64_t t[kBwdUnroll][VEC];
  A val[kBwdUnroll][VEC];
  int64_t i0[kBwdUnroll];
#pragma unroll
  for (int u = 0; u < kBwdUnroll; ++u) {
    i0[u] = tile0 + (static_cast<int64_t>(u) * 256 + threadIdx.x) * VEC;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      val[u][k] = A(0);
      t[u][k] = -1;
      if (i0[u] < p.inner) {  // inner is a multiple of VEC: a vector is inside the row or outside it as a whole
        const int64_t s = n * p.inner + i0[u] + k;
        if (nd_counts(p, s, t[u][k])) {
          const A wt = w ? convert<A, T>(w[t[u][k]]) : A(1);
          const A g = p.reduction == SB_REDUCTION_NONE ? convert<A, T>(grad_output[s]) : gscale;
          val[u][k] = -wt * g;
        } else {
          t[u][k] = -1;
        }
      }
    }
  }
  T* row = grad_input + (n * p.classes) * p.inner;
  for (int64_t c = 0; c < p.classes; ++c) {
#pragma unroll
    for (int u = 0; u < kBwdUnroll; ++u) {
      if (i0[u] < p.inner) {
        A o[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = t[u][k] == c ? val[u][k] : A(0);
        store_as<A, T, VEC>(row + c * p.inner + i0[u], o);
      }
    }
  }
}

int nd_validate(const sb_nll_nd_args* a) {
  if (!a || a->outer < 0 || a->classes < 0 || a->inner < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->reduction < SB_REDUCTION_NONE || a->reduction > SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  if (a->target_dtype != SB_I64 && a->target_dtype != SB_U8) return SB_ERR_UNSUPPORTED;
  if (a->dtype != SB_F32 && a->dtype != SB_BF16 && a->dtype != SB_F16 && a->dtype != SB_F64) return SB_ERR_UNSUPPORTED;
  if (a->inner != 0 && a->outer > INT64_MAX / a->inner) return SB_ERR_TOO_LARGE;
  const int64_t samples = a->outer * a->inner;
  if (samples > 0 && (!a->log_probs || !a->target)) return SB_ERR_INVALID_ARGUMENT;
  return SB_OK;
}

NdParams nd_params(const sb_nll_nd_args* a) {
  NdParams p;
  p.x = a->log_probs;
  p.target = a->target;
  p.weight = a->weight;
  p.outer = a->outer;
  p.classes = a->classes;
  p.inner = a->inner;
  p.samples = a->outer * a->inner;
  p.ignore_index = a->ignore_index;
  p.reduction = a->reduction;
  p.target_dtype = a->target_dtype;
  p.status = a->status;
  return p;
}

int nd_partial_ctas(int64_t samples) {
  int64_t ctas = (samples + 1023) / 1024;  // at least four samples per thread
  const int64_t cap = 8LL * sm_count() < kMaxPartials ? 8LL * sm_count() : kMaxPartials;
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  return static_cast<int>(ctas);
}

template <typename T, typename A>
int nd_launch_fwd(const sb_nll_nd_args* a, void* output, void* total_weight, cudaStream_t st) {
  NdParams p = nd_params(a);
  if (a->reduction == SB_REDUCTION_NONE) {
    if (p.samples == 0) return SB_OK;
    const int64_t ctas = (p.samples + 255) / 256;
    const int grid = static_cast<int>(ctas < 16LL * sm_count() ? ctas : 16LL * sm_count());
    nd_fwd_none_kernel<T, A><<<grid, 256, 0, st>>>(p, static_cast<T*>(output));
    return launch_status();
  }
  const int ctas = nd_partial_ctas(p.samples);
  if (!a->scratch || a->scratch_bytes < sizeof(double2) * static_cast<size_t>(ctas)) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(a->scratch) % alignof(double2)) return SB_ERR_MISALIGNED;
  double2* partial = static_cast<double2*>(a->scratch);
  nd_fwd_partial_kernel<T, A><<<ctas, 256, 0, st>>>(p, partial);
  int rc = launch_status();
  if (rc != SB_OK) return rc;
  nd_fwd_final_kernel<T, A><<<1, 256, 0, st>>>(partial, ctas, a->reduction, static_cast<T*>(output), static_cast<T*>(total_weight));
  return launch_status();
}

template <typename T, typename A, int VEC>
int nd_launch_bwd_vec(const NdParams& p, const void* grad_output, const void* total_weight, void* grad_input, cudaStream_t st) {
  const int64_t tile = 256LL * VEC * kBwdUnroll;
  const int64_t tiles_per_row = (p.inner + tile - 1) / tile;
  if (tiles_per_row > 0xffffffffLL || p.outer * tiles_per_row > 0x7fffffffLL) return SB_ERR_TOO_LARGE;
  nd_bwd_kernel<T, A, VEC><<<static_cast<unsigned>(p.outer * tiles_per_row), 256, 0, st>>>(
      p, static_cast<const T*>(grad_output), static_cast<const T*>(total_weight), static_cast<T*>(grad_input),
      static_cast<uint32_t>(tiles_per_row));
  return launch_status();
}

template <typename T, typename A>
int nd_launch_bwd(const sb_nll_nd_args* a, const void* grad_output, const void* total_weight, void* grad_input, cudaStream_t st) {
  NdParams p = nd_params(a);
  if (p.samples == 0 || p.classes == 0) return SB_OK;
  constexpr int kVec = 16 / sizeof(T);
  const bool vec = p.inner % kVec == 0 && reinterpret_cast<uintptr_t>(grad_input) % 16 == 0;
  if (vec) return nd_launch_bwd_vec<T, A, kVec>(p, grad_output, total_weight, grad_input, st);
  return nd_launch_bwd_vec<T, A, 1>(p, grad_output, total_weight, grad_input, st);
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_nll_loss_nd_scratch_bytes(const sb_nll_nd_args* a) {
  if (nd_validate(a) != SB_OK || a->reduction == SB_REDUCTION_NONE) return 0;
  return sizeof(double2) * static_cast<size_t>(nd_partial_ctas(a->outer * a->inner));
}

int sb_nll_loss_nd_forward(const sb_nll_nd_args* a, void* output, void* total_weight, sb_stream_t stream) {
  int rc = nd_validate(a);
  if (rc != SB_OK) return rc;
  if (!output || (a->reduction != SB_REDUCTION_NONE && !total_weight)) return SB_ERR_INVALID_ARGUMENT;
  cudaStream_t st = as_stream(stream);
  switch (a->dtype) {
    case SB_F32: return nd_launch_fwd<float, float>(a, output, total_weight, st);
    case SB_BF16: return nd_launch_fwd<__nv_bfloat16, float>(a, output, total_weight, st);
    case SB_F16: return nd_launch_fwd<__half, float>(a, output, total_weight, st);
    default: return nd_launch_fwd<double, double>(a, output, total_weight, st);
  }
}

int sb_nll_loss_nd_backward(const sb_nll_nd_args* a, const void* grad_output, const void* total_weight, void* grad_input,
                            sb_stream_t stream) {
  int rc = nd_validate(a);
  if (rc != SB_OK) return rc;
  if (a->outer * a->inner > 0 && a->classes > 0 && (!grad_output || !grad_input)) return SB_ERR_INVALID_ARGUMENT;
  if (a->reduction == SB_REDUCTION_MEAN && !total_weight) return SB_ERR_INVALID_ARGUMENT;
  cudaStream_t st = as_stream(stream);
  switch (a->dtype) {
    case SB_F32: return nd_launch_bwd<float, float>(a, grad_output, total_weight, grad_input, st);
    case SB_BF16: return nd_launch_bwd<__nv_bfloat16, float>(a, grad_output, total_weight, grad_input, st);
    case SB_F16: return nd_launch_bwd<__half, float>(a, grad_output, total_weight, grad_input, st);
    default: return nd_launch_bwd<double, double>(a, grad_output, total_weight, grad_input, st);
  }
}

}  // extern "C"

// binary_cross_entropy_with_logits with reduction mean / sum in one pass over the inputs: the unreduced loss
// (1 - t) x + lw * softplus(-x), lw = 1 + (pw - 1) t, times weight, is summed without being written.
//
// The reference materialises the loss tensor and reduces it with a second operator
// (torch_supa/csrc/aten/ops/BinaryCrossEntropyWithLogits.cpp:39-72); fused, the sum costs one read of each input
// and nothing else.  Two fixed-order stages (per-CTA partials in caller scratch, then one thread), so the result is
// bit-reproducible.  Inputs are contiguous and of one dtype; pos_weight, when given, has `pw_len` elements and is
// indexed by (flat index % pw_len), i.e. it runs along the last dimension.
#include "io.cuh"

namespace sb {
namespace {

constexpr int kBceThreads = 256;
constexpr int kBceMaxPartials = 2048;

struct BceParams {
  const void* x;
  const void* t;
  const void* pw;
  const void* w;
  int64_t numel;
  int64_t pw_len;
};

// fp32: softplus(-x) = max(-x, 0) + ln2 * lg2(1 + 2^(-|x| log2 e)) with the hardware ex2 / lg2 (absolute error of the
// logarithm term about 1e-7, far below what a sum of these terms resolves); keeps the pass bound by memory.
__device__ __forceinline__ float bce_term(float x, float t, float lw) {
  float e, l;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-fabsf(x) * 1.4426950408889634f));
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(1.f + e));
  const float sp = fmaf(l, 0.6931471805599453f, fmaxf(-x, 0.f));
  return fmaf(1.f - t, x, lw * sp);
}
__device__ __forceinline__ double bce_term(double x, double t, double lw) {
  const double sp = fmax(-x, 0.0) + log1p(exp(-fabs(x)));
  return (1.0 - t) * x + lw * sp;
}

template <typename T, typename A, int VEC>
__global__ void __launch_bounds__(kBceThreads) bce_partial_kernel(BceParams p, double* __restrict__ partial) {
  __shared__ double s_v[kBceThreads / 32];
  const T* x = static_cast<const T*>(p.x);
  const T* t = static_cast<const T*>(p.t);
  const T* pw = static_cast<const T*>(p.pw);
  const T* w = static_cast<const T*>(p.w);
  const int64_t nvec = p.numel / VEC;
  double acc = 0.0;
  // kU vectors of every input per thread and pass, all loads issued before the arithmetic
  constexpr int kU = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kBceThreads;
  for (int64_t v0 = static_cast<int64_t>(blockIdx.x) * kBceThreads + threadIdx.x; v0 < nvec; v0 += stride * kU) {
    A xv[kU][VEC], tv[kU][VEC], wv[kU][VEC];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = v0 + u * stride;
      if (v < nvec) {
        load_as<A, T, VEC>(x + v * VEC, xv[u]);
        load_as<A, T, VEC>(t + v * VEC, tv[u]);
        if (w) load_as<A, T, VEC>(w + v * VEC, wv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t v = v0 + u * stride;
      if (v < nvec) {
        A part = A(0);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          A lw = A(1);
          if (pw) lw = (convert<A, T>(pw[(v * VEC + k) % p.pw_len]) - A(1)) * tv[u][k] + A(1);
          A term = bce_term(xv[u][k], tv[u][k], lw);
          if (w) term *= wv[u][k];
          part += term;
        }
        acc += static_cast<double>(part);
      }
    }
  }
  // scalar tail, taken by the first threads of the first CTA
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * VEC + threadIdx.x; i < p.numel; i += kBceThreads) {
      const A xi = convert<A, T>(x[i]), ti = convert<A, T>(t[i]);
      A lw = A(1);
      if (pw) lw = (convert<A, T>(pw[i % p.pw_len]) - A(1)) * ti + A(1);
      A term = bce_term(xi, ti, lw);
      if (w) term *= convert<A, T>(w[i]);
      acc += static_cast<double>(term);
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_v[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double v = 0.0;
    for (int k = 0; k < kBceThreads / 32; ++k) v += s_v[k];
    partial[blockIdx.x] = v;
  }
}

// Stage 2: one CTA; thread k adds the partials k, k + 256, ..., then a fixed tree (the order never depends on timing).
template <typename T, typename A>
__global__ void __launch_bounds__(256) bce_final_kernel(const double* __restrict__ partial, int count, int64_t numel, int reduction,
                                                        T* __restrict__ out) {
  __shared__ double s_v[8];
  double v = 0.0;
  for (int k = threadIdx.x; k < count; k += 256) v += partial[k];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) s_v[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double r = 0.0;
    for (int k = 0; k < 8; ++k) r += s_v[k];
    if (reduction == SB_REDUCTION_MEAN) r = r / static_cast<double>(numel);  // 0/0 = NaN for an empty input, as mean() gives
    *out = convert<T, A>(static_cast<A>(r));
  }
}

int bce_ctas(int64_t numel) {
  int64_t ctas = (numel + 8LL * kBceThreads * 4 - 1) / (8LL * kBceThreads * 4);  // about four vectors per thread at least
  const int64_t cap = 12LL * sm_count() < kBceMaxPartials ? 12LL * sm_count() : kBceMaxPartials;
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  return static_cast<int>(ctas);
}

template <typename T, typename A>
int bce_launch(const BceParams& p, int reduction, void* out, void* scratch, cudaStream_t st) {
  const int ctas = bce_ctas(p.numel);
  double* partial = static_cast<double*>(scratch);
  constexpr int kVec = 16 / sizeof(T);
  const bool aligned = reinterpret_cast<uintptr_t>(p.x) % 16 == 0 && reinterpret_cast<uintptr_t>(p.t) % 16 == 0 &&
                       (!p.w || reinterpret_cast<uintptr_t>(p.w) % 16 == 0);
  if (aligned) bce_partial_kernel<T, A, kVec><<<ctas, kBceThreads, 0, st>>>(p, partial);
  else bce_partial_kernel<T, A, 1><<<ctas, kBceThreads, 0, st>>>(p, partial);
  int rc = launch_status();
  if (rc != SB_OK) return rc;
  bce_final_kernel<T, A><<<1, 256, 0, st>>>(partial, ctas, p.numel, reduction, static_cast<T*>(out));
  return launch_status();
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_bce_logits_scratch_bytes(int64_t numel) { return numel < 0 ? 0 : sizeof(double) * static_cast<size_t>(bce_ctas(numel)); }

int sb_bce_logits_reduce(const void* x, const void* target, const void* pos_weight, int64_t pw_len, const void* weight, int32_t dtype,
                         int64_t numel, int32_t reduction, void* out, void* scratch, size_t scratch_bytes, sb_stream_t stream) {
  if (numel < 0 || !out || (numel > 0 && (!x || !target))) return SB_ERR_INVALID_ARGUMENT;
  if (reduction != SB_REDUCTION_MEAN && reduction != SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  if (pos_weight && pw_len <= 0) return SB_ERR_INVALID_ARGUMENT;
  if (!scratch || scratch_bytes < sb_bce_logits_scratch_bytes(numel)) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(scratch) % alignof(double)) return SB_ERR_MISALIGNED;
  BceParams p{x, target, pos_weight, weight, numel, pos_weight ? pw_len : 1};
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case SB_F32: return bce_launch<float, float>(p, reduction, out, scratch, st);
    case SB_BF16: return bce_launch<__nv_bfloat16, float>(p, reduction, out, scratch, st);
    case SB_F16: return bce_launch<__half, float>(p, reduction, out, scratch, st);
    case SB_F64: return bce_launch<double, double>(p, reduction, out, scratch, st);
    default: return SB_ERR_UNSUPPORTED;
  }
}

}  // extern "C"

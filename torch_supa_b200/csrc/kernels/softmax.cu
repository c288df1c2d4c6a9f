// log_softmax forward / backward over one dimension of a tensor viewed as [outer, dim, inner].
//
// inner == 1 (softmax over the last, contiguous dimension): one CTA per row for long rows, one warp
// per row for short ones; the statistics sweep reads the row from HBM, the output sweep re-reads it
// from L1/L2.  inner > 1: one thread per (outer, inner) pair walking the strided dimension, coalesced
// across `inner`.
//
// Arithmetic is fp32 for fp32/bf16/fp16 storage and fp64 for fp64 storage.  Outputs may be wider than
// inputs (the `half_to_float` form of aten::_log_softmax) and input gradients narrower than output
// gradients (its backward).
#include "ce_common.cuh"
#include "io.cuh"

namespace sb {

namespace {

template <typename A> __device__ __forceinline__ A acc_exp(A x);
template <> __device__ __forceinline__ float acc_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double acc_exp<double>(double x) { return exp(x); }
template <typename A> __device__ __forceinline__ A acc_log(A x);
template <> __device__ __forceinline__ float acc_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double acc_log<double>(double x) { return log(x); }
template <typename A> __device__ __forceinline__ A neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -CUDART_INF_F; }
template <> __device__ __forceinline__ double neg_inf<double>() { return -CUDART_INF; }

template <typename A> __device__ __forceinline__ A shfl_xor(A v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }

template <typename A> __device__ __forceinline__ A warp_sum_t(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += shfl_xor(v, o);
  return v;
}
template <typename A> __device__ __forceinline__ A warp_max_t(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    A w = shfl_xor(v, o);
    v = (w > v || w != w) ? w : v;  // NaN wins, as in a max that propagates NaN
  }
  return v;
}

// (max, sum exp) merge with -inf partials kept neutral.
template <typename A> __device__ __forceinline__ void merge_ms(A& m, A& s, A m2, A s2) {
  const A mm = (m2 > m || m2 != m2) ? m2 : m;
  const A a = (m == neg_inf<A>()) ? A(0) : s * acc_exp<A>(m - mm);
  const A b = (m2 == neg_inf<A>()) ? A(0) : s2 * acc_exp<A>(m2 - mm);
  m = mm;
  s = a + b;
}

// Block-wide (max, sum exp) -> every thread; THREADS multiple of 32.
template <typename A, int THREADS>
__device__ __forceinline__ void block_merge_ms(A& m, A& s, A* sm_m, A* sm_s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge_ms(m, s, shfl_xor(m, o), shfl_xor(s, o));
  if (lane == 0) {
    sm_m[warp] = m;
    sm_s[warp] = s;
  }
  __syncthreads();
  A mm = lane < THREADS / 32 ? sm_m[lane] : neg_inf<A>();
  A ss = lane < THREADS / 32 ? sm_s[lane] : A(0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge_ms(mm, ss, shfl_xor(mm, o), shfl_xor(ss, o));
  m = mm;
  s = ss;
  __syncthreads();
}
template <typename A, int THREADS>
__device__ __forceinline__ A block_sum(A v, A* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum_t(v);
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  A r = lane < THREADS / 32 ? sm[lane] : A(0);
  r = warp_sum_t(r);
  __syncthreads();
  return r;
}

// ---- forward, rows -----------------------------------------------------------------------------------------
template <typename Tin, typename Tout, typename A, int VEC, int THREADS, bool LOG>
__global__ void __launch_bounds__(THREADS) lsm_fwd_cta_kernel(const Tin* __restrict__ in, Tout* __restrict__ out,
                                                              int64_t rows, int64_t C) {
  __shared__ A sm_m[32];
  __shared__ A sm_s[32];
  const int64_t nvec = C / VEC;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const Tin* x = in + row * C;
    Tout* y = out + row * C;
    A m = neg_inf<A>(), s = 0;
    for (int64_t i = threadIdx.x; i < nvec; i += THREADS) {
      A f[VEC];
      load_as<A, Tin, VEC>(x + i * VEC, f);
      A vmax = f[0];
#pragma unroll
      for (int k = 1; k < VEC; ++k) vmax = (f[k] > vmax || f[k] != f[k]) ? f[k] : vmax;
      if (vmax > m || vmax != vmax) {
        s *= acc_exp<A>(m - vmax);
        m = vmax;
      }
      const A mm = (m == neg_inf<A>()) ? A(0) : m;
#pragma unroll
      for (int k = 0; k < VEC; ++k) s += acc_exp<A>(f[k] - mm);
    }
    block_merge_ms<A, THREADS>(m, s, sm_m, sm_s);
    const A lse = m + acc_log<A>(s);
    for (int64_t i = threadIdx.x; i < nvec; i += THREADS) {
      A f[VEC];
      load_as<A, Tin, VEC>(x + i * VEC, f);
#pragma unroll
      for (int k = 0; k < VEC; ++k) f[k] = LOG ? f[k] - lse : acc_exp<A>(f[k] - lse);
      store_as<A, Tout, VEC>(y + i * VEC, f);
    }
  }
}

template <typename Tin, typename Tout, typename A, int THREADS, bool LOG>
__global__ void __launch_bounds__(THREADS) lsm_fwd_warp_kernel(const Tin* __restrict__ in, Tout* __restrict__ out,
                                                               int64_t rows, int64_t C) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * (THREADS / 32);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5); row < rows; row += stride) {
    const Tin* x = in + row * C;
    Tout* y = out + row * C;
    A m = neg_inf<A>();
    for (int64_t c = lane; c < C; c += 32) {
      const A f = convert<A, Tin>(x[c]);
      m = (f > m || f != f) ? f : m;
    }
    m = warp_max_t(m);
    const A mm = (m == neg_inf<A>()) ? A(0) : m;
    A s = 0;
    for (int64_t c = lane; c < C; c += 32) s += acc_exp<A>(convert<A, Tin>(x[c]) - mm);
    s = warp_sum_t(s);
    const A lse = m + acc_log<A>(s);
    for (int64_t c = lane; c < C; c += 32) {
      const A d = convert<A, Tin>(x[c]) - lse;
      y[c] = convert<Tout, A>(LOG ? d : acc_exp<A>(d));
    }
  }
}

// ---- forward, strided dimension --------------------------------------------------------------------------
template <typename Tin, typename Tout, typename A, bool LOG>
__global__ void __launch_bounds__(256) lsm_fwd_strided_kernel(const Tin* __restrict__ in, Tout* __restrict__ out,
                                                              int64_t outer, int64_t D, int64_t inner) {
  const int64_t total = outer * inner;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t o = idx / inner, i = idx - o * inner;
    const Tin* x = in + o * D * inner + i;
    Tout* y = out + o * D * inner + i;
    A m = neg_inf<A>();
    for (int64_t d = 0; d < D; ++d) {
      const A f = convert<A, Tin>(x[d * inner]);
      m = (f > m || f != f) ? f : m;
    }
    const A mm = (m == neg_inf<A>()) ? A(0) : m;
    A s = 0;
    for (int64_t d = 0; d < D; ++d) s += acc_exp<A>(convert<A, Tin>(x[d * inner]) - mm);
    const A lse = m + acc_log<A>(s);
    for (int64_t d = 0; d < D; ++d) {
      const A v = convert<A, Tin>(x[d * inner]) - lse;
      y[d * inner] = convert<Tout, A>(LOG ? v : acc_exp<A>(v));
    }
  }
}

// ---- backward: log_softmax: grad_in = g - exp(y) * sum(g);  softmax: grad_in = y * (g - sum(g * y)) -------
// The row of g is read twice (for the sum, then for the result).  The first read asks L2 to keep the lines (evict_last),
// the second one and the single read of y release them (evict_first): with several hundred rows of 100 KB and more in flight
// next to the streams of y and of the result, the second read of g otherwise misses L2 for part of the row.
template <typename A, typename T, int VEC>
__device__ __forceinline__ void load_hinted(const T* p, A (&out)[VEC], uint64_t policy) {
  if constexpr (sizeof(T) * VEC == 16) {
    const uint4 raw = ld_hint_u4(p, policy);
    load_as<A, T, VEC>(&raw, out);
  } else {
    load_as<A, T, VEC>(p, out);
  }
}

template <typename T, typename Tgi, typename A, int VEC, int THREADS, bool LOG>
__global__ void __launch_bounds__(THREADS) lsm_bwd_cta_kernel(const T* __restrict__ gout, const T* __restrict__ yout,
                                                              Tgi* __restrict__ gin, int64_t rows, int64_t C) {
  __shared__ A sm[32];
  const int64_t nvec = C / VEC;
  const uint64_t keep = l2_policy_keep(), stream = l2_policy_stream();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* g = gout + row * C;
    const T* y = yout + row * C;
    Tgi* o = gin + row * C;
    A acc = 0;
    for (int64_t i = threadIdx.x; i < nvec; i += THREADS) {
      A f[VEC];
      load_hinted<A, T, VEC>(g + i * VEC, f, keep);
      if (LOG) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc += f[k];
      } else {
        A yy[VEC];
        load_hinted<A, T, VEC>(y + i * VEC, yy, keep);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc += f[k] * yy[k];
      }
    }
    const A sum = block_sum<A, THREADS>(acc, sm);
    for (int64_t i = threadIdx.x; i < nvec; i += THREADS) {
      A f[VEC], yy[VEC];
      load_hinted<A, T, VEC>(g + i * VEC, f, stream);
      load_hinted<A, T, VEC>(y + i * VEC, yy, stream);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        // 16-bit results: the approximate exponential (2 ulp of fp32) is far inside the rounding of the result
        if constexpr (LOG && sizeof(Tgi) == 2 && std::is_same<A, float>::value) f[k] = f[k] - exp_fast(yy[k]) * sum;
        else f[k] = LOG ? f[k] - acc_exp<A>(yy[k]) * sum : yy[k] * (f[k] - sum);
      }
      store_as<A, Tgi, VEC>(o + i * VEC, f);
    }
  }
}

// Short rows (up to 1024 elements) with 16-byte aligned pitch: a warp (or 16 / 8 lanes of one, for rows of up to 16 / 8
// vectors) per row, 16-byte accesses, the row of g held in registers between the sum and the result (one read of g, one of
// y, one write).
template <typename T, typename Tgi, typename A, int VEC, int LPR, int NIT, bool LOG>
__global__ void __launch_bounds__(256) lsm_bwd_warp_vec_kernel(const T* __restrict__ gout, const T* __restrict__ yout,
                                                               Tgi* __restrict__ gin, int64_t rows, int64_t D) {
  // LPR lanes per row, up to NIT vectors per lane
  constexpr int kSubs = 32 / LPR;
  const int lane = threadIdx.x & 31, sub = lane / LPR, sl = lane % LPR;
  const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << (LPR & 31)) - 1u) << (LPR * sub));
  const int nvec = static_cast<int>(D / VEC);
  const int64_t first = (static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kSubs + sub;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 8 * kSubs;
  for (int64_t row = first; row < rows; row += stride) {
    const T* g = gout + row * D;
    const T* y = yout + row * D;
    Tgi* o = gin + row * D;
    A gv[NIT][VEC], yv[NIT][VEC];
    A acc = 0;
#pragma unroll
    for (int n = 0; n < NIT; ++n) {
      const int v = sl + LPR * n;
      if (v < nvec) {
        load_as<A, T, VEC>(g + v * VEC, gv[n]);
        load_as<A, T, VEC>(y + v * VEC, yv[n]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc += LOG ? gv[n][k] : gv[n][k] * yv[n][k];
      }
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(gmask, acc, off);
#pragma unroll
    for (int n = 0; n < NIT; ++n) {
      const int v = sl + LPR * n;
      if (v < nvec) {
        A r[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          if constexpr (LOG && sizeof(Tgi) == 2 && std::is_same<A, float>::value) r[k] = gv[n][k] - exp_fast(yv[n][k]) * acc;
          else r[k] = LOG ? gv[n][k] - acc_exp<A>(yv[n][k]) * acc : yv[n][k] * (gv[n][k] - acc);
        }
        store_as<A, Tgi, VEC>(o + v * VEC, r);
      }
    }
  }
}

template <typename T, typename Tgi, typename A, bool LOG>
__global__ void __launch_bounds__(256) lsm_bwd_strided_kernel(const T* __restrict__ gout, const T* __restrict__ yout,
                                                              Tgi* __restrict__ gin, int64_t outer, int64_t D,
                                                              int64_t inner, bool warp_rows) {
  if (warp_rows) {  // inner == 1 and short rows: one warp per row
    const int lane = threadIdx.x & 31;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 8;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < outer; row += stride) {
      const T* g = gout + row * D;
      const T* y = yout + row * D;
      Tgi* o = gin + row * D;
      A acc = 0;
      for (int64_t c = lane; c < D; c += 32) acc += LOG ? convert<A, T>(g[c]) : convert<A, T>(g[c]) * convert<A, T>(y[c]);
      acc = warp_sum_t(acc);
      for (int64_t c = lane; c < D; c += 32) {
        const A gv = convert<A, T>(g[c]), yv = convert<A, T>(y[c]);
        o[c] = convert<Tgi, A>(LOG ? gv - acc_exp<A>(yv) * acc : yv * (gv - acc));
      }
    }
    return;
  }
  const int64_t total = outer * inner;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t o_ = idx / inner, i = idx - o_ * inner;
    const int64_t base = o_ * D * inner + i;
    A acc = 0;
    for (int64_t d = 0; d < D; ++d)
      acc += LOG ? convert<A, T>(gout[base + d * inner]) : convert<A, T>(gout[base + d * inner]) * convert<A, T>(yout[base + d * inner]);
    for (int64_t d = 0; d < D; ++d) {
      const A gv = convert<A, T>(gout[base + d * inner]), yv = convert<A, T>(yout[base + d * inner]);
      gin[base + d * inner] = convert<Tgi, A>(LOG ? gv - acc_exp<A>(yv) * acc : yv * (gv - acc));
    }
  }
}

template <typename Tin, typename Tout, typename A, bool LOG>
int launch_fwd(const void* in, void* out, int64_t outer, int64_t D, int64_t inner, cudaStream_t st) {
  const Tin* x = static_cast<const Tin*>(in);
  Tout* y = static_cast<Tout*>(out);
  const int sms = sm_count();
  if (inner == 1 && std::is_same<Tin, Tout>::value && sizeof(Tin) <= 4) {
    // one HBM read, one HBM write: aligned rows of up to 32 KB on the slot ring (groups of rows, a warp or a team per row),
    // long rows resident in shared memory chunk by chunk
    int rc = lsm_launch_ring(in, out, DTypeOf<Tin>::value, outer, D, LOG ? 1 : 2, st);
    if (rc != SB_ERR_UNSUPPORTED) return rc;
    rc = lsm_launch_resident(in, out, DTypeOf<Tin>::value, outer, D, LOG ? 1 : 2, st);
    if (rc != SB_ERR_UNSUPPORTED) return rc;
  }
  if (inner == 1) {
    if (D <= 1024) {
      const int64_t ctas = (outer + 7) / 8;
      const int grid = static_cast<int>(ctas < 8LL * sms ? ctas : 8LL * sms);
      lsm_fwd_warp_kernel<Tin, Tout, A, 256, LOG><<<grid, 256, 0, st>>>(x, y, outer, D);
      return launch_status();
    }
    constexpr int kVec = 16 / sizeof(Tin);
    constexpr int kThreads = 512;
    const int grid = static_cast<int>(outer < 4LL * sms ? outer : 4LL * sms);
    const size_t out_align = sizeof(Tout) * kVec >= 16 ? 16 : sizeof(Tout) * kVec;
    const bool aligned = D % kVec == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(out) % out_align == 0;
    if (aligned) lsm_fwd_cta_kernel<Tin, Tout, A, kVec, kThreads, LOG><<<grid, kThreads, 0, st>>>(x, y, outer, D);
    else lsm_fwd_cta_kernel<Tin, Tout, A, 1, kThreads, LOG><<<grid, kThreads, 0, st>>>(x, y, outer, D);
    return launch_status();
  }
  const int64_t total = outer * inner;
  const int64_t ctas = (total + 255) / 256;
  const int grid = static_cast<int>(ctas < 16LL * sms ? ctas : 16LL * sms);
  lsm_fwd_strided_kernel<Tin, Tout, A, LOG><<<grid, 256, 0, st>>>(x, y, outer, D, inner);
  return launch_status();
}

template <typename T, typename Tgi, typename A, bool LOG>
int launch_bwd(const void* gout, const void* yout, void* gin, int64_t outer, int64_t D, int64_t inner, cudaStream_t st) {
  const T* g = static_cast<const T*>(gout);
  const T* y = static_cast<const T*>(yout);
  Tgi* o = static_cast<Tgi*>(gin);
  const int sms = sm_count();
  if (inner == 1 && D > 1024) {
    constexpr int kVec = 16 / sizeof(T);
    const size_t gi_align = sizeof(Tgi) * kVec >= 16 ? 16 : sizeof(Tgi) * kVec;
    const bool aligned = D % kVec == 0 && reinterpret_cast<uintptr_t>(gout) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(yout) % 16 == 0 && reinterpret_cast<uintptr_t>(gin) % gi_align == 0;
    // The rows being re-read should stay a fraction of L2 (126 MB): four CTAs of 512 threads per SM up to 96 MB of them in
    // flight (fp32 [16384,32000]: 0.87 of the copy peak, against 0.83 with two larger CTAs), two CTAs of 1024 threads beyond
    // (bf16 [8192,128256], rows of 256 KB: 0.85 against 0.80).
    if (aligned && 4.0 * sms * static_cast<double>(D) * sizeof(T) > 96.0 * 1024 * 1024) {
      constexpr int kBig = 1024;
      const int grid = static_cast<int>(outer < 2LL * sms ? outer : 2LL * sms);
      lsm_bwd_cta_kernel<T, Tgi, A, kVec, kBig, LOG><<<grid, kBig, 0, st>>>(g, y, o, outer, D);
      return launch_status();
    }
    constexpr int kThreads = 512;
    const int grid = static_cast<int>(outer < 4LL * sms ? outer : 4LL * sms);
    if (aligned) lsm_bwd_cta_kernel<T, Tgi, A, kVec, kThreads, LOG><<<grid, kThreads, 0, st>>>(g, y, o, outer, D);
    else lsm_bwd_cta_kernel<T, Tgi, A, 1, kThreads, LOG><<<grid, kThreads, 0, st>>>(g, y, o, outer, D);
    return launch_status();
  }
  if (inner == 1 && D <= 1024 && sizeof(T) <= 4) {
    constexpr int kVec = 16 / sizeof(T);
    const size_t gi_align = sizeof(Tgi) * kVec >= 16 ? 16 : sizeof(Tgi) * kVec;
    const bool aligned = D % kVec == 0 && reinterpret_cast<uintptr_t>(gout) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(yout) % 16 == 0 && reinterpret_cast<uintptr_t>(gin) % gi_align == 0;
    if (aligned) {
      const int64_t nvec = D / kVec;
      // rows per warp: as many as leave each lane two to four vectors (more rows in flight hide more latency)
      int lpr, nit;
      if (nvec <= 16) lpr = 8, nit = 2;
      else if (nvec <= 32) lpr = 16, nit = 2;
      else if (nvec <= 64) lpr = 16, nit = 4;
      else if (nvec <= 128) lpr = 32, nit = 4;
      else lpr = 32, nit = 8;
      const int64_t per_cta = 8 * (32 / lpr);
      const int64_t ctas = (outer + per_cta - 1) / per_cta;
      const int grid = static_cast<int>(ctas < 16LL * sms ? ctas : 16LL * sms);
      if (lpr == 8) lsm_bwd_warp_vec_kernel<T, Tgi, A, kVec, 8, 2, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D);
      else if (lpr == 16 && nit == 2) lsm_bwd_warp_vec_kernel<T, Tgi, A, kVec, 16, 2, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D);
      else if (lpr == 16) lsm_bwd_warp_vec_kernel<T, Tgi, A, kVec, 16, 4, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D);
      else if (nit == 4) lsm_bwd_warp_vec_kernel<T, Tgi, A, kVec, 32, 4, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D);
      else lsm_bwd_warp_vec_kernel<T, Tgi, A, kVec, 32, 8, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D);
      return launch_status();
    }
  }
  const bool warp_rows = inner == 1;
  const int64_t total = warp_rows ? (outer + 7) / 8 : (outer * inner + 255) / 256;
  const int grid = static_cast<int>(total < 16LL * sms ? total : 16LL * sms);
  lsm_bwd_strided_kernel<T, Tgi, A, LOG><<<grid, 256, 0, st>>>(g, y, o, outer, D, inner, warp_rows);
  return launch_status();
}

}  // namespace
}  // namespace sb

using namespace sb;

namespace {

template <bool LOG>
int softmax_forward_any(const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t outer, int64_t dim, int64_t inner,
                        sb_stream_t stream) {
  if (outer < 0 || dim < 0 || inner < 0) return SB_ERR_INVALID_ARGUMENT;
  if (outer == 0 || dim == 0 || inner == 0) return SB_OK;
  if (!in || !out) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(in) % dtype_size(in_dtype) || reinterpret_cast<uintptr_t>(out) % dtype_size(out_dtype))
    return SB_ERR_MISALIGNED;
  cudaStream_t st = as_stream(stream);
  if (in_dtype == SB_F32 && out_dtype == SB_F32) return launch_fwd<float, float, float, LOG>(in, out, outer, dim, inner, st);
  if (in_dtype == SB_BF16 && out_dtype == SB_BF16)
    return launch_fwd<__nv_bfloat16, __nv_bfloat16, float, LOG>(in, out, outer, dim, inner, st);
  if (in_dtype == SB_F16 && out_dtype == SB_F16) return launch_fwd<__half, __half, float, LOG>(in, out, outer, dim, inner, st);
  if (in_dtype == SB_BF16 && out_dtype == SB_F32) return launch_fwd<__nv_bfloat16, float, float, LOG>(in, out, outer, dim, inner, st);
  if (in_dtype == SB_F16 && out_dtype == SB_F32) return launch_fwd<__half, float, float, LOG>(in, out, outer, dim, inner, st);
  if (in_dtype == SB_F64 && out_dtype == SB_F64) return launch_fwd<double, double, double, LOG>(in, out, outer, dim, inner, st);
  return SB_ERR_UNSUPPORTED;
}

template <bool LOG>
int softmax_backward_any(const void* grad_out, const void* out, int32_t dtype, void* grad_in, int32_t grad_in_dtype, int64_t outer,
                         int64_t dim, int64_t inner, sb_stream_t stream) {
  if (outer < 0 || dim < 0 || inner < 0) return SB_ERR_INVALID_ARGUMENT;
  if (outer == 0 || dim == 0 || inner == 0) return SB_OK;
  if (!grad_out || !out || !grad_in) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(grad_out) % dtype_size(dtype) || reinterpret_cast<uintptr_t>(out) % dtype_size(dtype) ||
      reinterpret_cast<uintptr_t>(grad_in) % dtype_size(grad_in_dtype))
    return SB_ERR_MISALIGNED;
  cudaStream_t st = as_stream(stream);
  if (dtype == SB_F32 && grad_in_dtype == SB_F32) return launch_bwd<float, float, float, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  if (dtype == SB_BF16 && grad_in_dtype == SB_BF16)
    return launch_bwd<__nv_bfloat16, __nv_bfloat16, float, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  if (dtype == SB_F16 && grad_in_dtype == SB_F16) return launch_bwd<__half, __half, float, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  if (dtype == SB_F32 && grad_in_dtype == SB_BF16)
    return launch_bwd<float, __nv_bfloat16, float, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  if (dtype == SB_F32 && grad_in_dtype == SB_F16) return launch_bwd<float, __half, float, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  if (dtype == SB_F64 && grad_in_dtype == SB_F64) return launch_bwd<double, double, double, LOG>(grad_out, out, grad_in, outer, dim, inner, st);
  return SB_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

int sb_log_softmax_forward(const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t outer, int64_t dim,
                           int64_t inner, sb_stream_t stream) {
  return softmax_forward_any<true>(in, in_dtype, out, out_dtype, outer, dim, inner, stream);
}
int sb_log_softmax_backward(const void* grad_out, const void* out, int32_t dtype, void* grad_in, int32_t grad_in_dtype,
                            int64_t outer, int64_t dim, int64_t inner, sb_stream_t stream) {
  return softmax_backward_any<true>(grad_out, out, dtype, grad_in, grad_in_dtype, outer, dim, inner, stream);
}
int sb_softmax_forward(const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t outer, int64_t dim, int64_t inner,
                       sb_stream_t stream) {
  return softmax_forward_any<false>(in, in_dtype, out, out_dtype, outer, dim, inner, stream);
}
int sb_softmax_backward(const void* grad_out, const void* out, int32_t dtype, void* grad_in, int32_t grad_in_dtype, int64_t outer,
                        int64_t dim, int64_t inner, sb_stream_t stream) {
  return softmax_backward_any<false>(grad_out, out, dtype, grad_in, grad_in_dtype, outer, dim, inner, stream);
}

}  // extern "C"

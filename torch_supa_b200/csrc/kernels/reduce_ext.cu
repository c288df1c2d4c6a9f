// Reductions whose running state is more than one number: max / min with the index of the extremum (argmax, argmin,
// max.dim, min.dim) and variance / standard deviation (with the mean).  The tensor is seen as [outer, L, inner],
// contiguous, reduced over L, the view the softmax kernels use too.
//
//   inner == 1   rows: a CTA (or, with few rows, several CTAs per row, each on a segment, folded by a second kernel in
//                a fixed order) strides over the row with coalesced loads;
//   inner  > 1   columns: one thread per (outer, inner) position walks L, neighbouring threads read neighbouring
//                addresses.
//
// Index rules are those of PyTorch's CPU kernels, which the reference's tests take as golden: of equal extrema the
// lowest index wins; NaN beats every number for max AND for min, and of several NaN the first.  Variance follows
// var(correction): M2 / max(0, n - correction), accumulated in fp64 as shifted sums (shift = the row's first element).
#include <type_traits>

#include "io.cuh"

namespace sb {

namespace {

struct ExtParams {
  const void* in;
  void* out0;      // values (arg reduce, may be null) / variance or standard deviation
  void* out1;      // indices as int64 (arg reduce, may be null) / mean (may be null)
  int in_dtype, out_dtype;
  int64_t outer, L, inner;
  int64_t seg;     // rows path: elements per segment
  int nseg;
  void* scratch;   // rows path with nseg > 1: nseg partial states per row
  double correction;
  int take_sqrt;
};

// ---- states ------------------------------------------------------------------------------------------------
template <typename A> struct ArgState {
  A v;
  int64_t i;
};

template <typename A, bool IS_MAX> struct ArgOp {
  using State = ArgState<A>;
  using Acc = A;
  __device__ static __forceinline__ bool is_nan(A x) {
    if constexpr (std::is_floating_point<A>::value) return x != x;
    else return false;
  }
  // a (at index ia) wins over b (at index ib)
  __device__ static __forceinline__ bool wins(A a, int64_t ia, A b, int64_t ib) {
    if (ib < 0) return ia >= 0;
    if (ia < 0) return false;
    const bool na = is_nan(a), nb = is_nan(b);
    if (na || nb) return na && (!nb || ia < ib);
    if (a != b) return IS_MAX ? a > b : a < b;
    return ia < ib;
  }
  __device__ static __forceinline__ State init(A) { return State{A(0), -1}; }  // index -1: nothing seen yet
  __device__ static __forceinline__ State neutral_like(const State&) { return State{A(0), -1}; }
  __device__ static __forceinline__ void fold(State& s, A x, int64_t idx) {
    if (wins(x, idx, s.v, s.i)) {
      s.v = x;
      s.i = idx;
    }
  }
  __device__ static __forceinline__ void merge(State& s, const State& o) {
    if (wins(o.v, o.i, s.v, s.i)) s = o;
  }
  __device__ static __forceinline__ State shfl(const State& s, int o) {
    State r;
    if constexpr (sizeof(A) == 4) r.v = __shfl_down_sync(0xffffffffu, s.v, o);
    else r.v = shfl64(s.v, o);
    r.i = static_cast<int64_t>(__shfl_down_sync(0xffffffffu, static_cast<long long>(s.i), o));
    return r;
  }
  __device__ static __forceinline__ A shfl64(A v, int o) {
    long long bits;
    memcpy(&bits, &v, 8);
    bits = __shfl_down_sync(0xffffffffu, bits, o);
    A r;
    memcpy(&r, &bits, 8);
    return r;
  }
  __device__ static __forceinline__ void finish(const ExtParams& p, const State& s, int64_t out_index) {
    if (p.out0) {
      A v[1] = {s.v};
      DynamicIO::store<A, 1>(p.out0, out_index, p.out_dtype, v);
    }
    if (p.out1) static_cast<int64_t*>(p.out1)[out_index] = s.i;
  }
};

struct MomentState {
  double s1, s2;  // sums of (x - shift) and of its square
  double shift;
};
struct MomentOp {
  using State = MomentState;
  using Acc = double;
  __device__ static __forceinline__ State init(double first) { return State{0.0, 0.0, first}; }
  __device__ static __forceinline__ State neutral_like(const State& s) { return State{0.0, 0.0, s.shift}; }
  __device__ static __forceinline__ void fold(State& s, double x, int64_t) {
    const double d = x - s.shift;
    s.s1 += d;
    s.s2 = fma(d, d, s.s2);
  }
  __device__ static __forceinline__ void merge(State& s, const State& o) {  // every partial of a row uses the same shift
    s.s1 += o.s1;
    s.s2 += o.s2;
  }
  __device__ static __forceinline__ State shfl(const State& s, int o) {
    return State{__shfl_down_sync(0xffffffffu, s.s1, o), __shfl_down_sync(0xffffffffu, s.s2, o), s.shift};
  }
  __device__ static __forceinline__ void finish(const ExtParams& p, const State& s, int64_t out_index) {
    const double n = static_cast<double>(p.L);
    double m2 = s.s2 - s.s1 * s.s1 / n;
    if (m2 < 0.0) m2 = 0.0;  // rounding of a constant row
    const double denom = fmax(0.0, n - p.correction);
    double v = m2 / denom;   // n <= correction: inf or NaN, as on the CPU
    if (p.take_sqrt) v = sqrt(v);
    double o[1] = {v};
    DynamicIO::store<double, 1>(p.out0, out_index, p.out_dtype, o);
    if (p.out1) {
      double mean[1] = {s.shift + s.s1 / n};
      DynamicIO::store<double, 1>(p.out1, out_index, p.out_dtype, mean);
    }
  }
};

template <class Op> __device__ __forceinline__ typename Op::State warp_fold(typename Op::State s) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const typename Op::State other = Op::shfl(s, o);
    Op::merge(s, other);
  }
  return s;  // valid in lane 0
}

// ---- rows: grid (nseg, outer) ----------------------------------------------------------------------------------
template <class Op, int THREADS>
__global__ void __launch_bounds__(THREADS) ext_rows_kernel(ExtParams p) {
  using A = typename Op::Acc;
  using State = typename Op::State;
  __shared__ State sm[THREADS / 32];
  const int64_t row = blockIdx.y;
  const int64_t base = row * p.L;
  A first[1];
  DynamicIO::load<A, 1>(p.in, base, p.in_dtype, first);
  State s = Op::init(first[0]);
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * p.seg;
  int64_t end = begin + p.seg;
  if (end > p.L) end = p.L;
  constexpr int kUnroll = 4;
  int64_t e = begin + threadIdx.x;
  for (; e + static_cast<int64_t>(kUnroll - 1) * THREADS < end; e += static_cast<int64_t>(kUnroll) * THREADS) {
    A x[kUnroll][1];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) DynamicIO::load<A, 1>(p.in, base + e + static_cast<int64_t>(u) * THREADS, p.in_dtype, x[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) Op::fold(s, x[u][0], e + static_cast<int64_t>(u) * THREADS);
  }
  for (; e < end; e += THREADS) {
    A x[1];
    DynamicIO::load<A, 1>(p.in, base + e, p.in_dtype, x);
    Op::fold(s, x[0], e);
  }
  s = warp_fold<Op>(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    State t = threadIdx.x < THREADS / 32 ? sm[threadIdx.x] : Op::init(first[0]);  // init() is the neutral state of the row
    t = warp_fold<Op>(t);
    if (threadIdx.x == 0) {
      if (p.nseg == 1) Op::finish(p, t, row);
      else static_cast<State*>(p.scratch)[row * p.nseg + blockIdx.x] = t;
    }
  }
}

// One warp per row folds the segment partials in segment order.
template <class Op>
__global__ void __launch_bounds__(256) ext_rows_final_kernel(ExtParams p) {
  using State = typename Op::State;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= p.outer) return;
  const State* part = static_cast<const State*>(p.scratch) + row * p.nseg;
  // lanes hold partials lane, lane + 32, ...; lanes beyond nseg start from the neutral state
  State s = lane < p.nseg ? part[lane] : Op::neutral_like(part[0]);
  for (int k = lane + 32; k < p.nseg; k += 32) Op::merge(s, part[k]);
  s = warp_fold<Op>(s);
  if (lane == 0) Op::finish(p, s, row);
}

// ---- columns: one thread per (outer, inner) ----------------------------------------------------------------------
template <class Op>
__global__ void __launch_bounds__(256) ext_cols_kernel(ExtParams p) {
  using A = typename Op::Acc;
  const int64_t total = p.outer * p.inner;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; c < total; c += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t o = c / p.inner, i = c - o * p.inner;
    const int64_t base = o * p.L * p.inner + i;
    A first[1];
    DynamicIO::load<A, 1>(p.in, base, p.in_dtype, first);
    typename Op::State s = Op::init(first[0]);
    for (int64_t e = 0; e < p.L; ++e) {
      A x[1];
      DynamicIO::load<A, 1>(p.in, base + e * p.inner, p.in_dtype, x);
      Op::fold(s, x[0], e);
    }
    Op::finish(p, s, c);
  }
}

// Segments per row: enough CTAs to occupy the GPU when there are few rows, none shorter than 4096 elements.
int plan_segments(int64_t outer, int64_t L, int64_t* seg) {
  int nseg = 1;
  const int64_t target_ctas = 2LL * sm_count();
  if (outer < target_ctas && L >= 8192) {
    int64_t want = (target_ctas + outer - 1) / outer;
    const int64_t by_len = L / 4096;
    if (want > by_len) want = by_len;
    if (want > 1024) want = 1024;
    if (want >= 2) nseg = static_cast<int>(want);
  }
  *seg = (L + nseg - 1) / nseg;
  nseg = static_cast<int>((L + *seg - 1) / *seg);
  return nseg;
}

template <class Op>
int launch_ext(ExtParams p, cudaStream_t st) {
  if (p.inner == 1) {
    if (p.outer > 65535) {  // gridDim.y limit: treat the rows as columns of an [1, L, outer]-like walk is wrong; fold in slabs
      for (int64_t r0 = 0; r0 < p.outer; r0 += 65535) {
        ExtParams q = p;
        const int64_t n = p.outer - r0 < 65535 ? p.outer - r0 : 65535;
        q.outer = n;
        q.in = static_cast<const char*>(p.in) + r0 * p.L * dtype_size(p.in_dtype);
        if (p.out0) q.out0 = static_cast<char*>(p.out0) + r0 * dtype_size(p.out_dtype);
        if (p.out1) q.out1 = static_cast<char*>(p.out1) + r0 * (std::is_same<Op, MomentOp>::value ? dtype_size(p.out_dtype) : 8);
        q.nseg = 1;
        q.seg = q.L;
        ext_rows_kernel<Op, 256><<<dim3(1, static_cast<unsigned>(n)), 256, 0, st>>>(q);
        if (launch_status() != SB_OK) return SB_ERR_CUDA;
      }
      return SB_OK;
    }
    ext_rows_kernel<Op, 256><<<dim3(p.nseg, static_cast<unsigned>(p.outer)), 256, 0, st>>>(p);
    if (launch_status() != SB_OK) return SB_ERR_CUDA;
    if (p.nseg > 1) {
      ext_rows_final_kernel<Op><<<static_cast<unsigned>((p.outer + 7) / 8), 256, 0, st>>>(p);
      return launch_status();
    }
    return SB_OK;
  }
  const int64_t total = p.outer * p.inner;
  int64_t ctas = (total + 255) / 256;
  const int64_t cap = 32LL * sm_count();
  if (ctas > cap) ctas = cap;
  ext_cols_kernel<Op><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p);
  return launch_status();
}

int acc_kind(int dtype) {
  switch (dtype) {
    case SB_F16: case SB_BF16: case SB_F32: return 0;
    case SB_F64: return 1;
    case SB_BOOL: case SB_U8: case SB_I8: case SB_I16: case SB_I32: case SB_I64: return 2;
    default: return -1;
  }
}

size_t state_bytes(bool moments, int kind) {
  if (moments) return sizeof(MomentState);
  return kind == 0 ? sizeof(ArgState<float>) : sizeof(ArgState<double>);  // int64 states have the size of double ones
}

int fill_params(ExtParams* p, const void* in, int dtype, int64_t outer, int64_t L, int64_t inner, void* scratch, size_t scratch_bytes,
                bool moments) {
  if (outer < 0 || L < 0 || inner < 0) return SB_ERR_INVALID_ARGUMENT;
  const int kind = acc_kind(dtype);
  if (kind < 0) return SB_ERR_UNSUPPORTED;
  if (outer * inner > 0 && L > 0 && !in) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(in) % dtype_size(dtype)) return SB_ERR_MISALIGNED;
  p->in = in;
  p->in_dtype = dtype;
  p->outer = outer;
  p->L = L;
  p->inner = inner;
  p->nseg = 1;
  p->seg = L;
  p->scratch = nullptr;
  if (inner == 1 && outer > 0 && outer <= 65535 && L > 0) {
    p->nseg = plan_segments(outer, L, &p->seg);
    if (p->nseg > 1) {
      const size_t need = static_cast<size_t>(outer) * p->nseg * state_bytes(moments, kind);
      if (!scratch || scratch_bytes < need) return SB_ERR_INVALID_ARGUMENT;
      if (reinterpret_cast<uintptr_t>(scratch) % 8) return SB_ERR_MISALIGNED;
      p->scratch = scratch;
    }
  }
  return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_reduce_ext_scratch_bytes(int32_t dtype, int64_t outer, int64_t L, int64_t inner, int32_t moments) {
  if (inner != 1 || outer <= 0 || outer > 65535 || L <= 0) return 0;
  const int kind = acc_kind(dtype);
  if (kind < 0) return 0;
  int64_t seg = 0;
  const int nseg = plan_segments(outer, L, &seg);
  return nseg > 1 ? static_cast<size_t>(outer) * nseg * state_bytes(moments != 0, kind) : 0;
}

int sb_arg_reduce(const void* in, int32_t dtype, int64_t outer, int64_t L, int64_t inner, int32_t is_max, void* values,
                  int64_t* indices, void* scratch, size_t scratch_bytes, sb_stream_t stream) {
  ExtParams p{};
  int rc = fill_params(&p, in, dtype, outer, L, inner, scratch, scratch_bytes, false);
  if (rc != SB_OK) return rc;
  if (outer * inner == 0) return SB_OK;
  if (L == 0) return SB_ERR_INVALID_ARGUMENT;  // no extremum of an empty run (the caller raises, as the CPU does)
  if (!values && !indices) return SB_ERR_INVALID_ARGUMENT;
  p.out0 = values;
  p.out1 = indices;
  p.out_dtype = dtype;
  cudaStream_t st = as_stream(stream);
  switch (acc_kind(dtype)) {
    case 0: return is_max ? launch_ext<ArgOp<float, true>>(p, st) : launch_ext<ArgOp<float, false>>(p, st);
    case 1: return is_max ? launch_ext<ArgOp<double, true>>(p, st) : launch_ext<ArgOp<double, false>>(p, st);
    default: return is_max ? launch_ext<ArgOp<int64_t, true>>(p, st) : launch_ext<ArgOp<int64_t, false>>(p, st);
  }
}

int sb_moments(const void* in, int32_t dtype, int64_t outer, int64_t L, int64_t inner, double correction, int32_t take_sqrt, void* out,
               void* mean_out, void* scratch, size_t scratch_bytes, sb_stream_t stream) {
  if (dtype != SB_F16 && dtype != SB_BF16 && dtype != SB_F32 && dtype != SB_F64) return SB_ERR_UNSUPPORTED;
  ExtParams p{};
  int rc = fill_params(&p, in, dtype, outer, L, inner, scratch, scratch_bytes, true);
  if (rc != SB_OK) return rc;
  if (outer * inner == 0) return SB_OK;
  if (!out) return SB_ERR_INVALID_ARGUMENT;
  if (L == 0) return SB_ERR_INVALID_ARGUMENT;  // the caller fills NaN for an empty run
  p.out0 = out;
  p.out1 = mean_out;
  p.out_dtype = dtype;
  p.correction = correction;
  p.take_sqrt = take_sqrt;
  return launch_ext<MomentOp>(p, as_stream(stream));
}

}  // extern "C"

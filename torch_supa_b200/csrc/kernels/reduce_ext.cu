// Reductions whose running state is more than one number: max / min with the index of the extremum (argmax, argmin,
// max.dim, min.dim) and variance / standard deviation (with the mean).  The tensor is seen as [outer, L, inner],
// contiguous, reduced over L, the view the softmax kernels use too.
//
//   inner == 1   rows: up to 8 KB (32 KB for fp32 / bf16 / fp16 rows) a group of lanes (a power of two,
//                up to a warp) per row, 16-byte loads where the rows allow it; longer rows a CTA each (or, with few
//                rows, several CTAs per row, each on a segment, folded by a second kernel in a fixed order);
//   inner  > 1   columns: a CTA takes 32 neighbouring columns of one chunk of the L rows (its 8 warps take rows in
//                turn, four loads in flight), so that a tall narrow input still fills the GPU; the chunks' states go to
//                scratch and a second kernel merges them, a warp per output.
//
// Index rules are those of PyTorch's CPU kernels, which the reference's tests take as golden: of equal extrema the
// lowest index wins; NaN beats every number for max AND for min, and of several NaN the first.  Variance follows
// var(correction): M2 / max(0, n - correction), accumulated in fp64 as shifted sums (shift = the row's first element;
// over rows of fp32 / bf16 / fp16 values the sums of up to eight neighbouring terms are formed in fp32 first).
#include <limits>
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
  double inv_n, inv_denom;  // moments: 1 / L and 1 / max(0, L - correction) (inf when that is zero), formed on the host
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
  static constexpr bool kMoments = false;
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
  // Every kernel hands a thread its elements in rising index order, so a later element wins only when it is strictly
  // better: wins() with ia > ib.
  __device__ static __forceinline__ void fold(State& s, A x, int64_t idx) {
    const bool sn = is_nan(s.v), xn = is_nan(x);
    const bool take = s.i < 0 || (xn ? !sn : (!sn && (IS_MAX ? x > s.v : x < s.v)));
    if (take) {
      s.v = x;
      s.i = idx;
    }
  }
  // VEC elements at rising indices idx0 .. idx0 + VEC - 1.  For fp32 states the extremum of the vector is formed first
  // (NaN-propagating, one instruction per element) and a vector that beats the running state leaves only its extremum
  // and its first index behind, without a branch; resolve() finds the position inside that one vector afterwards.
  template <int VEC> __device__ static __forceinline__ void fold_vec(State& s, const A (&x)[VEC], int64_t idx0) {
    if constexpr (std::is_same<A, float>::value && VEC > 1) {
      float m = x[0];
#pragma unroll
      for (int k = 1; k < VEC; ++k) {
        if constexpr (IS_MAX) asm("max.NaN.f32 %0, %1, %2;" : "=f"(m) : "f"(m), "f"(x[k]));
        else asm("min.NaN.f32 %0, %1, %2;" : "=f"(m) : "f"(m), "f"(x[k]));
      }
      const bool sn = is_nan(s.v), mn = is_nan(m);
      const bool take = s.i < 0 || (mn ? !sn : (!sn && (IS_MAX ? m > s.v : m < s.v)));
      s.v = take ? m : s.v;
      s.i = take ? idx0 : s.i;
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) fold(s, x[k], idx0 + k);
    }
  }
  // After a thread's last fold_vec and before its state meets another thread's: s.i is the first index of the vector
  // that holds the extremum s.v; read that vector again and take the first element equal to it (the first NaN when
  // it is NaN), value and index.  `base` is the element offset of index 0.
  template <int VEC> __device__ static __forceinline__ void resolve(State& s, const void* in, int64_t base, int dtype) {
    if constexpr (std::is_same<A, float>::value && VEC > 1) {
      if (s.i >= 0) {
        float x[VEC];
        DynamicIO::load<float, VEC>(in, base + s.i, dtype, x);
        const bool mn = is_nan(s.v);
        int k0 = VEC - 1;
#pragma unroll
        for (int k = VEC - 2; k >= 0; --k)
          if (mn ? is_nan(x[k]) : x[k] == s.v) k0 = k;
        float v = x[VEC - 1];
#pragma unroll
        for (int k = VEC - 2; k >= 0; --k)
          if (k0 == k) v = x[k];
        s.v = v;
        s.i += k0;
      }
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
// A = float for fp32 / bf16 / fp16 inputs, double for fp64 inputs.  The state is fp64 either way.
template <typename A> struct MomentOpT {
  using State = MomentState;
  using Acc = A;
  static constexpr bool kMoments = true;
  __device__ static __forceinline__ State init(A first) { return State{0.0, 0.0, static_cast<double>(first)}; }
  __device__ static __forceinline__ State neutral_like(const State& s) { return State{0.0, 0.0, s.shift}; }
  __device__ static __forceinline__ void fold(State& s, A x, int64_t) {
    const double d = static_cast<double>(x) - s.shift;
    s.s1 += d;
    s.s2 = fma(d, d, s.s2);
  }
  // A vector of fp32 values: the differences from the shift (itself an fp32 value: the row's first element), their sum
  // and the sum of their squares are formed in fp32 (at most eight terms, a relative error of a few 2^-24 of the
  // vector's own terms) and only the two sums go through the fp64 pipe, which otherwise bounds the kernel at three fp64
  // operations and a conversion per element.
  template <int VEC> __device__ static __forceinline__ void fold_vec(State& s, const A (&x)[VEC], int64_t idx0) {
    if constexpr (std::is_same<A, float>::value && VEC > 1) {
      const float shift = static_cast<float>(s.shift);
      float b1 = 0.f, b2 = 0.f;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float d = x[k] - shift;
        b1 += d;
        b2 = fmaf(d, d, b2);
      }
      s.s1 += static_cast<double>(b1);
      s.s2 += static_cast<double>(b2);
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) fold(s, x[k], idx0 + k);
    }
  }
  template <int VEC> __device__ static __forceinline__ void resolve(State&, const void*, int64_t, int) {}
  __device__ static __forceinline__ void merge(State& s, const State& o) {  // every partial of a row uses the same shift
    s.s1 += o.s1;
    s.s2 += o.s2;
  }
  __device__ static __forceinline__ State shfl(const State& s, int o) {
    return State{__shfl_down_sync(0xffffffffu, s.s1, o), __shfl_down_sync(0xffffffffu, s.s2, o), s.shift};
  }
  __device__ static __forceinline__ void finish(const ExtParams& p, const State& s, int64_t out_index) {
    // products with the reciprocals instead of three fp64 divisions per output (the last bit of the fp64 value may
    // differ from the quotient's; it is rounded to the output type afterwards)
    double m2 = s.s2 - s.s1 * s.s1 * p.inv_n;
    if (m2 < 0.0) m2 = 0.0;  // rounding of a constant row
    double v = m2 * p.inv_denom;   // L <= correction: the reciprocal is inf, so inf or NaN, as on the CPU
    if (p.take_sqrt) v = sqrt(v);
    double o[1] = {v};
    DynamicIO::store<double, 1>(p.out0, out_index, p.out_dtype, o);
    if (p.out1) {
      double mean[1] = {s.shift + s.s1 * p.inv_n};
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
template <class Op, int THREADS, int VEC>
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
  // VEC elements per load (begin, end and L are multiples of VEC when VEC > 1), four loads in flight
  constexpr int kUnroll = 4;
  constexpr int64_t kStep = static_cast<int64_t>(THREADS) * VEC;
  int64_t e = begin + static_cast<int64_t>(threadIdx.x) * VEC;
  if constexpr (std::is_same<A, float>::value && VEC > 1) {
    // fp32 states over 16-byte vectors (4 fp32 or 8 16-bit elements): eight loads in flight, kept as loaded and widened
    // only when they are folded
    const int64_t es = p.in_dtype == SB_F32 ? 4 : 2;
    if (VEC * es == 16 && (p.in_dtype == SB_F32 || p.in_dtype == SB_BF16 || p.in_dtype == SB_F16)) {
      const char* src = static_cast<const char*>(p.in) + base * es;
      for (; e + 7 * kStep < end; e += 8 * kStep) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(src + (e + u * kStep) * es);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          A x[VEC];
          if (p.in_dtype == SB_F32) load_as<float, float, VEC>(&raw[u], x);
          else if (p.in_dtype == SB_BF16) load_as<float, __nv_bfloat16, VEC>(&raw[u], x);
          else load_as<float, __half, VEC>(&raw[u], x);
          Op::template fold_vec<VEC>(s, x, e + u * kStep);
        }
      }
    }
  }
  for (; e + (kUnroll - 1) * kStep < end; e += kUnroll * kStep) {
    A x[kUnroll][VEC];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) DynamicIO::load<A, VEC>(p.in, base + e + u * kStep, p.in_dtype, x[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) Op::template fold_vec<VEC>(s, x[u], e + u * kStep);
  }
  for (; e < end; e += kStep) {
    A x[VEC];
    DynamicIO::load<A, VEC>(p.in, base + e, p.in_dtype, x);
    Op::template fold_vec<VEC>(s, x, e);
  }
  Op::template resolve<VEC>(s, p.in, base, p.in_dtype);
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

// ---- short rows: `lpr` lanes per row ---------------------------------------------------------------------------
// Lane `sub` of a group takes elements (sub + k lpr) VEC .. + VEC - 1; two such loads are in flight.  The tree that
// folds a group's states only ever hands lane `sub` the state of lane `sub + o` of its own group on the way to lane 0.
template <class Op, int VEC>
__global__ void __launch_bounds__(256) ext_rows_group_kernel(ExtParams p, int lpr) {
  using A = typename Op::Acc;
  using State = typename Op::State;
  const int lane = threadIdx.x & 31, sub = lane & (lpr - 1);
  const int per_warp = 32 / lpr;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  const int64_t step = static_cast<int64_t>(lpr) * VEC;
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); w * per_warp < p.outer; w += nwarps) {
    int64_t row = w * per_warp + lane / lpr;
    const bool live = row < p.outer;
    row = live ? row : p.outer - 1;  // every lane takes part in the shuffles
    const int64_t base = row * p.L;
    A first[1];
    DynamicIO::load<A, 1>(p.in, base, p.in_dtype, first);
    State s = Op::init(first[0]);
    int64_t e = static_cast<int64_t>(sub) * VEC;
    if constexpr (std::is_same<A, float>::value && VEC > 1) {
      // fp32 states over 16-byte vectors: eight loads in flight per lane, widened only when they are folded (the launch
      // picks lpr so that a lane has about eight vectors of its row)
      const int64_t es = p.in_dtype == SB_F32 ? 4 : 2;
      if (VEC * es == 16 && (p.in_dtype == SB_F32 || p.in_dtype == SB_BF16 || p.in_dtype == SB_F16)) {
        const char* src = static_cast<const char*>(p.in) + base * es;
        for (; e + 7 * step < p.L; e += 8 * step) {
          uint4 raw[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(src + (e + u * step) * es);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            A x[VEC];
            if (p.in_dtype == SB_F32) load_as<float, float, VEC>(&raw[u], x);
            else if (p.in_dtype == SB_BF16) load_as<float, __nv_bfloat16, VEC>(&raw[u], x);
            else load_as<float, __half, VEC>(&raw[u], x);
            Op::template fold_vec<VEC>(s, x, e + u * step);
          }
        }
      }
    }
    for (; e + step < p.L; e += 2 * step) {
      A x[2][VEC];
      DynamicIO::load<A, VEC>(p.in, base + e, p.in_dtype, x[0]);
      DynamicIO::load<A, VEC>(p.in, base + e + step, p.in_dtype, x[1]);
#pragma unroll
      for (int u = 0; u < 2; ++u) Op::template fold_vec<VEC>(s, x[u], e + u * step);
    }
    if (e < p.L) {
      A x[VEC];
      DynamicIO::load<A, VEC>(p.in, base + e, p.in_dtype, x);
      Op::template fold_vec<VEC>(s, x, e);
    }
    Op::template resolve<VEC>(s, p.in, base, p.in_dtype);
    for (int o = lpr >> 1; o > 0; o >>= 1) {
      const State other = Op::shfl(s, o);
      Op::merge(s, other);
    }
    if (sub == 0 && live) Op::finish(p, s, row);
  }
}

// ---- columns in chunks: grid (column tiles of 32, chunks of rows, outer) -------------------------------------------
template <class Op, int CV>
__global__ void __launch_bounds__(256) ext_cols_chunk_kernel(ExtParams p, int cpr) {
  using A = typename Op::Acc;
  using State = typename Op::State;
  extern __shared__ __align__(16) unsigned char ext_smem[];
  State* sm = reinterpret_cast<State*>(ext_smem);  // [8 warps][cpr lanes][CV]
  // `cpr` lanes (a power of two) cover a row of the tile, CV neighbouring columns each; the warp's other lanes take
  // the next rows, so that a narrow tensor still gives every lane a column
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int csub = lane & (cpr - 1), rsub = lane / cpr, rpw = 32 / cpr;
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * cpr + csub) * CV;
  const int64_t o = blockIdx.z;
  const int64_t chunk = blockIdx.y;
  const int64_t begin = chunk * p.seg;
  const int64_t end = begin + p.seg < p.L ? begin + p.seg : p.L;
  const bool live = col < p.inner;  // inner is a multiple of CV
  const int64_t base = o * p.L * p.inner + (live ? col : 0);
  A first[CV];
  DynamicIO::load<A, CV>(p.in, base, p.in_dtype, first);  // the columns' first elements: the shift of every chunk
  State s[CV];
#pragma unroll
  for (int c = 0; c < CV; ++c) s[c] = Op::init(first[c]);
  if (live) {
    const int64_t step = 8 * rpw;
    int64_t e = begin + warp * rpw + rsub;
    for (; e + 3 * step < end; e += 4 * step) {
      A x[4][CV];
#pragma unroll
      for (int u = 0; u < 4; ++u) DynamicIO::load<A, CV>(p.in, base + (e + u * step) * p.inner, p.in_dtype, x[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int c = 0; c < CV; ++c) Op::fold(s[c], x[u][c], e + u * step);
    }
    for (; e < end; e += step) {
      A x[CV];
      DynamicIO::load<A, CV>(p.in, base + e * p.inner, p.in_dtype, x);
#pragma unroll
      for (int c = 0; c < CV; ++c) Op::fold(s[c], x[c], e);
    }
  }
  // lanes cpr apart hold the same columns (and, for the moments, the same shift)
  for (int d = 16; d >= cpr; d >>= 1) {
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      const State other = Op::shfl(s[c], d);
      Op::merge(s[c], other);
    }
  }
  if (rsub == 0) {
#pragma unroll
    for (int c = 0; c < CV; ++c) sm[(warp * cpr + csub) * CV + c] = s[c];
  }
  __syncthreads();
  if (warp == 0 && rsub == 0 && live) {
#pragma unroll
    for (int c = 0; c < CV; ++c) {
      State t = sm[csub * CV + c];
#pragma unroll
      for (int w = 1; w < 8; ++w) Op::merge(t, sm[(w * cpr + csub) * CV + c]);
      const int64_t out_index = o * p.inner + col + c;
      if (p.nseg == 1) Op::finish(p, t, out_index);
      else static_cast<State*>(p.scratch)[out_index * p.nseg + chunk] = t;
    }
  }
}

// The chunk states of one output, merged by a warp: lane l takes chunks l, l + 32, ... in order, then the lanes fold.
template <class Op>
__global__ void __launch_bounds__(256) ext_cols_final_kernel(ExtParams p) {
  using State = typename Op::State;
  const int lane = threadIdx.x & 31;
  const int64_t total = p.outer * p.inner;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); c < total; c += nwarps) {
    const State* part = static_cast<const State*>(p.scratch) + c * p.nseg;
    State s = lane < p.nseg ? part[lane] : Op::neutral_like(part[0]);
    for (int k = lane + 32; k < p.nseg; k += 32) Op::merge(s, part[k]);
    s = warp_fold<Op>(s);
    if (lane == 0) Op::finish(p, s, c);
  }
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
  if (nseg > 1) *seg = (*seg + 63) / 64 * 64;  // segment starts stay aligned for the vector loads
  nseg = static_cast<int>((L + *seg - 1) / *seg);
  return nseg;
}

// Chunks of rows for the column kernel: enough CTAs for eight per SM, at least 256 rows each, at most 1024 chunks.
int plan_chunks(int64_t outer, int64_t L, int64_t inner, int64_t* seg) {
  // the launch takes four columns per thread when inner allows it (tiles of up to 128 columns), else tiles of 32
  int64_t tile_cols = 32;
  if (inner % 4 == 0) {
    tile_cols = 4;
    while (tile_cols < 128 && tile_cols < inner) tile_cols <<= 1;
  }
  const int64_t tiles = (inner + tile_cols - 1) / tile_cols * outer;
  int64_t want = (8LL * sm_count() + tiles - 1) / tiles;
  const int64_t by_len = (L + 255) / 256;
  if (want > by_len) want = by_len;
  if (want > 1024) want = 1024;
  if (want < 1) want = 1;
  *seg = (L + want - 1) / want;
  return static_cast<int>((L + *seg - 1) / *seg);
}

// Longest row (bytes) that a group of lanes takes; longer rows get a CTA each.  fp32 / bf16 / fp16 rows keep eight 16-byte
// loads per lane in flight, which a warp sustains up to 32 KB; a CTA needs 64 KB rows for the same.
__host__ __device__ constexpr int64_t group_row_bytes(int dtype, bool moments) {
  (void)moments;
  return (dtype == SB_F32 || dtype == SB_BF16 || dtype == SB_F16) ? 32768 : 8192;
}

template <class Op>
int launch_ext(ExtParams p, cudaStream_t st) {
  if (p.inner == 1 && p.L * static_cast<int64_t>(dtype_size(p.in_dtype)) <= group_row_bytes(p.in_dtype, Op::kMoments)) {
    const int64_t es = static_cast<int64_t>(dtype_size(p.in_dtype));
    const bool vec = p.L % 4 == 0 && reinterpret_cast<uintptr_t>(p.in) % static_cast<uintptr_t>(es * 4 < 16 ? es * 4 : 16) == 0;
    const bool vec8 = es == 2 && p.L % 8 == 0 && reinterpret_cast<uintptr_t>(p.in) % 16 == 0;  // 16-byte loads of 16-bit elements
    const int64_t units = vec8 ? p.L / 8 : (vec ? p.L / 4 : p.L);  // loads per row
    int lpr = 1;
    while (lpr < 32 && lpr * 2 <= units) lpr <<= 1;  // at least one load per lane, two where the row has them
    if (lpr > 1 && lpr * 2 > units) lpr >>= 1;
    const bool deep = std::is_same<typename Op::Acc, float>::value && (vec8 || (vec && es == 4)) &&
                      (p.in_dtype == SB_F32 || p.in_dtype == SB_BF16 || p.in_dtype == SB_F16);
    if (deep) {  // 16-byte vectors and an fp32 state: eight vectors of the row per lane
      lpr = 1;
      while (lpr < 32 && lpr * 8 < units) lpr <<= 1;
    }
    const int64_t rows_per_cta = 8LL * (32 / lpr);
    int64_t ctas = (p.outer + rows_per_cta - 1) / rows_per_cta;
    const int64_t cap = 8LL * sm_count();
    if (ctas > cap) ctas = cap;
    if (vec8) ext_rows_group_kernel<Op, 8><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p, lpr);
    else if (vec) ext_rows_group_kernel<Op, 4><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p, lpr);
    else ext_rows_group_kernel<Op, 1><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p, lpr);
    return launch_status();
  }
  if (p.inner == 1) {
    // four elements per load when every row and every segment starts on the boundary such a load needs
    const int64_t es4 = static_cast<int64_t>(dtype_size(p.in_dtype)) * 4;
    // (not for the moments of fp64 inputs: with an fp64 operation per element the vector form measured slower)
    const bool vec4 = (!Op::kMoments || std::is_same<typename Op::Acc, float>::value) && p.L % 4 == 0 && p.seg % 4 == 0 &&
                      reinterpret_cast<uintptr_t>(p.in) % static_cast<uintptr_t>(es4 < 16 ? es4 : 16) == 0;
    const bool vec8 = vec4 && dtype_size(p.in_dtype) == 2 && p.L % 8 == 0 && p.seg % 8 == 0 && reinterpret_cast<uintptr_t>(p.in) % 16 == 0;
    if (p.outer > 65535) {  // gridDim.y limit: treat the rows as columns of an [1, L, outer]-like walk is wrong; fold in slabs
      for (int64_t r0 = 0; r0 < p.outer; r0 += 65535) {
        ExtParams q = p;
        const int64_t n = p.outer - r0 < 65535 ? p.outer - r0 : 65535;
        q.outer = n;
        q.in = static_cast<const char*>(p.in) + r0 * p.L * dtype_size(p.in_dtype);
        if (p.out0) q.out0 = static_cast<char*>(p.out0) + r0 * dtype_size(p.out_dtype);
        if (p.out1) q.out1 = static_cast<char*>(p.out1) + r0 * (Op::kMoments ? dtype_size(p.out_dtype) : 8);
        q.nseg = 1;
        q.seg = q.L;
        if (vec8) ext_rows_kernel<Op, 256, 8><<<dim3(1, static_cast<unsigned>(n)), 256, 0, st>>>(q);
        else if (vec4) ext_rows_kernel<Op, 256, 4><<<dim3(1, static_cast<unsigned>(n)), 256, 0, st>>>(q);
        else ext_rows_kernel<Op, 256, 1><<<dim3(1, static_cast<unsigned>(n)), 256, 0, st>>>(q);
        if (launch_status() != SB_OK) return SB_ERR_CUDA;
      }
      return SB_OK;
    }
    if (vec8) ext_rows_kernel<Op, 256, 8><<<dim3(p.nseg, static_cast<unsigned>(p.outer)), 256, 0, st>>>(p);
    else if (vec4) ext_rows_kernel<Op, 256, 4><<<dim3(p.nseg, static_cast<unsigned>(p.outer)), 256, 0, st>>>(p);
    else ext_rows_kernel<Op, 256, 1><<<dim3(p.nseg, static_cast<unsigned>(p.outer)), 256, 0, st>>>(p);
    if (launch_status() != SB_OK) return SB_ERR_CUDA;
    if (p.nseg > 1) {
      ext_rows_final_kernel<Op><<<static_cast<unsigned>((p.outer + 7) / 8), 256, 0, st>>>(p);
      return launch_status();
    }
    return SB_OK;
  }
  const int64_t total = p.outer * p.inner;
  if (p.outer <= 65535 && p.L >= 64) {
    // four neighbouring columns per thread when every row of columns starts on the boundary such a load needs
    const int64_t es4 = static_cast<int64_t>(dtype_size(p.in_dtype)) * 4;
    const bool cv4 = p.inner % 4 == 0 && reinterpret_cast<uintptr_t>(p.in) % static_cast<uintptr_t>(es4 < 16 ? es4 : 16) == 0;
    const int cv = cv4 ? 4 : 1;
    const int64_t units = p.inner / cv;  // column groups per row
    int cpr = 1;
    while (cpr < 32 && cpr < units) cpr <<= 1;
    dim3 grid(static_cast<unsigned>((units + cpr - 1) / cpr), static_cast<unsigned>(p.nseg), static_cast<unsigned>(p.outer));
    const size_t smem = sizeof(typename Op::State) * 8 * cpr * cv;
    if (cv4) ext_cols_chunk_kernel<Op, 4><<<grid, 256, smem, st>>>(p, cpr);
    else ext_cols_chunk_kernel<Op, 1><<<grid, 256, smem, st>>>(p, cpr);
    if (launch_status() != SB_OK) return SB_ERR_CUDA;
    if (p.nseg > 1) {
      int64_t ctas = (total + 7) / 8;
      const int64_t cap = 8LL * sm_count();
      if (ctas > cap) ctas = cap;
      ext_cols_final_kernel<Op><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p);
      return launch_status();
    }
    return SB_OK;
  }
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
  const bool group_rows = inner == 1 && L * static_cast<int64_t>(dtype_size(dtype)) <= group_row_bytes(dtype, moments);
  if (!group_rows && outer > 0 && outer <= 65535 && L > 0 && (inner == 1 || L >= 64)) {
    p->nseg = inner == 1 ? plan_segments(outer, L, &p->seg) : plan_chunks(outer, L, inner, &p->seg);
    if (p->nseg > 1) {
      const size_t need = static_cast<size_t>(outer) * static_cast<size_t>(inner) * p->nseg * state_bytes(moments, kind);
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
  if (inner <= 0 || outer <= 0 || outer > 65535 || L <= 0) return 0;
  const int kind = acc_kind(dtype);
  if (kind < 0) return 0;
  if (inner == 1 && L * static_cast<int64_t>(dtype_size(dtype)) <= group_row_bytes(dtype, moments != 0)) return 0;
  if (inner > 1 && L < 64) return 0;
  int64_t seg = 0;
  const int nseg = inner == 1 ? plan_segments(outer, L, &seg) : plan_chunks(outer, L, inner, &seg);
  return nseg > 1 ? static_cast<size_t>(outer) * static_cast<size_t>(inner) * nseg * state_bytes(moments != 0, kind) : 0;
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
  p.inv_n = 1.0 / static_cast<double>(L);
  {
    const double denom = static_cast<double>(L) - correction;
    p.inv_denom = denom > 0.0 ? 1.0 / denom : std::numeric_limits<double>::infinity();
  }
  p.take_sqrt = take_sqrt;
  if (dtype == SB_F64) return launch_ext<MomentOpT<double>>(p, as_stream(stream));
  return launch_ext<MomentOpT<float>>(p, as_stream(stream));
}

}  // extern "C"

// Reductions sum / mean / amax / amin / prod / nansum over any set of dimensions.
//
// The dimensions of the descriptor may come in any order; they are sorted by input stride, then neighbours that walk
// memory as one dimension are merged.
//
// Path 0  rows       the reduced run is contiguous (unit input stride) and every other dimension is kept.  Rows of
//                    whole 16-byte vectors of fp32 / bf16 / fp16: up to 4 KB a group of lanes per row, eight
//                    vectors in flight per lane (several rows where a row has fewer), the groups' sums added
//                    crosswise when the row is a power of two of vectors; up to 8 KB a warp per row; longer rows
//                    and all other types: one CTA (long rows) or one warp (short rows) per output, 16-byte
//                    loads where the pitch allows, shuffle + shared-memory tree.
// Path 1  split rows same layout but too few outputs to fill the GPU: each row is cut into segments,
//                    one CTA per segment writes a partial into caller-provided scratch, a second
//                    kernel folds the partials in a fixed order (no atomics: bit-reproducible).
// Path 2  columns    the fastest dimension is kept with unit strides and one dimension is reduced: lanes run along
//                    the kept dimension (16-byte column vectors where the pitch allows), the reduced rows are cut
//                    into chunks over the grid so that a tall narrow input fills the GPU, the chunks' partial
//                    results go to scratch and a second kernel adds them, a warp per output.
// Path 3  generic    one thread per output walking the reduced index space.
//
// Accumulation type: fp32 for fp32/bf16/fp16, fp64 for fp64, int64 for integer and bool inputs.
#include <type_traits>

#include "io.cuh"

namespace sb {

namespace {

constexpr int kRedKeep = 3;  // kept (non-reduced) dimensions handled by paths 0-2

struct RedParams {
  const void* in;
  void* out;
  int in_dtype, out_dtype;
  int64_t L;                 // reduced run length (paths 0-2)
  int64_t red_stride;        // input stride of the reduced dimension (path 2)
  int64_t noutputs;
  uint32_t keep_sizes[kRedKeep];
  int64_t keep_in_strides[kRedKeep];
  int64_t keep_out_strides[kRedKeep];
  double scale;              // 1/count for mean, 1 otherwise
  int splits;                // path 1
  int64_t seg;               // path 1: elements per segment (multiple of the vector width)
  void* scratch;
  int vpr;                   // path 2: column vectors one warp covers per row (a power of two up to 32)
  int col_vec;               // path 2: 1 = 16-byte column vectors
};

struct RedGenericParams {
  const void* in;
  void* out;
  int in_dtype, out_dtype;
  int nkeep, nred;
  uint32_t keep_sizes[SB_MAX_DIMS];
  int64_t keep_in_strides[SB_MAX_DIMS];
  int64_t keep_out_strides[SB_MAX_DIMS];
  uint32_t red_sizes[SB_MAX_DIMS];
  int64_t red_in_strides[SB_MAX_DIMS];
  int64_t noutputs, nreduce;
  double scale;
};

// ---- functors -----------------------------------------------------------------------------------------------
// `pre` is applied to every element as it is loaded (not to partial results).
template <typename A> struct SumOp {
  static constexpr bool kMinMax = false;
  static constexpr bool kIsMax = false;
  __device__ static __forceinline__ A identity() { return A(0); }
  __device__ static __forceinline__ A pre(A x) { return x; }
  __device__ static __forceinline__ A combine(A a, A b) { return a + b; }
};
template <typename A> struct NanSumOp {  // NaN elements count as zero
  static constexpr bool kMinMax = false;
  static constexpr bool kIsMax = false;
  __device__ static __forceinline__ A identity() { return A(0); }
  __device__ static __forceinline__ A pre(A x) {
    if constexpr (std::is_floating_point<A>::value) return x != x ? A(0) : x;
    else return x;
  }
  __device__ static __forceinline__ A combine(A a, A b) { return a + b; }
};
template <typename A> struct ProdOp {
  static constexpr bool kMinMax = false;
  static constexpr bool kIsMax = false;
  __device__ static __forceinline__ A identity() { return A(1); }
  __device__ static __forceinline__ A pre(A x) { return x; }
  __device__ static __forceinline__ A combine(A a, A b) { return a * b; }
};
// max / min propagate NaN (amax semantics).  fp32 uses the single-instruction max.NaN / min.NaN forms.
template <typename A> struct MaxOp {
  static constexpr bool kMinMax = true;
  static constexpr bool kIsMax = true;
  __device__ static __forceinline__ A identity() {
    if constexpr (std::is_same<A, float>::value) return -CUDART_INF_F;
    else if constexpr (std::is_same<A, double>::value) return -CUDART_INF;
    else return INT64_MIN;
  }
  __device__ static __forceinline__ A pre(A x) { return x; }
  __device__ static __forceinline__ A combine(A a, A b) {
    if constexpr (std::is_same<A, float>::value) {
      float r;
      asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
      return r;
    } else if constexpr (std::is_floating_point<A>::value) {
      return (b > a || b != b) ? b : a;
    } else {
      return b > a ? b : a;
    }
  }
};
template <typename A> struct MinOp {
  static constexpr bool kMinMax = true;
  static constexpr bool kIsMax = false;
  __device__ static __forceinline__ A identity() {
    if constexpr (std::is_same<A, float>::value) return CUDART_INF_F;
    else if constexpr (std::is_same<A, double>::value) return CUDART_INF;
    else return INT64_MAX;
  }
  __device__ static __forceinline__ A pre(A x) { return x; }
  __device__ static __forceinline__ A combine(A a, A b) {
    if constexpr (std::is_same<A, float>::value) {
      float r;
      asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
      return r;
    } else if constexpr (std::is_floating_point<A>::value) {
      return (b < a || b != b) ? b : a;
    } else {
      return b < a ? b : a;
    }
  }
};

// Packed 16-bit max / min (two elements per instruction, NaN propagating); exact, since the extremum of
// 16-bit values is itself one of them.
template <typename T2, bool IS_MAX> __device__ __forceinline__ T2 minmax2(T2 a, T2 b) {
  if constexpr (IS_MAX) return __hmax2_nan(a, b);
  else return __hmin2_nan(a, b);
}

template <typename A> __device__ __forceinline__ A shfl_down_t(A v, int o) { return __shfl_down_sync(0xffffffffu, v, o); }
template <> __device__ __forceinline__ int64_t shfl_down_t<int64_t>(int64_t v, int o) {
  return static_cast<int64_t>(__shfl_down_sync(0xffffffffu, static_cast<long long>(v), o));
}

template <class F, typename A> __device__ __forceinline__ A warp_reduce(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = F::combine(v, shfl_down_t<A>(v, o));
  return v;  // valid in lane 0
}

template <class F, typename A, int THREADS> __device__ __forceinline__ A block_reduce(A v, A* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_reduce<F, A>(v);
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  A r = F::identity();
  if (warp == 0) {
    r = lane < THREADS / 32 ? sm[lane] : F::identity();
    r = warp_reduce<F, A>(r);
  }
  __syncthreads();
  return r;  // valid in thread 0
}

template <typename A> __device__ __forceinline__ A apply_scale(A v, double scale) {
  if constexpr (std::is_floating_point<A>::value) return static_cast<A>(v * static_cast<A>(scale));
  else return v;
}

// Offsets of output number `o` (kept dims, fastest first).
__device__ __forceinline__ void keep_offsets(const RedParams& p, int64_t o, int64_t& in_off, int64_t& out_off) {
  uint64_t r = static_cast<uint64_t>(o);
  in_off = 0;
  out_off = 0;
#pragma unroll
  for (int d = 0; d < kRedKeep; ++d) {
    const uint64_t i = r % p.keep_sizes[d];
    r /= p.keep_sizes[d];
    in_off += static_cast<int64_t>(i) * p.keep_in_strides[d];
    out_off += static_cast<int64_t>(i) * p.keep_out_strides[d];
  }
}

// Reduces elements [begin, end) of a contiguous run starting at element offset `base`; the vector body
// covers the 16-byte-aligned middle, the ragged ends are scalar.
template <class IO, class F, typename A, int VEC, int THREADS>
__device__ __forceinline__ A thread_reduce_run(const void* in, int dtype, int64_t base, int64_t n) {
  using S = typename IO::storage;
  constexpr bool kPacked = F::kMinMax && VEC == 8 && std::is_same<A, float>::value &&
                           (std::is_same<S, __half>::value || std::is_same<S, __nv_bfloat16>::value);
  const int64_t nvec = n / VEC;
  constexpr int kUnroll = 4;
  A r = F::identity();
  if constexpr (kPacked) {
    using S2 = typename std::conditional<std::is_same<S, __half>::value, __half2, __nv_bfloat162>::type;
    const S* src = static_cast<const S*>(in) + base;
    S2 acc2[4];
    {
      const S lim = convert<S, float>(F::identity());
      S2 init;
      init.x = lim;
      init.y = lim;
#pragma unroll
      for (int k = 0; k < 4; ++k) acc2[k] = init;
    }
    int64_t i = threadIdx.x;
    for (; i + static_cast<int64_t>(kUnroll - 1) * THREADS < nvec; i += THREADS * kUnroll) {
      uint4 raw[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) raw[u] = *reinterpret_cast<const uint4*>(src + (i + static_cast<int64_t>(u) * THREADS) * VEC);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const S2* h = reinterpret_cast<const S2*>(&raw[u]);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc2[k] = minmax2<S2, F::kIsMax>(acc2[k], h[k]);
      }
    }
    for (; i < nvec; i += THREADS) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i * VEC);
      const S2* h = reinterpret_cast<const S2*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc2[k] = minmax2<S2, F::kIsMax>(acc2[k], h[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      r = F::combine(r, convert<float, S>(acc2[k].x));
      r = F::combine(r, convert<float, S>(acc2[k].y));
    }
  } else {
    A acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = F::identity();
    // main part: all kUnroll vectors of a pass exist, so the loads carry no guards and are issued together
    int64_t i = threadIdx.x;
    for (; i + static_cast<int64_t>(kUnroll - 1) * THREADS < nvec; i += THREADS * kUnroll) {
      A f[kUnroll][VEC];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) IO::template load<A, VEC>(in, base + (i + static_cast<int64_t>(u) * THREADS) * VEC, dtype, f[u]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], F::pre(f[u][k]));
      }
    }
    for (; i < nvec; i += THREADS) {  // remainder, one vector at a time
      A f[VEC];
      IO::template load<A, VEC>(in, base + i * VEC, dtype, f);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], F::pre(f[k]));
    }
    r = acc[0];
#pragma unroll
    for (int k = 1; k < VEC; ++k) r = F::combine(r, acc[k]);
  }
  for (int64_t e = nvec * VEC + threadIdx.x; e < n; e += THREADS) {
    A one[1];
    IO::template load<A, 1>(in, base + e, dtype, one);
    r = F::combine(r, F::pre(one[0]));
  }
  return r;
}

// ---- path 0 ------------------------------------------------------------------------------------------------
template <class IO, class F, typename A, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS, sizeof(A) == 4 ? 2048 / THREADS : 1) red_rows_cta_kernel(RedParams p) {
  // fp32 accumulation: capped at 32 registers so that 2048 threads stay resident (the kernel is latency bound)

  __shared__ A sm[32];
  for (int64_t o = blockIdx.x; o < p.noutputs; o += gridDim.x) {
    int64_t in_off, out_off;
    keep_offsets(p, o, in_off, out_off);
    A v = thread_reduce_run<IO, F, A, VEC, THREADS>(p.in, p.in_dtype, in_off, p.L);
    v = block_reduce<F, A, THREADS>(v, sm);
    if (threadIdx.x == 0) {
      A r[1] = {apply_scale<A>(v, p.scale)};
      DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
    }
  }
}

template <class IO, class F, typename A, int THREADS>
__global__ void __launch_bounds__(THREADS) red_rows_warp_kernel(RedParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * (THREADS / 32);
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5); o < p.noutputs; o += stride) {
    int64_t in_off, out_off;
    keep_offsets(p, o, in_off, out_off);
    A v = F::identity();
    for (int64_t e = lane; e < p.L; e += 32) {
      A one[1];
      IO::template load<A, 1>(p.in, in_off + e, p.in_dtype, one);
      v = F::combine(v, F::pre(one[0]));
    }
    v = warp_reduce<F, A>(v);
    if (lane == 0) {
      A r[1] = {apply_scale<A>(v, p.scale)};
      DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
    }
  }
}

// Offsets of output row `o` when only kept dimension 0 has more than one element (no divisions).
__device__ __forceinline__ void row_offsets(const RedParams& p, bool flat, int64_t o, int64_t& in_off, int64_t& out_off) {
  if (flat) {
    in_off = o * p.keep_in_strides[0];
    out_off = o * p.keep_out_strides[0];
  } else {
    keep_offsets(p, o, in_off, out_off);
  }
}

// Rows of up to 256 vectors of 16 bytes, every row on a 16-byte boundary.  `lpr` lanes (a power of two) share a row
// and a lane keeps eight vectors in flight: 8 / nv consecutive rows with nv vectors of each (nv a power of two), so
// that a row of 256 bytes costs a lane one load and a row of 4 KB eight.
template <class IO, class F, typename A, int VEC>
__global__ void __launch_bounds__(256) red_rows_sub_kernel(RedParams p, int lpr, int nv) {
  using S = typename IO::storage;
  static_assert(sizeof(S) * VEC == 16, "one 16-byte vector per load");
  const int lane = threadIdx.x & 31;
  const int sub = lane & (lpr - 1);
  const int nv_shift = __ffs(nv) - 1;
  const int ru = 8 >> nv_shift;  // rows per lane group and step
  const int nvec = static_cast<int>(p.L / VEC);
  const int groups_per_warp = 32 / lpr;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t rows_per_warp = static_cast<int64_t>(groups_per_warp) * ru;
  const bool flat = p.keep_sizes[1] == 1 && p.keep_sizes[2] == 1;
  // the trip count is the same for the whole warp: the shuffles below name every lane
  for (int64_t wbase = gwarp * rows_per_warp; wbase < p.noutputs; wbase += nwarps * rows_per_warp) {
    const int64_t base = wbase + static_cast<int64_t>(lane / lpr) * ru;
    // Every slot loads: a slot past the last row or the last vector reads the nearest valid one instead and is left out
    // when the values are folded (a load under a condition would make the loads wait for one another).
    uint4 raw[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int64_t row = base + (k >> nv_shift);
      row = row < p.noutputs ? row : p.noutputs - 1;
      int v = sub + (k & (nv - 1)) * lpr;
      v = v < nvec ? v : nvec - 1;
      int64_t in_off, out_off;
      row_offsets(p, flat, row, in_off, out_off);
      raw[k] = *reinterpret_cast<const uint4*>(static_cast<const S*>(p.in) + in_off + static_cast<int64_t>(v) * VEC);
    }
    A s[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool live = base + (k >> nv_shift) < p.noutputs && sub + (k & (nv - 1)) * lpr < nvec;
      A x[VEC];
      load_as<A, S, VEC>(&raw[k], x);
      s[k] = live ? F::pre(x[0]) : F::identity();
#pragma unroll
      for (int e = 1; e < VEC; ++e) s[k] = F::combine(s[k], live ? F::pre(x[e]) : F::identity());
    }
    if (nv > 1) {
#pragma unroll
      for (int k = 0; k < 8; k += 2) s[k] = F::combine(s[k], s[k + 1]);
    }
    if (nv > 2) {
      s[0] = F::combine(s[0], s[2]);
      s[4] = F::combine(s[4], s[6]);
    }
    if (nv > 4) s[0] = F::combine(s[0], s[4]);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if ((k & (nv - 1)) == 0) {  // the same for every lane
        A v = s[k];
        for (int off = 1; off < lpr; off <<= 1) v = F::combine(v, __shfl_xor_sync(0xffffffffu, v, off));
        const int64_t row = base + (k >> nv_shift);
        if (sub == 0 && row < p.noutputs) {
          int64_t in_off, out_off;
          row_offsets(p, flat, row, in_off, out_off);
          A r[1] = {apply_scale<A>(v, p.scale)};
          DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
        }
      }
    }
  }
}

// The same split of the work for rows of exactly lpr * NV vectors (a power of two of them) whose kept dimensions collapse
// to one row pitch: no slot needs clamping, the addresses are a row pointer plus constants, and the lane groups add
// their R = 8 / NV row sums crosswise - each exchange hands half of a lane's sums to its partner, so after log2 R
// exchanges lane `sub` holds row `sub` alone - which takes R - 1 + log2(lpr / R) shuffles and one store for R rows
// where the kernel above spends R log2 lpr shuffles and R stores.  Needs lpr >= R.
template <class IO, class F, typename A, int VEC, int NV>
__global__ void __launch_bounds__(256) red_rows_pow2_kernel(RedParams p, int lpr) {
  using S = typename IO::storage;
  static_assert(sizeof(S) * VEC == 16, "one 16-byte vector per load");
  constexpr int R = 8 / NV;
  const int lane = threadIdx.x & 31;
  const int sub = lane & (lpr - 1);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t rows_per_warp = static_cast<int64_t>(32 / lpr) * R;
  const int64_t pitch = p.keep_in_strides[0];
  const int64_t opitch = p.keep_out_strides[0];
  const S* in = static_cast<const S*>(p.in) + sub * VEC;
  const int64_t kstep = static_cast<int64_t>(lpr) * VEC;
  for (int64_t wbase = gwarp * rows_per_warp; wbase < p.noutputs; wbase += nwarps * rows_per_warp) {
    const int64_t base = wbase + static_cast<int64_t>(lane / lpr) * R;
    const bool whole = wbase + rows_per_warp <= p.noutputs;  // the same for the warp
    uint4 raw[8];
    if (whole) {
      const S* src = in + base * pitch;
#pragma unroll
      for (int k = 0; k < 8; ++k) raw[k] = *reinterpret_cast<const uint4*>(src + (k / NV) * pitch + (k % NV) * kstep);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        int64_t row = base + k / NV;
        row = row < p.noutputs ? row : p.noutputs - 1;
        raw[k] = *reinterpret_cast<const uint4*>(in + row * pitch + (k % NV) * kstep);
      }
    }
    A t[R];
#pragma unroll
    for (int u = 0; u < R; ++u) {
#pragma unroll
      for (int kk = 0; kk < NV; ++kk) {
        A x[VEC];
        load_as<A, S, VEC>(&raw[u * NV + kk], x);
        if (kk == 0) t[u] = F::pre(x[0]);
        else t[u] = F::combine(t[u], F::pre(x[0]));
#pragma unroll
        for (int e = 1; e < VEC; ++e) t[u] = F::combine(t[u], F::pre(x[e]));
      }
    }
    // crosswise: after the exchange at distance d a lane keeps the rows whose index has the lane's bit d
#pragma unroll
    for (int d = 1, held = R; d < R; d <<= 1, held >>= 1) {
      const bool upper = (sub & d) != 0;
#pragma unroll
      for (int j = 0; j < held / 2; ++j) {
        const A keep = upper ? t[2 * j + 1] : t[2 * j];
        const A send = upper ? t[2 * j] : t[2 * j + 1];
        t[j] = F::combine(keep, __shfl_xor_sync(0xffffffffu, send, d));
      }
    }
    A v = t[0];
    for (int d = R; d < lpr; d <<= 1) v = F::combine(v, __shfl_xor_sync(0xffffffffu, v, d));
    const int64_t row = base + sub;
    if (sub < R && row < p.noutputs) {
      A r[1] = {apply_scale<A>(v, p.scale)};
      DynamicIO::store<A, 1>(p.out, row * opitch, p.out_dtype, r);
    }
  }
}

// Rows of more than 256 vectors, up to 8 KB unless tuned otherwise: a warp per row, eight vectors in flight per lane, one
// accumulator per vector element.  No shared memory and no CTA barrier, which is what a CTA per row pays for at this
// length.
template <class IO, class F, typename A, int VEC>
__global__ void __launch_bounds__(256) red_rows_warp_vec_kernel(RedParams p) {
  const int lane = threadIdx.x & 31;
  const int nvec = static_cast<int>(p.L / VEC);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  const bool flat = p.keep_sizes[1] == 1 && p.keep_sizes[2] == 1;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < p.noutputs; row += nwarps) {
    int64_t in_off, out_off;
    row_offsets(p, flat, row, in_off, out_off);
    A acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = F::identity();
    int v = lane;
    for (; v + 7 * 32 < nvec; v += 8 * 32) {
      A x[8][VEC];
#pragma unroll
      for (int k = 0; k < 8; ++k) IO::template load<A, VEC>(p.in, in_off + static_cast<int64_t>(v + k * 32) * VEC, p.in_dtype, x[k]);
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = F::combine(acc[e], F::pre(x[k][e]));
    }
    for (; v < nvec; v += 32) {
      A x[VEC];
      IO::template load<A, VEC>(p.in, in_off + static_cast<int64_t>(v) * VEC, p.in_dtype, x);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = F::combine(acc[e], F::pre(x[e]));
    }
#pragma unroll
    for (int e = 1; e < VEC; ++e) acc[0] = F::combine(acc[0], acc[e]);
    const A r0 = warp_reduce<F, A>(acc[0]);
    if (lane == 0) {
      A r[1] = {apply_scale<A>(r0, p.scale)};
      DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
    }
  }
}

// ---- path 1 ------------------------------------------------------------------------------------------------
template <class IO, class F, typename A, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS) red_split_partial_kernel(RedParams p) {
  __shared__ A sm[32];
  const int64_t o = blockIdx.y;
  const int s = blockIdx.x;
  int64_t in_off, out_off;
  keep_offsets(p, o, in_off, out_off);
  const int64_t begin = static_cast<int64_t>(s) * p.seg;
  int64_t n = p.L - begin;
  if (n > p.seg) n = p.seg;
  A v = F::identity();
  if (n > 0) v = thread_reduce_run<IO, F, A, VEC, THREADS>(p.in, p.in_dtype, in_off + begin, n);
  v = block_reduce<F, A, THREADS>(v, sm);
  if (threadIdx.x == 0) static_cast<A*>(p.scratch)[o * p.splits + s] = v;
}

template <class F, typename A>
__global__ void __launch_bounds__(256) red_split_final_kernel(RedParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); o < p.noutputs; o += stride) {
    int64_t in_off, out_off;
    keep_offsets(p, o, in_off, out_off);
    const A* part = static_cast<const A*>(p.scratch) + o * p.splits;
    A v = F::identity();
    for (int s = lane; s < p.splits; s += 32) v = F::combine(v, part[s]);
    v = warp_reduce<F, A>(v);
    if (lane == 0) {
      A r[1] = {apply_scale<A>(v, p.scale)};
      DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
    }
  }
}

// A 16-byte load that stays where it is written: eight of them in a row are eight loads in flight (left to itself the
// compiler moves each load down to its use to save registers).
__device__ __forceinline__ uint4 load_u4_in_order(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

// Elements per 16-byte column vector of the statically typed inputs (fp32, bf16, fp16); the dynamically typed ones (double
// and integer accumulation) go element by element.
template <class IO> struct ColumnVector { static constexpr int value = 1; };
template <typename S> struct ColumnVector<StaticIO<S>> { static constexpr int value = 16 / static_cast<int>(sizeof(S)); };

// ---- path 2 ------------------------------------------------------------------------------------------------
// keep_sizes[0] = kept dimension 0 (unit strides), keep_sizes[1..2] = outer kept dims; L rows of stride red_stride are
// reduced (the shape of `x.sum(0)`).  The L rows are cut into `splits` chunks of `seg` rows so that tall, narrow inputs
// still fill the GPU; a CTA takes one chunk of one tile of columns.  A warp covers `vpr` column vectors (16 bytes each when
// the pitch allows it) of 32 / vpr rows at a time, its 8 warps further rows; the partial results of the chunks are added
// by a second kernel in an order that the plan alone fixes (bit-reproducible), or written directly when there is one chunk.
template <class IO, class F, typename A, int VEC>
__global__ void __launch_bounds__(256) red_cols_kernel(RedParams p) {
  __shared__ A sm[8][32 * VEC];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int vpr = p.vpr, rows_per_warp = 32 / vpr;
  const int cvl = lane % vpr, rsub = lane / vpr;
  const int64_t nvec = p.keep_sizes[0] / VEC;
  const int64_t cv = static_cast<int64_t>(blockIdx.x) * vpr + cvl;
  const uint64_t r = blockIdx.z;
  const uint64_t i1 = r % p.keep_sizes[1];
  const uint64_t i2 = r / p.keep_sizes[1];
  const int64_t in_base = static_cast<int64_t>(i1) * p.keep_in_strides[1] + static_cast<int64_t>(i2) * p.keep_in_strides[2];
  const int64_t chunk = blockIdx.y;
  const int64_t begin = chunk * p.seg;
  const int64_t end = begin + p.seg < p.L ? begin + p.seg : p.L;
  A acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = F::identity();
  if (cv < nvec) {
    const int64_t col0 = in_base + cv * VEC;
    const int64_t step = 8 * rows_per_warp;
    int64_t j = begin + warp * rows_per_warp + rsub;
    if constexpr (VEC > 1) {
      // Full-width tiles: eight rows in flight per thread, kept as loaded and widened only when they are added.
      // Narrower tiles measured faster with the four rows of the loop below.
      using S = typename IO::storage;
      static_assert(sizeof(S) * VEC == 16, "one 16-byte vector per load");
      if (vpr == 32) {
        const S* src = static_cast<const S*>(p.in) + col0;
        const int64_t rs = p.red_stride;
        for (; j + 7 * step < end; j += 8 * step) {
          uint4 raw[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) raw[u] = load_u4_in_order(src + (j + u * step) * rs);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            A x[VEC];
            load_as<A, S, VEC>(&raw[u], x);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], F::pre(x[k]));
          }
        }
      }
    }
    // four rows in flight per thread
    for (; j + 3 * step < end; j += 4 * step) {
      A v[4][VEC];
#pragma unroll
      for (int u = 0; u < 4; ++u) IO::template load<A, VEC>(p.in, col0 + (j + u * step) * p.red_stride, p.in_dtype, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], F::pre(v[u][k]));
    }
    for (; j < end; j += step) {
      A v[VEC];
      IO::template load<A, VEC>(p.in, col0 + j * p.red_stride, p.in_dtype, v);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], F::pre(v[k]));
    }
  }
  // rows that share the warp, then the 8 warps
  for (int off = vpr; off < 32; off <<= 1)
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = F::combine(acc[k], __shfl_xor_sync(0xffffffffu, acc[k], off));
  if (rsub == 0)
#pragma unroll
    for (int k = 0; k < VEC; ++k) sm[warp][cvl * VEC + k] = acc[k];
  __syncthreads();
  const int t = threadIdx.x;
  if (t < vpr * VEC) {
    const int64_t col = (static_cast<int64_t>(blockIdx.x) * vpr) * VEC + t;
    if (col < static_cast<int64_t>(p.keep_sizes[0])) {
      A a = sm[0][t];
#pragma unroll
      for (int w = 1; w < 8; ++w) a = F::combine(a, sm[w][t]);
      if (p.splits > 1) {
        const int64_t o = static_cast<int64_t>(r) * p.keep_sizes[0] + col;
        static_cast<A*>(p.scratch)[o * p.splits + chunk] = a;
      } else {
        const int64_t out_base = static_cast<int64_t>(i1) * p.keep_out_strides[1] + static_cast<int64_t>(i2) * p.keep_out_strides[2];
        A o1[1] = {apply_scale<A>(a, p.scale)};
        DynamicIO::store<A, 1>(p.out, out_base + col * p.keep_out_strides[0], p.out_dtype, o1);
      }
    }
  }
}

// The chunks' partial results of one output, added by `lanes` lanes (a power of two): lane l adds chunks l, l + lanes,
// ... in that order and the lanes' sums are added pairwise; the order depends on nothing but the plan, so the result
// is the same on every run.
template <class F, typename A>
__global__ void __launch_bounds__(256) red_cols_final_kernel(RedParams p, int lanes) {
  const int lane = threadIdx.x & 31, sub = lane & (lanes - 1);
  const int per_warp = 32 / lanes;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); w * per_warp < p.noutputs; w += nwarps) {
    const int64_t o = w * per_warp + lane / lanes;
    A v = F::identity();
    if (o < p.noutputs) {
      const A* part = static_cast<const A*>(p.scratch) + o * p.splits;
      int s2 = sub;
      for (; s2 + 7 * lanes < p.splits; s2 += 8 * lanes) {  // eight loads in flight
        A a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) a[u] = part[s2 + u * lanes];
#pragma unroll
        for (int u = 0; u < 8; ++u) v = F::combine(v, a[u]);
      }
      for (; s2 < p.splits; s2 += lanes) v = F::combine(v, part[s2]);
    }
    for (int d = 1; d < lanes; d <<= 1) v = F::combine(v, __shfl_xor_sync(0xffffffffu, v, d));
    if (sub == 0 && o < p.noutputs) {
      int64_t in_off, out_off;
      keep_offsets(p, o, in_off, out_off);
      A r[1] = {apply_scale<A>(v, p.scale)};
      DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, r);
    }
  }
}

// ---- path 3 ------------------------------------------------------------------------------------------------
template <class F, typename A>
__global__ void __launch_bounds__(256) red_generic_kernel(RedGenericParams p) {
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; o < p.noutputs;
       o += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t in_off = 0, out_off = 0;
    uint64_t r = static_cast<uint64_t>(o);
    for (int d = 0; d < p.nkeep; ++d) {
      const uint64_t i = r % p.keep_sizes[d];
      r /= p.keep_sizes[d];
      in_off += static_cast<int64_t>(i) * p.keep_in_strides[d];
      out_off += static_cast<int64_t>(i) * p.keep_out_strides[d];
    }
    A v = F::identity();
    for (int64_t j = 0; j < p.nreduce; ++j) {
      uint64_t q = static_cast<uint64_t>(j);
      int64_t off = in_off;
      for (int d = 0; d < p.nred; ++d) {
        const uint64_t i = q % p.red_sizes[d];
        q /= p.red_sizes[d];
        off += static_cast<int64_t>(i) * p.red_in_strides[d];
      }
      A one[1];
      DynamicIO::load<A, 1>(p.in, off, p.in_dtype, one);
      v = F::combine(v, F::pre(one[0]));
    }
    A res[1] = {apply_scale<A>(v, p.scale)};
    DynamicIO::store<A, 1>(p.out, out_off, p.out_dtype, res);
  }
}

// ---- host side -------------------------------------------------------------------------------------------
struct Dim {
  int64_t size, in_stride, out_stride;
  bool reduced;
};

struct Plan {
  int path;
  int acc;  // 0 float, 1 double, 2 int64
  RedParams p;
  RedGenericParams g;
  bool vec_ok;
  size_t scratch_bytes;
};

int acc_of(int dtype) {
  switch (dtype) {
    case SB_F16: case SB_BF16: case SB_F32: return 0;
    case SB_F64: return 1;
    case SB_BOOL: case SB_U8: case SB_I8: case SB_I16: case SB_I32: case SB_I64: return 2;
    default: return -1;
  }
}

int make_plan(const sb_reduce_desc* d, Plan* plan) {
  if (!d) return SB_ERR_INVALID_ARGUMENT;
  if (d->op < 0 || d->op >= SB_RED_OP_COUNT) return SB_ERR_INVALID_ARGUMENT;
  if (d->ndim < 1 || d->ndim > SB_MAX_DIMS) return SB_ERR_INVALID_ARGUMENT;
  if (d->in_dtype < 0 || d->in_dtype >= SB_DTYPE_COUNT || d->out_dtype < 0 || d->out_dtype >= SB_DTYPE_COUNT)
    return SB_ERR_UNSUPPORTED;
  plan->acc = acc_of(d->in_dtype);
  if (plan->acc < 0) return SB_ERR_UNSUPPORTED;
  if (d->op == SB_RED_MEAN && plan->acc == 2) return SB_ERR_UNSUPPORTED;  // mean is defined on floating types
  if ((d->op == SB_RED_AMAX || d->op == SB_RED_AMIN) && d->in_dtype == SB_BOOL) plan->acc = 2;

  // Drop size-1 dims, order the rest by input stride (callers list them in any order: a TensorIterator puts the
  // reduced dimensions first, whatever their strides), then merge neighbours that walk memory as one dimension.
  Dim raw[SB_MAX_DIMS];
  int nraw = 0;
  int64_t noutputs = 1, nreduce = 1;
  for (int i = 0; i < d->ndim; ++i) {
    if (d->sizes[i] < 0) return SB_ERR_INVALID_ARGUMENT;
    if (d->sizes[i] > 0xffffffffLL && d->ndim > 1) return SB_ERR_TOO_LARGE;
    const bool red = d->out_strides[i] == 0;
    if (red) nreduce *= d->sizes[i];
    else noutputs *= d->sizes[i];
    if (d->sizes[i] == 1) continue;
    raw[nraw++] = Dim{d->sizes[i], d->in_strides[i], d->out_strides[i], red};
  }
  // a stride of zero (an expanded input) names no position in memory: such dimensions go last
  auto mag = [](int64_t v) { return v == 0 ? INT64_MAX : (v < 0 ? -v : v); };
  for (int i = 1; i < nraw; ++i) {  // insertion sort: stable, at most SB_MAX_DIMS entries
    const Dim cur = raw[i];
    int j = i;
    for (; j > 0 && mag(raw[j - 1].in_stride) > mag(cur.in_stride); --j) raw[j] = raw[j - 1];
    raw[j] = cur;
  }
  Dim dims[SB_MAX_DIMS];
  int n = 0;
  for (int i = 0; i < nraw; ++i) {
    const Dim& cur = raw[i];
    if (n > 0) {
      Dim& prev = dims[n - 1];
      if (prev.reduced == cur.reduced && cur.in_stride == prev.in_stride * prev.size &&
          (cur.reduced || cur.out_stride == prev.out_stride * prev.size)) {
        prev.size *= cur.size;
        continue;
      }
    }
    dims[n++] = cur;
  }
  if (n == 0) {
    dims[0] = Dim{1, 1, 0, true};
    n = 1;
  }
  if (noutputs > 0 && nreduce > 0 && (!d->in || !d->out)) return SB_ERR_INVALID_ARGUMENT;
  if (noutputs > 0 && !d->out) return SB_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(d->in) % dtype_size(d->in_dtype) || reinterpret_cast<uintptr_t>(d->out) % dtype_size(d->out_dtype))
    return SB_ERR_MISALIGNED;

  const double scale = d->op == SB_RED_MEAN ? 1.0 / static_cast<double>(nreduce) : 1.0;
  plan->scratch_bytes = 0;
  plan->vec_ok = false;

  // generic parameters are always filled (path 3 fallback)
  RedGenericParams& g = plan->g;
  g.in = d->in;
  g.out = d->out;
  g.in_dtype = d->in_dtype;
  g.out_dtype = d->out_dtype;
  g.nkeep = g.nred = 0;
  for (int i = 0; i < n; ++i) {
    if (dims[i].reduced) {
      g.red_sizes[g.nred] = static_cast<uint32_t>(dims[i].size);
      g.red_in_strides[g.nred++] = dims[i].in_stride;
    } else {
      g.keep_sizes[g.nkeep] = static_cast<uint32_t>(dims[i].size);
      g.keep_in_strides[g.nkeep] = dims[i].in_stride;
      g.keep_out_strides[g.nkeep++] = dims[i].out_stride;
    }
  }
  g.noutputs = noutputs;
  g.nreduce = nreduce;
  g.scale = scale;
  plan->path = 3;

  int nred = g.nred, nkeep = g.nkeep;
  RedParams& p = plan->p;
  p.in = d->in;
  p.out = d->out;
  p.in_dtype = d->in_dtype;
  p.out_dtype = d->out_dtype;
  p.scale = scale;
  p.noutputs = noutputs;
  p.splits = 1;
  p.seg = 0;
  p.scratch = d->scratch;
  p.red_stride = 1;
  for (int k = 0; k < kRedKeep; ++k) {
    p.keep_sizes[k] = 1;
    p.keep_in_strides[k] = 0;
    p.keep_out_strides[k] = 0;
  }
  if (noutputs == 0 || nreduce == 0) return SB_OK;  // nothing to launch (empty reduce handled by the caller)

  const size_t es = dtype_size(d->in_dtype);
  const size_t valign = es * 8 >= 16 ? 16 : es * 8;
  if (nred == 1 && nkeep <= kRedKeep && dims[0].reduced && dims[0].in_stride == 1) {
    // paths 0 / 1
    p.L = dims[0].size;
    bool vec_ok = reinterpret_cast<uintptr_t>(d->in) % valign == 0;
    for (int k = 0; k < nkeep; ++k) {
      p.keep_sizes[k] = g.keep_sizes[k];
      p.keep_in_strides[k] = g.keep_in_strides[k];
      p.keep_out_strides[k] = g.keep_out_strides[k];
      const uint64_t s = static_cast<uint64_t>(g.keep_in_strides[k] < 0 ? -g.keep_in_strides[k] : g.keep_in_strides[k]);
      vec_ok = vec_ok && (s * es) % valign == 0;
    }
    plan->vec_ok = vec_ok;
    plan->path = 0;
    const int sms = sm_count();
    // Too few rows to occupy the GPU and rows long enough to be worth cutting.
    if (noutputs < 2LL * sms && p.L >= 32768 && noutputs <= 65535) {
      int64_t want = (4LL * sms + noutputs - 1) / noutputs;
      const int64_t max_by_len = p.L / 8192;
      if (want > max_by_len) want = max_by_len;
      if (want > 1024) want = 1024;
      if (want >= 2) {
        int64_t seg = (p.L + want - 1) / want;
        seg = (seg + 63) / 64 * 64;  // keeps every segment start 16-byte aligned for all dtypes
        p.seg = seg;
        p.splits = static_cast<int>((p.L + seg - 1) / seg);
        plan->path = 1;
        const size_t acc_size = 8;  // sized for the widest accumulator (fp64 / int64)
        plan->scratch_bytes = static_cast<size_t>(noutputs) * p.splits * acc_size;
      }
    }
    return SB_OK;
  }
  if (nred == 1 && nkeep >= 1 && nkeep <= kRedKeep && !dims[0].reduced && dims[0].in_stride == 1) {
    // path 2: find the reduced dim
    uint64_t outer = 1;
    for (int k = 0; k < nkeep; ++k) {
      p.keep_sizes[k] = g.keep_sizes[k];
      p.keep_in_strides[k] = g.keep_in_strides[k];
      p.keep_out_strides[k] = g.keep_out_strides[k];
      if (k >= 1) outer *= g.keep_sizes[k];
    }
    p.L = g.red_sizes[0];
    p.red_stride = g.red_in_strides[0];
    if (outer <= 65535) {
      plan->path = 2;
      // 16-byte column vectors when every row segment starts on a 16-byte boundary
      const int vec = static_cast<int>(16 / es);
      bool col_vec = acc_of(d->in_dtype) == 0 && g.keep_sizes[0] % vec == 0 && reinterpret_cast<uintptr_t>(d->in) % 16 == 0 &&
                     (static_cast<uint64_t>(p.red_stride < 0 ? -p.red_stride : p.red_stride) * es) % 16 == 0;
      for (int k = 1; k < nkeep; ++k) {
        const uint64_t st = static_cast<uint64_t>(g.keep_in_strides[k] < 0 ? -g.keep_in_strides[k] : g.keep_in_strides[k]);
        col_vec = col_vec && (st * es) % 16 == 0;
      }
      p.col_vec = col_vec ? 1 : 0;
      const int64_t nvec = col_vec ? g.keep_sizes[0] / vec : g.keep_sizes[0];
      int vpr = 1;
      while (vpr < 32 && vpr < nvec) vpr <<= 1;
      p.vpr = vpr;
      // chunks of rows: enough CTAs for eight per SM, at least 256 rows each, at most 1024 chunks
      const int64_t tiles = (nvec + vpr - 1) / vpr * static_cast<int64_t>(outer);
      int64_t want = (8LL * sm_count() + tiles - 1) / tiles;
      const int64_t max_by_len = (p.L + 255) / 256;
      if (want > max_by_len) want = max_by_len;
      if (want > 1024) want = 1024;
      if (want < 1) want = 1;
      p.seg = (p.L + want - 1) / want;
      p.splits = static_cast<int>((p.L + p.seg - 1) / p.seg);
      if (p.splits > 1) plan->scratch_bytes = static_cast<size_t>(noutputs) * p.splits * 8;
      return SB_OK;
    }
  }
  return SB_OK;
}

// Longest row (bytes) that a single warp reduces; longer rows take a CTA each.  0 switches the vector row kernels off.
int64_t g_warp_row_bytes = 8192;

template <class IO, class F, typename A>
int launch_paths(const Plan& plan, cudaStream_t st) {
  const RedParams& p = plan.p;
  const int sms = sm_count();
  if (plan.path == 0) {
    constexpr int kVec = ColumnVector<IO>::value;
    if constexpr (kVec > 1) {
      // rows of whole 16-byte vectors on 16-byte boundaries
      const int64_t nvec = p.L / kVec;
      if (plan.vec_ok && p.L % kVec == 0 && nvec >= 1 && g_warp_row_bytes > 0) {
        if (nvec <= 256) {
          int lpr = 1, nv = 1;
          while (lpr < 32 && lpr < nvec) lpr <<= 1;
          while (static_cast<int64_t>(lpr) * nv < nvec) nv <<= 1;
          const int64_t rows_per_cta = 8LL * (32 / lpr) * (8 / nv);
          int64_t ctas = (p.noutputs + rows_per_cta - 1) / rows_per_cta;
          if (ctas > 8LL * sms) ctas = 8LL * sms;
          if (static_cast<int64_t>(lpr) * nv == nvec && lpr >= 8 / nv && p.keep_sizes[1] == 1 && p.keep_sizes[2] == 1) {
            const unsigned grid = static_cast<unsigned>(ctas);
            switch (nv) {
              case 1: red_rows_pow2_kernel<IO, F, A, kVec, 1><<<grid, 256, 0, st>>>(p, lpr); break;
              case 2: red_rows_pow2_kernel<IO, F, A, kVec, 2><<<grid, 256, 0, st>>>(p, lpr); break;
              case 4: red_rows_pow2_kernel<IO, F, A, kVec, 4><<<grid, 256, 0, st>>>(p, lpr); break;
              default: red_rows_pow2_kernel<IO, F, A, kVec, 8><<<grid, 256, 0, st>>>(p, lpr); break;
            }
            return launch_status();
          }
          red_rows_sub_kernel<IO, F, A, kVec><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p, lpr, nv);
          return launch_status();
        }
        if (nvec * 16 <= g_warp_row_bytes) {
          int64_t ctas = (p.noutputs + 7) / 8;
          if (ctas > 8LL * sms) ctas = 8LL * sms;
          red_rows_warp_vec_kernel<IO, F, A, kVec><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p);
          return launch_status();
        }
      }
    }
    if (p.L <= 1024) {
      const int64_t ctas = (p.noutputs + 7) / 8;
      const int grid = static_cast<int>(ctas < 16LL * sms ? ctas : 16LL * sms);
      red_rows_warp_kernel<IO, F, A, 256><<<grid, 256, 0, st>>>(p);
    } else {
      // one CTA per row while that stays below a few hundred waves: a fresh CTA issues its first loads at once,
      // which keeps more reads in flight than a persistent loop does at its row boundaries
      const int grid = static_cast<int>(p.noutputs < 2048LL * sms ? p.noutputs : 2048LL * sms);
      if (plan.vec_ok) red_rows_cta_kernel<IO, F, A, 8, 256><<<grid, 256, 0, st>>>(p);
      else red_rows_cta_kernel<IO, F, A, 1, 256><<<grid, 256, 0, st>>>(p);
    }
    return launch_status();
  }
  if (plan.path == 1) {
    dim3 grid(p.splits, static_cast<unsigned>(p.noutputs));
    if (plan.vec_ok) red_split_partial_kernel<IO, F, A, 8, 256><<<grid, 256, 0, st>>>(p);
    else red_split_partial_kernel<IO, F, A, 1, 256><<<grid, 256, 0, st>>>(p);
    int rc = launch_status();
    if (rc != SB_OK) return rc;
    const int64_t ctas = (p.noutputs + 7) / 8;
    red_split_final_kernel<F, A><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p);
    return launch_status();
  }
  if (plan.path == 2) {
    const uint64_t outer = static_cast<uint64_t>(p.keep_sizes[1]) * p.keep_sizes[2];
    constexpr int kVec = ColumnVector<IO>::value;
    const int64_t nvec = p.col_vec ? p.keep_sizes[0] / kVec : p.keep_sizes[0];
    dim3 grid(static_cast<unsigned>((nvec + p.vpr - 1) / p.vpr), static_cast<unsigned>(p.splits), static_cast<unsigned>(outer));
    if (p.col_vec) red_cols_kernel<IO, F, A, kVec><<<grid, 256, 0, st>>>(p);
    else red_cols_kernel<IO, F, A, 1><<<grid, 256, 0, st>>>(p);
    int rc = launch_status();
    if (rc != SB_OK || p.splits == 1) return rc;
    int lanes = 1;
    while (lanes < 32 && lanes < p.splits) lanes <<= 1;
    int64_t ctas = (p.noutputs + 8 * (32 / lanes) - 1) / (8 * (32 / lanes));
    if (ctas > 8LL * sms) ctas = 8LL * sms;
    red_cols_final_kernel<F, A><<<static_cast<unsigned>(ctas), 256, 0, st>>>(p, lanes);
    return launch_status();
  }
  int64_t ctas = (plan.g.noutputs + 255) / 256;
  if (ctas > 32LL * sms) ctas = 32LL * sms;
  red_generic_kernel<F, A><<<static_cast<unsigned>(ctas), 256, 0, st>>>(plan.g);
  return launch_status();
}

template <class IO, typename A>
int launch_op(int op, const Plan& plan, cudaStream_t st) {
  switch (op) {
    case SB_RED_SUM: case SB_RED_MEAN: return launch_paths<IO, SumOp<A>, A>(plan, st);
    case SB_RED_AMAX: return launch_paths<IO, MaxOp<A>, A>(plan, st);
    case SB_RED_AMIN: return launch_paths<IO, MinOp<A>, A>(plan, st);
    case SB_RED_PROD: return launch_paths<IO, ProdOp<A>, A>(plan, st);
    case SB_RED_NANSUM: return launch_paths<IO, NanSumOp<A>, A>(plan, st);
    default: return SB_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace

int red_set_warp_row_bytes(int n) {
  if (n != 0 && (n < 4096 || n > 262144)) return SB_ERR_INVALID_ARGUMENT;
  g_warp_row_bytes = n;
  return SB_OK;
}
}  // namespace sb

using namespace sb;

extern "C" {

size_t sb_reduce_scratch_bytes(const sb_reduce_desc* d) {
  Plan plan;
  if (make_plan(d, &plan) != SB_OK) return 0;
  return plan.scratch_bytes;
}

int sb_reduce_path(const sb_reduce_desc* d) {
  Plan plan;
  int rc = make_plan(d, &plan);
  return rc != SB_OK ? rc : plan.path;
}

int sb_reduce(const sb_reduce_desc* d, sb_stream_t stream) {
  Plan plan;
  int rc = make_plan(d, &plan);
  if (rc != SB_OK) return rc;
  if (plan.g.noutputs == 0) return SB_OK;
  if (plan.g.nreduce == 0) return SB_ERR_INVALID_ARGUMENT;  // the caller fills identities for empty reductions
  if (plan.scratch_bytes > 0) {
    if (!d->scratch || d->scratch_bytes < plan.scratch_bytes) return SB_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(d->scratch) % 8) return SB_ERR_MISALIGNED;
  }
  cudaStream_t st = as_stream(stream);
  switch (plan.acc) {
    case 0:
      switch (d->in_dtype) {
        case SB_F32: return launch_op<StaticIO<float>, float>(d->op, plan, st);
        case SB_BF16: return launch_op<StaticIO<__nv_bfloat16>, float>(d->op, plan, st);
        default: return launch_op<StaticIO<__half>, float>(d->op, plan, st);
      }
    case 1: return launch_op<DynamicIO, double>(d->op, plan, st);
    default: return launch_op<DynamicIO, int64_t>(d->op, plan, st);
  }
}

}  // extern "C"

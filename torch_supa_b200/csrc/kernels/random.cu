// Counter-based random fills (Philox4x32-10, Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) driven by
// the (seed, offset) pair a generator hands out (philox_engine_inputs, torch_supa/csrc/aten/SUPAGeneratorImpl.cpp:450-455).
//
// The stream is defined by the element index alone, not by the launch geometry:
//   group g holds elements [g*E, (g+1)*E), E = 4 for element types of up to 4 bytes and 2 for 8-byte types;
//   its four 32-bit words are philox4x32_10(counter = {lo(offset/4), hi(offset/4), lo(g), hi(g)}, key = {lo(seed), hi(seed)});
//   element k of the group is made from word k (E = 4) or from words 2k, 2k+1 (E = 2).
// One fill consumes one 128-bit block per group, so the generator advances its offset by 4 per fill.
// Write-only work: 16-byte stores, one or more groups per thread, grid sized to the SM count.
#include "common.cuh"

namespace sb {

namespace {

constexpr uint32_t kPhiloxM0 = 0xD2511F53u, kPhiloxM1 = 0xCD9E8D57u;
constexpr uint32_t kPhiloxW0 = 0x9E3779B9u, kPhiloxW1 = 0xBB67AE85u;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    // one 32x32 -> 64 multiply per product (both halves are used)
    const uint64_t p0 = static_cast<uint64_t>(kPhiloxM0) * c.x;
    const uint64_t p1 = static_cast<uint64_t>(kPhiloxM1) * c.z;
    c = make_uint4(static_cast<uint32_t>(p1 >> 32) ^ c.y ^ k0, static_cast<uint32_t>(p1), static_cast<uint32_t>(p0 >> 32) ^ c.w ^ k1,
                   static_cast<uint32_t>(p0));
    k0 += kPhiloxW0;
    k1 += kPhiloxW1;
  }
  return c;
}

struct RngParams {
  void* dst;
  int64_t numel;
  double a, b;     // uniform: from, to; normal: mean, std; bernoulli: p
  int64_t low;     // integers: low
  uint64_t range;  // integers: number of values (0 = 2^64)
  uint32_t k0, k1, o0, o1;
};

__device__ __forceinline__ uint4 group_words(const RngParams& p, int64_t g) {
  return philox4x32_10(make_uint4(p.o0, p.o1, static_cast<uint32_t>(g), static_cast<uint32_t>(static_cast<uint64_t>(g) >> 32)),
                       p.k0, p.k1);
}

__device__ __forceinline__ float u24(uint32_t w) { return static_cast<float>(w >> 8) * 0x1p-24f; }
__device__ __forceinline__ double u53(uint32_t lo, uint32_t hi) {
  return static_cast<double>(((static_cast<uint64_t>(hi) << 32) | lo) >> 11) * 0x1p-53;
}

template <typename T> __device__ __forceinline__ T cast_real(float v) { return from_float<T>(v); }
template <typename T> __device__ __forceinline__ T cast_real_d(double v) { return static_cast<T>(v); }

// Each distribution turns the four words of a group into E elements.
template <typename T, int KIND>
struct Dist;

// [from, to): from + u * (to - from), u = 24 (53 for doubles) random bits scaled to [0, 1); a value that rounds up to `to`
// in the element type is replaced by `from` (uniform_impl_, aten/src/ATen/native/DistributionTemplates.h, does the same).
template <typename T>
struct Dist<T, SB_RNG_UNIFORM> {
  static constexpr int E = 4;
  __device__ static void make(const RngParams& p, uint4 w, T* out) {
    const float from = static_cast<float>(p.a), width = static_cast<float>(p.b - p.a);
    const T hi = cast_real<T>(static_cast<float>(p.b));
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      T v = cast_real<T>(fmaf(u24(ws[k]), width, from));
      if (width > 0.f && to_float(v) >= to_float(hi)) v = cast_real<T>(from);
      out[k] = v;
    }
  }
};
template <>
struct Dist<double, SB_RNG_UNIFORM> {
  static constexpr int E = 2;
  __device__ static void make(const RngParams& p, uint4 w, double* out) {
    const double width = p.b - p.a;
    out[0] = fma(u53(w.x, w.y), width, p.a);
    out[1] = fma(u53(w.z, w.w), width, p.a);
    if (width > 0.0) {
      if (out[0] >= p.b) out[0] = p.a;
      if (out[1] >= p.b) out[1] = p.a;
    }
  }
};

// Box-Muller on word pairs: u1 in (0, 1], u2 in [0, 1); z = sqrt(-2 ln u1) * (cos, sin)(2 pi u2).
template <typename T>
struct Dist<T, SB_RNG_NORMAL> {
  static constexpr int E = 4;
  __device__ static void make(const RngParams& p, uint4 w, T* out) {
    const float mean = static_cast<float>(p.a), sd = static_cast<float>(p.b);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float u1 = static_cast<float>((ws[2 * k] >> 8) + 1u) * 0x1p-24f;
      const float r = sqrtf(-2.f * logf(u1)) * sd;  // the accurate logarithm: an approximate one can turn positive next to u1 = 1
      float s, c;
      sincospif(2.f * u24(ws[2 * k + 1]), &s, &c);
      out[2 * k] = cast_real<T>(fmaf(r, c, mean));
      out[2 * k + 1] = cast_real<T>(fmaf(r, s, mean));
    }
  }
};
template <>
struct Dist<double, SB_RNG_NORMAL> {
  static constexpr int E = 2;
  __device__ static void make(const RngParams& p, uint4 w, double* out) {
    const double u1 = static_cast<double>((((static_cast<uint64_t>(w.y) << 32) | w.x) >> 11) + 1ull) * 0x1p-53;
    const double r = sqrt(-2.0 * log(u1)) * p.b;
    double s, c;
    sincospi(2.0 * u53(w.z, w.w), &s, &c);
    out[0] = fma(r, c, p.a);
    out[1] = fma(r, s, p.a);
  }
};

// low + r mod range; r is one word for types of up to 4 bytes, two words for 8-byte types (one when range fits 32 bits,
// as random_from_to_kernel does).
template <typename T>
struct Dist<T, SB_RNG_INTEGER> {
  static constexpr int E = sizeof(T) == 8 ? 2 : 4;
  __device__ static T cast(int64_t v) {
    if constexpr (std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) return from_float<T>(static_cast<float>(v));
    else return static_cast<T>(v);
  }
  __device__ static void make(const RngParams& p, uint4 w, T* out) {
    if constexpr (E == 4) {
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
      const uint32_t range = static_cast<uint32_t>(p.range);  // 0 = 2^32
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = cast(p.low + static_cast<int64_t>(range ? ws[k] % range : ws[k]));
    } else {
      const uint32_t lo[2] = {w.x, w.z}, hi[2] = {w.y, w.w};
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        uint64_t r;
        if (p.range != 0 && p.range <= 0x100000000ull) r = p.range == 0x100000000ull ? lo[k] : lo[k] % static_cast<uint32_t>(p.range);
        else {
          r = (static_cast<uint64_t>(hi[k]) << 32) | lo[k];
          if (p.range) r %= p.range;
        }
        out[k] = cast(static_cast<int64_t>(static_cast<uint64_t>(p.low) + r));
      }
    }
  }
};

// 1 where u < p.
template <typename T>
struct Dist<T, SB_RNG_BERNOULLI> {
  static constexpr int E = sizeof(T) == 8 ? 2 : 4;
  __device__ static T one(bool b) {
    if constexpr (std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) return from_float<T>(b ? 1.f : 0.f);
    else return static_cast<T>(b ? 1 : 0);
  }
  __device__ static void make(const RngParams& p, uint4 w, T* out) {
    if constexpr (E == 4) {
      const float pr = static_cast<float>(p.a);
      out[0] = one(u24(w.x) < pr);
      out[1] = one(u24(w.y) < pr);
      out[2] = one(u24(w.z) < pr);
      out[3] = one(u24(w.w) < pr);
    } else {
      out[0] = one(u53(w.x, w.y) < p.a);
      out[1] = one(u53(w.z, w.w) < p.a);
    }
  }
};

// One thread per 16-byte vector (G groups of E elements); `vectors` full vectors, then the ragged end by the first threads.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) rng_fill_kernel(RngParams p, int64_t vectors) {
  using D = Dist<T, KIND>;
  constexpr int E = D::E;
  constexpr int G = 16 / (E * static_cast<int>(sizeof(T)));
  T* dst = static_cast<T*>(p.dst);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t v = first; v < vectors; v += stride) {
    alignas(16) T out[E * G];
#pragma unroll
    for (int j = 0; j < G; ++j) D::make(p, group_words(p, v * G + j), out + j * E);
    st_stream_u4(dst + v * (E * G), *reinterpret_cast<const uint4*>(out));
  }
  // Elements past the last full vector: one group per thread, element-wise stores.
  const int64_t g0 = vectors * G;
  const int64_t groups = (p.numel + E - 1) / E;
  for (int64_t g = g0 + first; g < groups; g += stride) {
    T out[E];
    D::make(p, group_words(p, g), out);
#pragma unroll
    for (int k = 0; k < E; ++k)
      if (g * E + k < p.numel) dst[g * E + k] = out[k];
  }
}

template <typename T, int KIND>
int launch_fill(const RngParams& p, cudaStream_t st) {
  constexpr int E = Dist<T, KIND>::E;
  constexpr int per_vec = 16 / static_cast<int>(sizeof(T));
  // A destination that does not start on a 16-byte boundary takes the element-wise loop for everything.
  const bool aligned = reinterpret_cast<uintptr_t>(p.dst) % 16 == 0;
  const int64_t vectors = aligned ? p.numel / per_vec : 0;
  const int64_t work = vectors + ((p.numel - vectors * per_vec) + E - 1) / E;
  const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 8;
  int64_t blocks = (work + 255) / 256;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  rng_fill_kernel<T, KIND><<<static_cast<int>(blocks), 256, 0, st>>>(p, vectors);
  return launch_status();
}

template <int KIND>
int dispatch_real(int dtype, const RngParams& p, cudaStream_t st) {
  switch (dtype) {
    case SB_F32: return launch_fill<float, KIND>(p, st);
    case SB_F64: return launch_fill<double, KIND>(p, st);
    case SB_BF16: return launch_fill<__nv_bfloat16, KIND>(p, st);
    case SB_F16: return launch_fill<__half, KIND>(p, st);
    default: return SB_ERR_UNSUPPORTED;
  }
}

template <int KIND>
int dispatch_any(int dtype, const RngParams& p, cudaStream_t st) {
  switch (dtype) {
    case SB_BOOL: return launch_fill<bool, KIND>(p, st);
    case SB_U8: return launch_fill<uint8_t, KIND>(p, st);
    case SB_I8: return launch_fill<int8_t, KIND>(p, st);
    case SB_I16: return launch_fill<int16_t, KIND>(p, st);
    case SB_I32: return launch_fill<int32_t, KIND>(p, st);
    case SB_I64: return launch_fill<int64_t, KIND>(p, st);
    default: return dispatch_real<KIND>(dtype, p, st);
  }
}

// ---- dropout ---------------------------------------------------------------------------------------------------------------
// out = x * keep * scale, mask = keep, keep = (u >= p) with u the uniform of the element's word (same stream as above, E = 4).
struct DropParams {
  const void* x;
  void* out;
  uint8_t* mask;
  int64_t numel;
  float p, scale;
  uint32_t k0, k1, o0, o1;
};

template <typename T>
__global__ void __launch_bounds__(256) dropout_kernel(DropParams p, int64_t vectors) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));  // elements per 16-byte vector
  constexpr int G = V / 4;
  const T* x = static_cast<const T*>(p.x);
  T* out = static_cast<T*>(p.out);
  RngParams rp{};
  rp.k0 = p.k0, rp.k1 = p.k1, rp.o0 = p.o0, rp.o1 = p.o1;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t v = first; v < vectors; v += stride) {
    const uint4 raw = ld_stream_u4(x + v * V);
    alignas(16) T xin[V];
    *reinterpret_cast<uint4*>(xin) = raw;
    alignas(16) T o[V];
    alignas(8) uint8_t m[V];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const uint4 w = group_words(rp, v * G + j);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool keep = u24(ws[k]) >= p.p;
        m[j * 4 + k] = keep ? 1 : 0;
        o[j * 4 + k] = from_float<T>(keep ? to_float(xin[j * 4 + k]) * p.scale : 0.f);
      }
    }
    st_stream_u4(out + v * V, *reinterpret_cast<const uint4*>(o));
    if constexpr (V == 4) *reinterpret_cast<uint32_t*>(p.mask + v * V) = *reinterpret_cast<const uint32_t*>(m);
    else *reinterpret_cast<uint2*>(p.mask + v * V) = *reinterpret_cast<const uint2*>(m);
  }
  const int64_t g0 = vectors * G;
  const int64_t groups = (p.numel + 3) / 4;
  for (int64_t g = g0 + first; g < groups; g += stride) {
    const uint4 w = group_words(rp, g);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t i = g * 4 + k;
      if (i < p.numel) {
        const bool keep = u24(ws[k]) >= p.p;
        p.mask[i] = keep ? 1 : 0;
        out[i] = from_float<T>(keep ? to_float(x[i]) * p.scale : 0.f);
      }
    }
  }
}

template <typename T>
int launch_dropout(const DropParams& p, cudaStream_t st) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  const auto al = [](const void* q, int a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
  const bool aligned = al(p.x, 16) && al(p.out, 16) && al(p.mask, 8);
  const int64_t vectors = aligned ? p.numel / V : 0;
  const int64_t work = vectors + ((p.numel - vectors * V) + 3) / 4;
  const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 8;
  int64_t blocks = (work + 255) / 256;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  dropout_kernel<T><<<static_cast<int>(blocks), 256, 0, st>>>(p, vectors);
  return launch_status();
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" int sb_rng_fill(const sb_rng_args* a, sb_stream_t stream) {
  if (!a || a->numel < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->numel == 0) return SB_OK;
  if (!a->dst) return SB_ERR_INVALID_ARGUMENT;
  if (a->offset % 4) return SB_ERR_INVALID_ARGUMENT;
  const int es = dtype_size(a->dtype);
  if (es <= 0) return SB_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(a->dst) % es) return SB_ERR_MISALIGNED;
  RngParams p;
  p.dst = a->dst;
  p.numel = a->numel;
  p.a = a->a;
  p.b = a->b;
  p.low = a->low;
  p.range = a->range;
  p.k0 = static_cast<uint32_t>(a->seed);
  p.k1 = static_cast<uint32_t>(a->seed >> 32);
  const uint64_t block = a->offset / 4;
  p.o0 = static_cast<uint32_t>(block);
  p.o1 = static_cast<uint32_t>(block >> 32);
  const cudaStream_t st = as_stream(stream);
  switch (a->kind) {
    case SB_RNG_UNIFORM:
      if (!(a->a <= a->b)) return SB_ERR_INVALID_ARGUMENT;
      return dispatch_real<SB_RNG_UNIFORM>(a->dtype, p, st);
    case SB_RNG_NORMAL:
      if (!(a->b >= 0.0)) return SB_ERR_INVALID_ARGUMENT;
      return dispatch_real<SB_RNG_NORMAL>(a->dtype, p, st);
    case SB_RNG_INTEGER:
      if (es < 8 && (a->range == 0 || a->range > 0x100000000ull)) return SB_ERR_INVALID_ARGUMENT;
      if (a->range == 0x100000000ull && es < 8) p.range = 0;  // all 32 bits of the word
      return dispatch_any<SB_RNG_INTEGER>(a->dtype, p, st);
    case SB_RNG_BERNOULLI:
      if (!(a->a >= 0.0 && a->a <= 1.0)) return SB_ERR_INVALID_ARGUMENT;
      return dispatch_any<SB_RNG_BERNOULLI>(a->dtype, p, st);
    default: return SB_ERR_INVALID_ARGUMENT;
  }
}

extern "C" int sb_dropout(const void* x, void* out, void* mask, int32_t dtype, int64_t numel, double p, uint64_t seed,
                          uint64_t offset, sb_stream_t stream) {
  if (numel < 0 || !(p >= 0.0 && p <= 1.0) || offset % 4) return SB_ERR_INVALID_ARGUMENT;
  if (numel == 0) return SB_OK;
  if (!x || !out || !mask) return SB_ERR_INVALID_ARGUMENT;
  if (dtype != SB_F32 && dtype != SB_BF16 && dtype != SB_F16) return SB_ERR_UNSUPPORTED;
  const int es = dtype_size(dtype);
  if (reinterpret_cast<uintptr_t>(x) % es || reinterpret_cast<uintptr_t>(out) % es) return SB_ERR_MISALIGNED;
  DropParams d;
  d.x = x;
  d.out = out;
  d.mask = static_cast<uint8_t*>(mask);
  d.numel = numel;
  d.p = static_cast<float>(p);
  d.scale = p < 1.0 ? static_cast<float>(1.0 / (1.0 - p)) : 0.f;
  d.k0 = static_cast<uint32_t>(seed);
  d.k1 = static_cast<uint32_t>(seed >> 32);
  const uint64_t block = offset / 4;
  d.o0 = static_cast<uint32_t>(block);
  d.o1 = static_cast<uint32_t>(block >> 32);
  switch (dtype) {
    case SB_F32: return launch_dropout<float>(d, as_stream(stream));
    case SB_BF16: return launch_dropout<__nv_bfloat16>(d, as_stream(stream));
    default: return launch_dropout<__half>(d, as_stream(stream));
  }
}

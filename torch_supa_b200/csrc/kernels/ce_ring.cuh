// Device helpers shared by the cross-entropy kernels that keep rows in shared memory: mbarrier / bulk-copy / cluster PTX
// wrappers, packed fp32 pair arithmetic, the per-dtype 16-byte unit codecs and the online-softmax sweeps over loaded units.
#pragma once

#include <type_traits>

#include "ce_common.cuh"

namespace sb {
namespace ring {

constexpr uint32_t kMaxSpin = 1u << 22;  // try_wait attempts (each suspends up to ~1 us) before giving up

// ---- PTX wrappers --------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe of a phase.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kMaxSpin; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NaN-propagating maximum (fmaxf drops a NaN operand; a NaN logit must poison its row as it does on the CPU).
__device__ __forceinline__ float max_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

// ---- packed fp32 pairs (sm_100) -----------------------------------------------------------------------
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// 2^y for a pair, y <= 0 (clamped at -127, where the result is 0), entirely on the FMA and integer pipes:
// y = j + f with j the nearest integer (magic-number rounding), a minimax polynomial of degree DEG for 2^f on
// [-0.5, 0.5], times 2^j built in the exponent field.  Relative error 7.5e-5 (DEG 3), 2.7e-6 (DEG 4), 2.4e-7 (DEG 5).  The 16-bit
// kernels send one pair in four this way because their sweeps are bound by the special-function unit.  A NaN
// argument does not come out as NaN here: the callers make NaN rows NaN through the other three pairs.
template <int DEG>
__device__ __forceinline__ float2 ex2_poly2(float2 y) {
  y.x = fmaxf(y.x, -127.f);  // j = -127 turns the scale below into +0: arguments down to -inf give exactly 0
  y.y = fmaxf(y.y, -127.f);
  const float2 magic = make_float2(12582912.f, 12582912.f);  // 1.5 * 2^23: the sum's mantissa holds round(y)
  const float2 r = add2(y, magic);
  const float2 j = add2(r, make_float2(-12582912.f, -12582912.f));
  const float2 f = fma2(j, make_float2(-1.f, -1.f), y);
  float2 p;
  if (DEG == 3) {
    p = fma2(make_float2(0.05517163872718811f, 0.05517163872718811f), f, make_float2(0.2426111251115799f, 0.2426111251115799f));
    p = fma2(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
    p = fma2(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
  } else if (DEG == 4) {
    p = fma2(make_float2(0.009570098482072353f, 0.009570098482072353f), f, make_float2(0.05591785907745361f, 0.05591785907745361f));
    p = fma2(p, f, make_float2(0.240247443318367f, 0.240247443318367f));
    p = fma2(p, f, make_float2(0.6931217908859253f, 0.6931217908859253f));
    p = fma2(p, f, make_float2(0.9999992847442627f, 0.9999992847442627f));
  } else {
    p = fma2(make_float2(0.0013276468962430954f, 0.0013276468962430954f), f, make_float2(0.009675540961325169f, 0.009675540961325169f));
    p = fma2(p, f, make_float2(0.05550713464617729f, 0.05550713464617729f));
    p = fma2(p, f, make_float2(0.24022120237350464f, 0.24022120237350464f));
    p = fma2(p, f, make_float2(0.6931469440460205f, 0.6931469440460205f));
    p = fma2(p, f, make_float2(1.0000001192092896f, 1.0000001192092896f));
  }
  // 2^j as a float: exponent field 127 + j (the bits of r above the integer part shift out)
  const float2 scale = make_float2(__int_as_float((__float_as_int(r.x) << 23) + 0x3f800000),
                                   __int_as_float((__float_as_int(r.y) << 23) + 0x3f800000));
  return mul2(p, scale);
}

// 16 bytes of T as fp32 pairs.
template <typename T> struct Unit;
template <> struct Unit<float> {
  static constexpr int kPairs = 2;
  static constexpr int kPolyDeg = 0;  // 4-byte elements: the sweeps are bound by memory, every exponential is an ex2
  __device__ static __forceinline__ void unpack(const uint4& r, float2 (&f)[2]) {
    f[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
    f[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
  }
  __device__ static __forceinline__ uint4 pack(const float2 (&f)[2]) {
    return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x), __float_as_uint(f[1].y));
  }
  __device__ static __forceinline__ float vmax(const uint4& r) {
    return max_nan(max_nan(__uint_as_float(r.x), __uint_as_float(r.y)), max_nan(__uint_as_float(r.z), __uint_as_float(r.w)));
  }
};
template <> struct Unit<__nv_bfloat16> {
  static constexpr int kPairs = 4;
  static constexpr int kPolyDeg = 3;  // polynomial degree of the gradient sweep's offloaded pair (8-bit significand out)
  __device__ static __forceinline__ void unpack(const uint4& r, float2 (&f)[4]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  }
  __device__ static __forceinline__ uint4 pack(const float2 (&f)[4]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[i].x, f[i].y);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  // maximum of the 8 values with packed bf16 maxima, widened once at the end
  __device__ static __forceinline__ float vmax(const uint4& r) {
    const __nv_bfloat162 a = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&r.x), *reinterpret_cast<const __nv_bfloat162*>(&r.y));
    const __nv_bfloat162 b = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&r.z), *reinterpret_cast<const __nv_bfloat162*>(&r.w));
    const __nv_bfloat162 c = __hmax2_nan(a, b);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&c);
    return max_nan(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
};
template <> struct Unit<__half> {
  static constexpr int kPairs = 4;
  static constexpr int kPolyDeg = 4;  // 11-bit significand out
  __device__ static __forceinline__ void unpack(const uint4& r, float2 (&f)[4]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
  }
  __device__ static __forceinline__ uint4 pack(const float2 (&f)[4]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[i].x, f[i].y);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static __forceinline__ float vmax(const uint4& r) {
    const __half2 a = __hmax2_nan(*reinterpret_cast<const __half2*>(&r.x), *reinterpret_cast<const __half2*>(&r.y));
    const __half2 b = __hmax2_nan(*reinterpret_cast<const __half2*>(&r.z), *reinterpret_cast<const __half2*>(&r.w));
    const float2 c = __half22float2(__hmax2_nan(a, b));
    return max_nan(c.x, c.y);
  }
};

#ifndef SB_CE_POLY_PAIRS
#define SB_CE_POLY_PAIRS 0
#endif
// Pairs per 16-byte vector of 16-bit logits whose exponentials go through ex2_poly2 instead of the special-function unit.
// Measured on B200: one pair gains 1 % for a short burst and loses 3 % under sustained load, where the 1000 W cap lowers
// the clock as the instruction count rises; the default is therefore 0.
constexpr int kPolyPairs = SB_CE_POLY_PAIRS;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(uint32_t id, uint32_t threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// (max2, sum) merge in base 2 with empty partials (-inf, 0) kept neutral.
__device__ __forceinline__ void merge2(float& m, float& s, float om, float os) {
  const float nm = fmaxf(m, om);
  const float a = (m == -CUDART_INF_F) ? 0.f : s * ex2(m - nm);
  const float b = (om == -CUDART_INF_F) ? 0.f : os * ex2(om - nm);
  m = nm;
  s = a + b;
}

// Per-thread online-softmax state in base 2: two packed accumulators to shorten the dependent chains.
struct RowStats {
  float m2;
  float2 s[2];
  float2 sx[2];
};

// Folds NV vectors (already loaded) into the statistics.
// kKeep: also return the exponentials 2^(x log2e - m2) packed in the storage type (m2 = the maximum after this update).
template <typename T, int NV, bool kSumX, bool kKeep = false>
__device__ __forceinline__ void stats_update(RowStats& st, const uint4 (&r)[NV], uint4* kept = nullptr) {
  using U = Unit<T>;
  constexpr int P = U::kPairs;
  float vm = U::vmax(r[0]);
#pragma unroll
  for (int q = 1; q < NV; ++q) vm = max_nan(vm, U::vmax(r[q]));
  // Logits may be -inf (masked classes): keep (-inf) - (-inf) out of the arithmetic.  A NaN logit makes the
  // maximum NaN, and with it every term below.
  const float nm = max_nan(st.m2, vm * kLog2e);
  const float resc = ex2(nm == -CUDART_INF_F ? 0.f : st.m2 - nm);  // m2 = -inf < nm: the sums are 0, ex2(-inf) = 0
  const float2 resc2 = make_float2(resc, resc);
  st.s[0] = mul2(st.s[0], resc2);
  st.s[1] = mul2(st.s[1], resc2);
  st.m2 = nm;
  const float mm = (nm == -CUDART_INF_F) ? 0.f : nm;
  const float2 negm = make_float2(-mm, -mm);
  const float2 l2e2 = make_float2(kLog2e, kLog2e);
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    float2 f[P];
    U::unpack(r[q], f);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const float2 y = fma2(f[i], l2e2, negm);
      // one pair in four of a 16-bit vector goes through the FMA pipe (degree 5: the sum feeds an fp32 loss)
      const float2 e = (U::kPolyDeg && i >= P - kPolyPairs) ? ex2_poly2<5>(y) : make_float2(ex2(y.x), ex2(y.y));
      st.s[i & 1] = add2(st.s[i & 1], e);
      if (kSumX) st.sx[i & 1] = add2(st.sx[i & 1], f[i]);
      if (kKeep) f[i] = e;
    }
    if (kKeep) kept[q] = U::pack(f);
  }
}

// Gradient of one vector from its kept exponentials: e * factor - sub.
template <typename T>
__device__ __forceinline__ uint4 grad_from_kept(const uint4& r, float2 factor2, float2 nsub2) {
  using U = Unit<T>;
  constexpr int P = U::kPairs;
  float2 f[P];
  U::unpack(r, f);
#pragma unroll
  for (int i = 0; i < P; ++i) f[i] = fma2(f[i], factor2, nsub2);
  return U::pack(f);
}

// The same on bf16 pairs directly: one packed FMA per pair instead of unpack + fp32 FMA + pack.  The factor and the
// smoothing share are rounded to bf16 first (2^-9 relative each, on top of the 2^-9 of the kept value and of the
// result); the class of the target is patched separately from fp32 arithmetic.
__device__ __forceinline__ uint4 grad_from_kept_bf16(const uint4& r, __nv_bfloat162 factor, __nv_bfloat162 nsub) {
  uint4 o;
  const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&r);
  __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = __hfma2(in[i], factor, nsub);
  return o;
}

// Gradient of one vector: (2^(x log2e - lse2)) * scale - sub.
template <typename T>
__device__ __forceinline__ uint4 grad_vector(const uint4& r, float2 neg_lse2, float2 scale2, float2 nsub2) {
  using U = Unit<T>;
  constexpr int P = U::kPairs;
  const float2 l2e2 = make_float2(kLog2e, kLog2e);
  float2 f[P];
  U::unpack(r, f);
#pragma unroll
  for (int i = 0; i < P; ++i) {
    const float2 y = fma2(f[i], l2e2, neg_lse2);
    const float2 e = (U::kPolyDeg && i >= P - kPolyPairs) ? ex2_poly2<U::kPolyDeg ? U::kPolyDeg : 3>(y) : make_float2(ex2(y.x), ex2(y.y));
    f[i] = fma2(e, scale2, nsub2);
  }
  return U::pack(f);
}

// MODE 0: cross entropy (gradient out).  MODE 1: log_softmax (x - lse out; no targets, no losses).  MODE 2: softmax
// (exp(x - lse) out: the gradient formula with scale 1 and nothing subtracted).
// log_softmax of one vector: x - lse.
template <typename T>
__device__ __forceinline__ uint4 shift_vector(const uint4& r, float2 neg_lse) {
  using U = Unit<T>;
  constexpr int P = U::kPairs;
  float2 f[P];
  U::unpack(r, f);
#pragma unroll
  for (int i = 0; i < P; ++i) f[i] = add2(f[i], neg_lse);
  return U::pack(f);
}

}  // namespace ring
}  // namespace sb

// Typed and dtype-switched loads/stores into a compute type.  Used by the elementwise engine and
// the reductions.  A vector access moves VEC consecutive elements with the widest aligned
// instruction the element size allows (16 bytes per piece).
#pragma once

#include <type_traits>

#include "common.cuh"

namespace sb {

// ---- value conversion -----------------------------------------------------------------------------
// C++ conversion semantics (what static_cast does on the host), except bool which is `!= 0`.
template <typename To, typename From>
__device__ __forceinline__ To convert(From v) {
  return static_cast<To>(v);
}
template <> __device__ __forceinline__ float convert<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float convert<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ double convert<double, __half>(__half v) { return static_cast<double>(__half2float(v)); }
template <> __device__ __forceinline__ double convert<double, __nv_bfloat16>(__nv_bfloat16 v) { return static_cast<double>(__bfloat162float(v)); }
template <> __device__ __forceinline__ int32_t convert<int32_t, __half>(__half v) { return static_cast<int32_t>(__half2float(v)); }
template <> __device__ __forceinline__ int32_t convert<int32_t, __nv_bfloat16>(__nv_bfloat16 v) { return static_cast<int32_t>(__bfloat162float(v)); }
template <> __device__ __forceinline__ int64_t convert<int64_t, __half>(__half v) { return static_cast<int64_t>(__half2float(v)); }
template <> __device__ __forceinline__ int64_t convert<int64_t, __nv_bfloat16>(__nv_bfloat16 v) { return static_cast<int64_t>(__bfloat162float(v)); }
template <> __device__ __forceinline__ bool convert<bool, __half>(__half v) { return __half2float(v) != 0.f; }
template <> __device__ __forceinline__ bool convert<bool, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v) != 0.f; }
template <> __device__ __forceinline__ bool convert<bool, float>(float v) { return v != 0.f; }
template <> __device__ __forceinline__ bool convert<bool, double>(double v) { return v != 0.0; }

template <> __device__ __forceinline__ __half convert<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 convert<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half convert<__half, double>(double v) { return __double2half(v); }
template <> __device__ __forceinline__ __nv_bfloat16 convert<__nv_bfloat16, double>(double v) { return __double2bfloat16(v); }
template <> __device__ __forceinline__ __half convert<__half, int32_t>(int32_t v) { return __float2half_rn(static_cast<float>(v)); }
template <> __device__ __forceinline__ __nv_bfloat16 convert<__nv_bfloat16, int32_t>(int32_t v) { return __float2bfloat16_rn(static_cast<float>(v)); }
template <> __device__ __forceinline__ __half convert<__half, int64_t>(int64_t v) { return __float2half_rn(static_cast<float>(v)); }
template <> __device__ __forceinline__ __nv_bfloat16 convert<__nv_bfloat16, int64_t>(int64_t v) { return __float2bfloat16_rn(static_cast<float>(v)); }
template <> __device__ __forceinline__ __half convert<__half, bool>(bool v) { return __float2half_rn(v ? 1.f : 0.f); }
template <> __device__ __forceinline__ __nv_bfloat16 convert<__nv_bfloat16, bool>(bool v) { return __float2bfloat16_rn(v ? 1.f : 0.f); }
// float -> uint8 goes through a signed integer, which is what x86 produces for negative inputs.
template <> __device__ __forceinline__ uint8_t convert<uint8_t, float>(float v) { return static_cast<uint8_t>(static_cast<int32_t>(v)); }
template <> __device__ __forceinline__ uint8_t convert<uint8_t, double>(double v) { return static_cast<uint8_t>(static_cast<int32_t>(v)); }

// Storage type of a dtype code; bool is stored as one byte holding 0 or 1.
struct BoolByte {
  uint8_t b;
};
template <typename To> __device__ __forceinline__ To convert_from_boolbyte(BoolByte v) { return convert<To, bool>(v.b != 0); }

// ---- vector pieces ---------------------------------------------------------------------------------
template <typename S, int VEC>
struct PieceOf {
  static constexpr int kBytes = sizeof(S) * VEC;
  static constexpr int kPieceBytes = kBytes >= 16 ? 16 : kBytes;
  static constexpr int kPieces = kBytes / kPieceBytes;
  static constexpr int kPerPiece = kPieceBytes / sizeof(S);
};

template <int BYTES> struct RawPiece;
template <> struct RawPiece<16> { using type = uint4; };
template <> struct RawPiece<8> { using type = uint2; };
template <> struct RawPiece<4> { using type = uint32_t; };
template <> struct RawPiece<2> { using type = uint16_t; };
template <> struct RawPiece<1> { using type = uint8_t; };

// 32-bit words of a raw piece, by value (keeps everything in registers: no pointer into a local array).
template <int NW> struct Words { uint32_t w[NW]; };
__device__ __forceinline__ Words<4> words_of(const uint4& r) { return Words<4>{{r.x, r.y, r.z, r.w}}; }
__device__ __forceinline__ Words<2> words_of(const uint2& r) { return Words<2>{{r.x, r.y}}; }
__device__ __forceinline__ Words<1> words_of(const uint32_t& r) { return Words<1>{{r}}; }
__device__ __forceinline__ uint4 raw_of(const Words<4>& w) { return make_uint4(w.w[0], w.w[1], w.w[2], w.w[3]); }
__device__ __forceinline__ uint2 raw_of(const Words<2>& w) { return make_uint2(w.w[0], w.w[1]); }
__device__ __forceinline__ uint32_t raw_of(const Words<1>& w) { return w.w[0]; }

template <typename S> struct Is16BitFloat { static constexpr bool value = std::is_same<S, __half>::value || std::is_same<S, __nv_bfloat16>::value; };

// One 32-bit word holding two 16-bit floats <-> two fp32 values.  bf16 widens with a shift and a mask, fp16
// with one packed conversion; both narrow with one packed round-to-nearest-even conversion.
template <typename S> __device__ __forceinline__ float2 widen_pair(uint32_t w) {
  if constexpr (std::is_same<S, __nv_bfloat16>::value) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    __half2 h;
    *reinterpret_cast<uint32_t*>(&h) = w;
    return __half22float2(h);
  }
}
template <typename S> __device__ __forceinline__ uint32_t narrow_pair(float a, float b) {
  if constexpr (std::is_same<S, __nv_bfloat16>::value) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// Loads VEC elements of storage type S starting at p (aligned to PieceOf::kPieceBytes) and converts
// them to CT.
template <typename CT, typename S, int VEC>
__device__ __forceinline__ void load_as(const void* p, CT (&out)[VEC]) {
  using P = PieceOf<S, VEC>;
  using Raw = typename RawPiece<P::kPieceBytes>::type;
#pragma unroll
  for (int i = 0; i < P::kPieces; ++i) {
    const Raw raw = static_cast<const Raw*>(p)[i];
    if constexpr (std::is_same<CT, float>::value && Is16BitFloat<S>::value && P::kPieceBytes >= 4) {
      const auto ws = words_of(raw);
#pragma unroll
      for (int k = 0; k < P::kPieceBytes / 4; ++k) {
        const float2 f = widen_pair<S>(ws.w[k]);
        out[i * P::kPerPiece + 2 * k] = f.x;
        out[i * P::kPerPiece + 2 * k + 1] = f.y;
      }
    } else if constexpr (sizeof(S) == 4 && P::kPieceBytes >= 4) {
      const auto ws = words_of(raw);
#pragma unroll
      for (int k = 0; k < P::kPerPiece; ++k) {
        S v;
        static_assert(sizeof(S) == sizeof(uint32_t), "");
        memcpy(&v, &ws.w[k], 4);
        out[i * P::kPerPiece + k] = convert<CT, S>(v);
      }
    } else {
      union {
        Raw raw;
        S s[P::kPerPiece];
      } u;
      u.raw = raw;
#pragma unroll
      for (int k = 0; k < P::kPerPiece; ++k) out[i * P::kPerPiece + k] = convert<CT, S>(u.s[k]);
    }
  }
}
template <typename CT, int VEC>
__device__ __forceinline__ void load_bool_as(const void* p, CT (&out)[VEC]) {
  uint8_t tmp[VEC];
  load_as<uint8_t, uint8_t, VEC>(p, tmp);
#pragma unroll
  for (int k = 0; k < VEC; ++k) out[k] = convert<CT, bool>(tmp[k] != 0);
}

template <typename CT, typename S, int VEC>
__device__ __forceinline__ void store_as(void* p, const CT (&in)[VEC]) {
  using P = PieceOf<S, VEC>;
  using Raw = typename RawPiece<P::kPieceBytes>::type;
#pragma unroll
  for (int i = 0; i < P::kPieces; ++i) {
    if constexpr (std::is_same<CT, float>::value && Is16BitFloat<S>::value && P::kPieceBytes >= 4) {
      Words<P::kPieceBytes / 4> ws;
#pragma unroll
      for (int k = 0; k < P::kPieceBytes / 4; ++k)
        ws.w[k] = narrow_pair<S>(in[i * P::kPerPiece + 2 * k], in[i * P::kPerPiece + 2 * k + 1]);
      static_cast<Raw*>(p)[i] = raw_of(ws);
    } else if constexpr (sizeof(S) == 4 && P::kPieceBytes >= 4) {
      Words<P::kPieceBytes / 4> ws;
#pragma unroll
      for (int k = 0; k < P::kPerPiece; ++k) {
        const S v = convert<S, CT>(in[i * P::kPerPiece + k]);
        memcpy(&ws.w[k], &v, 4);
      }
      static_cast<Raw*>(p)[i] = raw_of(ws);
    } else {
      union {
        Raw raw;
        S s[P::kPerPiece];
      } u;
#pragma unroll
      for (int k = 0; k < P::kPerPiece; ++k) u.s[k] = convert<S, CT>(in[i * P::kPerPiece + k]);
      static_cast<Raw*>(p)[i] = u.raw;
    }
  }
}
template <typename CT, int VEC>
__device__ __forceinline__ void store_bool_as(void* p, const CT (&in)[VEC]) {
  uint8_t tmp[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) tmp[k] = convert<bool, CT>(in[k]) ? 1 : 0;
  store_as<uint8_t, uint8_t, VEC>(p, tmp);
}

// ---- IO policies -----------------------------------------------------------------------------------
// StaticIO<T>: every operand is stored as T (no type promotion).  DynamicIO: the storage type of each
// operand is a runtime sb_dtype; the switch is uniform across the grid.
template <typename T>
struct StaticIO {
  static constexpr bool kDynamic = false;
  using storage = T;
  template <typename CT, int VEC>
  __device__ static __forceinline__ void load(const void* base, int64_t elem, int /*dtype*/, CT (&out)[VEC]) {
    load_as<CT, T, VEC>(static_cast<const T*>(base) + elem, out);
  }
  template <typename CT, int VEC>
  __device__ static __forceinline__ void store(void* base, int64_t elem, int /*dtype*/, const CT (&in)[VEC]) {
    store_as<CT, T, VEC>(static_cast<T*>(base) + elem, in);
  }
};

struct DynamicIO {
  static constexpr bool kDynamic = true;
  using storage = void;
  template <typename CT, int VEC>
  __device__ static __forceinline__ void load(const void* base, int64_t elem, int dtype, CT (&out)[VEC]) {
    const char* b = static_cast<const char*>(base);
    switch (dtype) {
      case SB_BOOL: load_bool_as<CT, VEC>(b + elem, out); break;
      case SB_U8: load_as<CT, uint8_t, VEC>(b + elem, out); break;
      case SB_I8: load_as<CT, int8_t, VEC>(b + elem, out); break;
      case SB_I16: load_as<CT, int16_t, VEC>(b + elem * 2, out); break;
      case SB_I32: load_as<CT, int32_t, VEC>(b + elem * 4, out); break;
      case SB_I64: load_as<CT, int64_t, VEC>(b + elem * 8, out); break;
      case SB_F16: load_as<CT, __half, VEC>(b + elem * 2, out); break;
      case SB_BF16: load_as<CT, __nv_bfloat16, VEC>(b + elem * 2, out); break;
      case SB_F32: load_as<CT, float, VEC>(b + elem * 4, out); break;
      default: load_as<CT, double, VEC>(b + elem * 8, out); break;
    }
  }
  template <typename CT, int VEC>
  __device__ static __forceinline__ void store(void* base, int64_t elem, int dtype, const CT (&in)[VEC]) {
    char* b = static_cast<char*>(base);
    switch (dtype) {
      case SB_BOOL: store_bool_as<CT, VEC>(b + elem, in); break;
      case SB_U8: store_as<CT, uint8_t, VEC>(b + elem, in); break;
      case SB_I8: store_as<CT, int8_t, VEC>(b + elem, in); break;
      case SB_I16: store_as<CT, int16_t, VEC>(b + elem * 2, in); break;
      case SB_I32: store_as<CT, int32_t, VEC>(b + elem * 4, in); break;
      case SB_I64: store_as<CT, int64_t, VEC>(b + elem * 8, in); break;
      case SB_F16: store_as<CT, __half, VEC>(b + elem * 2, in); break;
      case SB_BF16: store_as<CT, __nv_bfloat16, VEC>(b + elem * 2, in); break;
      case SB_F32: store_as<CT, float, VEC>(b + elem * 4, in); break;
      default: store_as<CT, double, VEC>(b + elem * 8, in); break;
    }
  }
};

}  // namespace sb

// Shared device/host helpers of the sm_100a kernel library: element types, 128-bit vector access,
// warp/CTA reductions, launch-geometry constants.  No ATen or torch includes anywhere below this
// directory: the library is plain CUDA behind a C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "supa_b200_kernels.h"

namespace sb {

// B200: 148 SMs on two dies.  Persistent grids are sized from the live device, this is only the
// fallback when the attribute query fails.
constexpr int kDefaultSmCount = 148;

int sm_count();                 // multiprocessors of the current device (cached per device)
int max_smem_optin();           // cudaDevAttrMaxSharedMemoryPerBlockOptin of the current device
int launch_status();            // cudaGetLastError() -> sb_status

inline cudaStream_t as_stream(sb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- element type traits ----------------------------------------------------------------------
template <typename T> struct DTypeOf;
template <> struct DTypeOf<bool> { static constexpr int value = SB_BOOL; };
template <> struct DTypeOf<uint8_t> { static constexpr int value = SB_U8; };
template <> struct DTypeOf<int8_t> { static constexpr int value = SB_I8; };
template <> struct DTypeOf<int16_t> { static constexpr int value = SB_I16; };
template <> struct DTypeOf<int32_t> { static constexpr int value = SB_I32; };
template <> struct DTypeOf<int64_t> { static constexpr int value = SB_I64; };
template <> struct DTypeOf<__half> { static constexpr int value = SB_F16; };
template <> struct DTypeOf<__nv_bfloat16> { static constexpr int value = SB_BF16; };
template <> struct DTypeOf<float> { static constexpr int value = SB_F32; };
template <> struct DTypeOf<double> { static constexpr int value = SB_F64; };

__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case SB_BOOL: case SB_U8: case SB_I8: return 1;
    case SB_I16: case SB_F16: case SB_BF16: return 2;
    case SB_I32: case SB_F32: return 4;
    case SB_I64: case SB_F64: return 8;
    default: return 0;
  }
}

// ---- scalar conversions (to/from the fp32 math type) -------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(double v) { return static_cast<float>(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ double from_float<double>(float v) { return static_cast<double>(v); }

// ---- 128-bit vectors ---------------------------------------------------------------------------
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec(const T* p) {
  return *reinterpret_cast<const Vec<T, N>*>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T* p, const Vec<T, N>& v) {
  *reinterpret_cast<Vec<T, N>*>(p) = v;
}

// Streaming (evict-first) 16-byte global accesses for write-once / read-once data.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream_u4(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// launch_dependents lets the next kernel of the stream start while this one still runs, provided that kernel
// was launched with the programmatic-stream-serialization attribute; grid_dep_wait, executed in such a kernel,
// returns once every kernel before it in the stream has completed and its writes are visible.  Both are no-ops
// in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- reductions --------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// (max, sum-of-exp) pair of an online softmax; `merge` folds b into a.
struct MaxSum {
  float m;
  float s;
};
__device__ __forceinline__ MaxSum merge(MaxSum a, MaxSum b) {
  // exp(-inf - -inf) would be NaN: an empty partial (m = -inf, s = 0) must stay neutral.
  float m = fmaxf(a.m, b.m);
  float sa = (a.m == -CUDART_INF_F) ? 0.f : a.s * expf(a.m - m);
  float sb_ = (b.m == -CUDART_INF_F) ? 0.f : b.s * expf(b.m - m);
  return MaxSum{m, sa + sb_};
}
__device__ __forceinline__ MaxSum warp_merge(MaxSum v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = merge(v, other);
  }
  return v;
}

// ---- exp -----------------------------------------------------------------------------------------
// exp for fp32 element types: the CUDA library expf (2 ulp), not the ex2.approx shortcut, whose error
// grows with |x| and would show in fp32 parity.
__device__ __forceinline__ float exp_accurate(float x) { return expf(x); }
// exp for 16-bit element types: the result is rounded to 8 or 11 bits anyway.
__device__ __forceinline__ float exp_fast(float x) { return __expf(x); }

}  // namespace sb

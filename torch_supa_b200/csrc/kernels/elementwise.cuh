// Elementwise engine: functors, the four launch paths and the host-side classifier.
//
// Path 0  contiguous    every operand is a dense 1-D run: 8 elements per thread per access, two
//                       accesses in flight per operand, scalar tail.
// Path 1  rows          unit (or zero) stride along the fastest dimension for every operand, anything
//                       along the outer ones (broadcast rows, row-strided views): vector accesses along
//                       the row, the outer index is decomposed once per thread.
// Path 2  transpose     the output runs along dimension 0 while some input runs along dimension 1: that
//                       input is staged through a shared-memory tile so that both sides stay coalesced.
// Path 3  generic       per-element offset arithmetic for anything else (up to SB_MAX_DIMS dimensions).
#pragma once

#include <type_traits>

#include "io.cuh"

namespace sb {

constexpr int kEwVec = 8;        // elements per vector access
constexpr int kEwThreads = 256;
constexpr int kEwRowDims = 4;    // path 1 handles up to this many dimensions

struct EwParams {
  void* data[SB_MAX_OPERANDS];
  int dtype[SB_MAX_OPERANDS];
  int64_t strides[SB_MAX_OPERANDS][kEwRowDims];  // elements
  uint32_t sizes[kEwRowDims];
  int64_t numel;          // path 0
  uint32_t row_chunks;    // path 1: blocks along one row
  uint32_t span;          // path 1: vectors of the row one block walks
  int bcast;              // path 1: some input has stride 0 along the row
  uint32_t rows;          // path 1: product of sizes[1..]
  int bx;                 // path 1: threads along the row (power of two), by = kEwThreads / bx
  int unroll;             // path 1: vectors per thread along the row
  int op;                 // runtime op code for paths 2 and 3
  double alpha, scalar;
  int64_t ialpha, iscalar;
};

struct EwGenericParams {
  void* data[SB_MAX_OPERANDS];
  int dtype[SB_MAX_OPERANDS];
  int ndim;
  int noperands;
  int op;
  uint32_t sizes[SB_MAX_DIMS];
  int64_t strides[SB_MAX_OPERANDS][SB_MAX_DIMS];
  int64_t numel;
  double alpha, scalar;
  int64_t ialpha, iscalar;
};

// ---- scalars carried by a functor, in the compute type --------------------------------------------------
template <typename CT> struct OpScalars {
  CT alpha;
  CT scalar;
};
template <typename CT, typename P>
__device__ __forceinline__ OpScalars<CT> make_scalars(const P& p) {
  if constexpr (std::is_floating_point<CT>::value) {
    return OpScalars<CT>{static_cast<CT>(p.alpha), static_cast<CT>(p.scalar)};
  } else if constexpr (std::is_same<CT, bool>::value) {
    return OpScalars<CT>{p.ialpha != 0 || p.alpha != 0.0, p.iscalar != 0 || p.scalar != 0.0};
  } else {
    return OpScalars<CT>{static_cast<CT>(p.ialpha), static_cast<CT>(p.iscalar)};
  }
}

// ---- math helpers ------------------------------------------------------------------------------------------
// FAST selects the single-MUFU approximations; it is used when the result is rounded to bf16, whose
// 8-bit significand hides their 2^-11 relative error.
template <bool FAST> __device__ __forceinline__ float tanh_f(float x) {
  if constexpr (FAST) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  } else {
    return tanhf(x);
  }
}
__device__ __forceinline__ double tanh_f(double x) { return tanh(x); }

template <bool FAST> __device__ __forceinline__ float sigmoid_f(float x) {
  if constexpr (FAST) {
    return fmaf(tanh_f<true>(0.5f * x), 0.5f, 0.5f);
  } else {
    return 1.f / (1.f + expf(-x));
  }
}
__device__ __forceinline__ double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }

template <bool FAST, typename CT> __device__ __forceinline__ CT sigmoid_t(CT x) {
  if constexpr (std::is_same<CT, double>::value) return sigmoid_d(x);
  else return sigmoid_f<FAST>(x);
}
template <bool FAST, typename CT> __device__ __forceinline__ CT tanh_t(CT x) {
  if constexpr (std::is_same<CT, double>::value) return tanh(x);
  else return tanh_f<FAST>(x);
}
// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7): one reciprocal, one ex2 and five FMAs; used when the
// result is rounded to bf16.  `e` receives exp(-x^2), which the gelu derivative needs as well.
__device__ __forceinline__ float erf_fast(float x, float& e) {
  const float ax = fabsf(x);
  const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  e = exp2f(-ax * ax * 1.4426950408889634f);
  const float r = fmaf(-poly * t, e, 1.f);
  return copysignf(r, x);
}
// gelu(x) = x Phi(x) for results that are rounded to bf16, with one special-function instruction and no reciprocal:
// with z = |x| / sqrt 2, erfc(z) = 2^q(z), q a degree-5 polynomial without constant term fitted to log2 erfc on
// [0, 4] (|error| <= 4.7e-4, i.e. 3.3e-4 relative on erfc); then Phi(-|x|) = erfc(z) / 2 = 2^(q - 1) =: h and
// gelu(x) = x h for x < 0, x (1 - h) for x >= 0.  The relative error of the result stays below 4e-4 everywhere (2^-9 =
// 2e-3 is what bf16 resolves); beyond |x| = 5.66 the argument is clamped, where h < 8e-9.
__device__ __forceinline__ float gelu_erf_fast(float x) {
  const float ax = fminf(fabsf(x), 5.6568542f);
  // coefficients of q in powers of |x| (those in z divided by sqrt(2)^k)
  float p = -2.3073101e-04f;
  p = fmaf(p, ax, 4.8618629e-03f);
  p = fmaf(p, ax, -4.4720481e-02f);
  p = fmaf(p, ax, -4.6900228e-01f);
  p = fmaf(p, ax, -1.1472815f);
  const float qm1 = fmaf(p, ax, -1.f);
  float h;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(h) : "f"(qm1));
  return x * (x < 0.f ? h : 1.f - h);
}

template <bool FAST, typename CT> __device__ __forceinline__ CT erf_t(CT x) {
  if constexpr (std::is_same<CT, double>::value) return erf(x);
  else if constexpr (FAST) {
    float e;
    return erf_fast(x, e);
  } else return erff(x);
}
template <typename CT> __device__ __forceinline__ CT exp_t(CT x) {
  if constexpr (std::is_same<CT, double>::value) return exp(x);
  else return expf(x);
}

// ---- functors --------------------------------------------------------------------------------------------------
// Each functor has `arity` inputs and `apply(a, b, c, scalars)`.
template <int OP, typename CT, bool FAST> struct EwOp;

#define SB_DEFINE_OP(OPCODE, ARITY, ...)                                                         \
  template <typename CT, bool FAST> struct EwOp<OPCODE, CT, FAST> {                             \
    static constexpr int arity = ARITY;                                                         \
    __device__ static __forceinline__ CT apply(CT a, CT b, CT c, const OpScalars<CT>& s) {      \
      (void)a; (void)b; (void)c; (void)s;                                                       \
      __VA_ARGS__                                                                               \
    }                                                                                           \
  };

SB_DEFINE_OP(SB_EW_COPY, 1, return a;)
SB_DEFINE_OP(SB_EW_FILL, 0, return s.scalar;)
SB_DEFINE_OP(SB_EW_ADD, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a || (s.alpha && b);
  else return a + s.alpha * b;
})
SB_DEFINE_OP(SB_EW_MUL, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a && b;
  else return a * b;
})
SB_DEFINE_OP(SB_EW_SUB, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a != (s.alpha && b);
  else return a - s.alpha * b;
})
SB_DEFINE_OP(SB_EW_DIV, 2, {
  if constexpr (std::is_floating_point<CT>::value) return a / b;
  else return a;
})
// trunc(a / b); integers: C division (0 for a zero divisor: nothing traps on the device).
SB_DEFINE_OP(SB_EW_DIV_TRUNC, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a && b;
  else if constexpr (std::is_floating_point<CT>::value) return trunc(a / b);
  else return b == 0 ? CT(0) : (b == CT(-1) ? CT(0) - a : a / b);
})
// Python's floor division.  Floating types: the quotient of (a - fmod(a, b)) by b, one less when the remainder and the
// divisor differ in sign, then floored with the half-way guard of c10::div_floor_floating; a zero divisor gives a / b.
SB_DEFINE_OP(SB_EW_DIV_FLOOR, 2, {
  if constexpr (std::is_same<CT, bool>::value) {
    return a && b;
  } else if constexpr (std::is_floating_point<CT>::value) {
    if (b == CT(0)) return a / b;
    const CT mod = fmod(a, b);
    CT div = (a - mod) / b;
    if (mod != CT(0) && (b < CT(0)) != (mod < CT(0))) div -= CT(1);
    CT floordiv;
    if (div != CT(0)) {
      floordiv = floor(div);
      if (div - floordiv > CT(0.5)) floordiv += CT(1);
    } else {
      floordiv = copysign(CT(0), a / b);
    }
    return floordiv;
  } else {
    if (b == 0) return CT(0);
    if (b == CT(-1)) return CT(0) - a;
    CT q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0))) q -= 1;
    return q;
  }
})
SB_DEFINE_OP(SB_EW_ADD_SCALAR, 1, {
  if constexpr (std::is_same<CT, bool>::value) return a || (s.alpha && s.scalar);
  else return a + s.alpha * s.scalar;
})
SB_DEFINE_OP(SB_EW_MUL_SCALAR, 1, {
  if constexpr (std::is_same<CT, bool>::value) return a && s.scalar;
  else return a * s.scalar;
})
SB_DEFINE_OP(SB_EW_NEG, 1, {
  if constexpr (std::is_same<CT, bool>::value) return a;
  else return -a;
})
// gelu(x) = x * Phi(x), exact (erf) form.
SB_DEFINE_OP(SB_EW_GELU_ERF, 1, {
  if constexpr (FAST && std::is_same<CT, float>::value) return gelu_erf_fast(a);
  else if constexpr (std::is_floating_point<CT>::value) return a * CT(0.5) * (CT(1) + erf_t<FAST, CT>(a * CT(0.70710678118654752440)));
  else return a;
})
// tanh approximation: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).
SB_DEFINE_OP(SB_EW_GELU_TANH, 1, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT kBeta = CT(0.79788456080286535588);  // sqrt(2) * (2/sqrt(pi)) * 0.5
    const CT kKappa = CT(0.044715);
    const CT inner = kBeta * (a + kKappa * a * a * a);
    return CT(0.5) * a * (CT(1) + tanh_t<FAST, CT>(inner));
  } else return a;
})
SB_DEFINE_OP(SB_EW_SILU, 1, {
  if constexpr (std::is_floating_point<CT>::value) return a * sigmoid_t<FAST, CT>(a);
  else return a;
})
// glu: first half times sigmoid of the second half.
SB_DEFINE_OP(SB_EW_GLU, 2, {
  if constexpr (std::is_floating_point<CT>::value) return a * sigmoid_t<FAST, CT>(b);
  else return a;
})
// d gelu_erf: grad * (Phi(x) + x * phi(x));  a = grad, b = x.
SB_DEFINE_OP(SB_EW_GELU_ERF_BWD, 2, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT kAlpha = CT(0.70710678118654752440);
    const CT kBeta = CT(0.39894228040143267794);  // (2/sqrt(pi)) * sqrt(1/2) * 0.5
    if constexpr (FAST && std::is_same<CT, float>::value) {
      float e;  // exp(-(x / sqrt 2)^2) = exp(-x^2 / 2), shared by the cdf and the pdf
      const float cdf = 0.5f * (1.f + erf_fast(b * kAlpha, e));
      return a * (cdf + b * e * kBeta);
    } else {
      const CT cdf = CT(0.5) * (CT(1) + erf_t<false, CT>(b * kAlpha));
      const CT pdf = exp_t<CT>(CT(-0.5) * b * b) * kBeta;
      return a * (cdf + b * pdf);
    }
  } else return a;
})
SB_DEFINE_OP(SB_EW_GELU_TANH_BWD, 2, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT kBeta = CT(0.79788456080286535588);
    const CT kKappa = CT(0.044715);
    const CT x_sq = b * b;
    const CT inner = kBeta * (b + kKappa * x_sq * b);
    const CT th = tanh_t<FAST, CT>(inner);
    const CT left = CT(0.5) * b;
    const CT right = CT(1) + th;
    const CT left_d = CT(0.5) * right;
    const CT tanh_d = CT(1) - th * th;
    const CT inner_d = kBeta * (CT(1) + CT(3) * kKappa * x_sq);
    return a * (left_d + left * tanh_d * inner_d);
  } else return a;
})
// d silu: grad * s * (1 + x (1 - s));  a = grad, b = x.
SB_DEFINE_OP(SB_EW_SILU_BWD, 2, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT sg = sigmoid_t<FAST, CT>(b);
    return a * sg * (CT(1) + b * (CT(1) - sg));
  } else return a;
})
// glu backward, first half: sigmoid(b) * grad;  a = grad, b = second half.
SB_DEFINE_OP(SB_EW_GLU_BWD_A, 2, {
  if constexpr (std::is_floating_point<CT>::value) return sigmoid_t<FAST, CT>(b) * a;
  else return a;
})
// glu backward, second half: (1 - s) s grad a_half;  a = grad, b = second half, c = first half.
SB_DEFINE_OP(SB_EW_GLU_BWD_B, 3, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT sg = sigmoid_t<FAST, CT>(b);
    return (CT(1) - sg) * sg * a * c;
  } else return a;
})
// softplus(-x) = -log(sigmoid(x)) = max(-x, 0) + log1p(exp(-|x|)), the stable form.
template <typename CT> __device__ __forceinline__ CT softplus_neg(CT x) {
  if constexpr (std::is_same<CT, double>::value) return fmax(-x, 0.0) + log1p(exp(-fabs(x)));
  else return fmaxf(-x, 0.f) + log1pf(expf(-fabsf(x)));
}
// binary cross entropy on logits: a = x, b = target [, c = pos_weight]; times alpha.
SB_DEFINE_OP(SB_EW_BCE_LOGITS, 2, {
  if constexpr (std::is_floating_point<CT>::value) return s.alpha * ((CT(1) - b) * a + softplus_neg<CT>(a));
  else return a;
})
SB_DEFINE_OP(SB_EW_BCE_LOGITS_PW, 3, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT lw = (c - CT(1)) * b + CT(1);
    return s.alpha * ((CT(1) - b) * a + lw * softplus_neg<CT>(a));
  } else return a;
})
// its derivative in x: a = x, b = target, c = upstream gradient (no pos_weight) or pos_weight.
// sigmoid for the derivative below: fp32 through ex2 and the approximate reciprocal (relative error about 5e-7 where the
// value is not tiny), so that the kernel stays bound by its three streams.
template <typename CT> __device__ __forceinline__ CT sigmoid_bce(CT x) {
  if constexpr (std::is_same<CT, double>::value) return sigmoid_d(x);
  else {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-x * 1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return r;
  }
}
SB_DEFINE_OP(SB_EW_BCE_LOGITS_BWD, 3, {
  if constexpr (std::is_floating_point<CT>::value) return s.alpha * c * (sigmoid_bce<CT>(a) - b);
  else return a;
})
SB_DEFINE_OP(SB_EW_BCE_LOGITS_PW_BWD, 3, {
  if constexpr (std::is_floating_point<CT>::value) {
    const CT lw = (c - CT(1)) * b + CT(1);
    return s.alpha * (lw * sigmoid_bce<CT>(a) - c * b);
  } else return a;
})
SB_DEFINE_OP(SB_EW_SIGMOID, 1, {
  if constexpr (std::is_floating_point<CT>::value) return sigmoid_t<FAST, CT>(a);
  else return a;
})
SB_DEFINE_OP(SB_EW_TANH, 1, {
  if constexpr (std::is_floating_point<CT>::value) return tanh_t<FAST, CT>(a);
  else return a;
})
SB_DEFINE_OP(SB_EW_EXP, 1, {
  if constexpr (std::is_floating_point<CT>::value) return exp_t<CT>(a);
  else return a;
})
SB_DEFINE_OP(SB_EW_LOG, 1, {
  if constexpr (std::is_same<CT, double>::value) return log(a);
  else if constexpr (std::is_same<CT, float>::value) return logf(a);
  else return a;
})
SB_DEFINE_OP(SB_EW_SIGMOID_BWD, 2, {
  if constexpr (std::is_floating_point<CT>::value) return a * (CT(1) - b) * b;
  else return a;
})
SB_DEFINE_OP(SB_EW_TANH_BWD, 2, {
  if constexpr (std::is_floating_point<CT>::value) return a * (CT(1) - b * b);
  else return a;
})
SB_DEFINE_OP(SB_EW_MAXIMUM, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a || b;
  else if constexpr (std::is_floating_point<CT>::value) return (a != a) ? a : ((b != b) ? b : (a > b ? a : b));
  else return a > b ? a : b;
})
SB_DEFINE_OP(SB_EW_MINIMUM, 2, {
  if constexpr (std::is_same<CT, bool>::value) return a && b;
  else if constexpr (std::is_floating_point<CT>::value) return (a != a) ? a : ((b != b) ? b : (a < b ? a : b));
  else return a < b ? a : b;
})
SB_DEFINE_OP(SB_EW_EQ, 2, return static_cast<CT>(a == b);)
SB_DEFINE_OP(SB_EW_NE, 2, return static_cast<CT>(a != b);)
SB_DEFINE_OP(SB_EW_LT, 2, return static_cast<CT>(a < b);)
SB_DEFINE_OP(SB_EW_LE, 2, return static_cast<CT>(a <= b);)
SB_DEFINE_OP(SB_EW_GT, 2, return static_cast<CT>(a > b);)
SB_DEFINE_OP(SB_EW_GE, 2, return static_cast<CT>(a >= b);)
SB_DEFINE_OP(SB_EW_WHERE, 3, return a != CT(0) ? b : c;)
SB_DEFINE_OP(SB_EW_MASKED_FILL, 2, return b != CT(0) ? s.scalar : a;)
#undef SB_DEFINE_OP

__host__ __device__ inline int ew_arity(int op) {
  switch (op) {
    case SB_EW_FILL: return 0;
    case SB_EW_COPY: case SB_EW_GELU_ERF: case SB_EW_GELU_TANH: case SB_EW_SILU: case SB_EW_ADD_SCALAR:
    case SB_EW_MUL_SCALAR: case SB_EW_NEG: case SB_EW_SIGMOID: case SB_EW_TANH: case SB_EW_EXP: case SB_EW_LOG: return 1;
    case SB_EW_GLU_BWD_B: case SB_EW_BCE_LOGITS_PW: case SB_EW_BCE_LOGITS_BWD: case SB_EW_BCE_LOGITS_PW_BWD: case SB_EW_WHERE: return 3;
    default: return 2;
  }
}
__host__ __device__ inline bool ew_float_only(int op) {
  return op == SB_EW_DIV || (op >= SB_EW_GELU_ERF && op <= SB_EW_GLU_BWD_B) || (op >= SB_EW_BCE_LOGITS && op <= SB_EW_TANH_BWD);
}

// Runtime-op evaluation for paths 2 and 3 (a uniform switch per element; those paths are bound by
// their access pattern, not by this branch).
template <typename CT>
__device__ __forceinline__ CT ew_apply_runtime(int op, CT a, CT b, CT c, const OpScalars<CT>& s) {
  switch (op) {
#define SB_CASE(OPCODE) case OPCODE: return EwOp<OPCODE, CT, false>::apply(a, b, c, s);
    SB_CASE(SB_EW_COPY) SB_CASE(SB_EW_FILL) SB_CASE(SB_EW_ADD) SB_CASE(SB_EW_MUL) SB_CASE(SB_EW_SUB)
    SB_CASE(SB_EW_ADD_SCALAR) SB_CASE(SB_EW_MUL_SCALAR) SB_CASE(SB_EW_NEG) SB_CASE(SB_EW_MAXIMUM) SB_CASE(SB_EW_MINIMUM)
    SB_CASE(SB_EW_EQ) SB_CASE(SB_EW_NE) SB_CASE(SB_EW_LT) SB_CASE(SB_EW_LE) SB_CASE(SB_EW_GT) SB_CASE(SB_EW_GE)
    SB_CASE(SB_EW_WHERE) SB_CASE(SB_EW_MASKED_FILL) SB_CASE(SB_EW_DIV_TRUNC) SB_CASE(SB_EW_DIV_FLOOR)
#undef SB_CASE
    default: break;
  }
  if constexpr (std::is_floating_point<CT>::value) {
    switch (op) {
#define SB_CASE(OPCODE) case OPCODE: return EwOp<OPCODE, CT, false>::apply(a, b, c, s);
      SB_CASE(SB_EW_DIV) SB_CASE(SB_EW_GELU_ERF) SB_CASE(SB_EW_GELU_TANH) SB_CASE(SB_EW_SILU) SB_CASE(SB_EW_GLU)
      SB_CASE(SB_EW_GELU_ERF_BWD) SB_CASE(SB_EW_GELU_TANH_BWD) SB_CASE(SB_EW_SILU_BWD) SB_CASE(SB_EW_GLU_BWD_A)
      SB_CASE(SB_EW_GLU_BWD_B) SB_CASE(SB_EW_BCE_LOGITS) SB_CASE(SB_EW_BCE_LOGITS_PW) SB_CASE(SB_EW_BCE_LOGITS_BWD)
      SB_CASE(SB_EW_BCE_LOGITS_PW_BWD) SB_CASE(SB_EW_SIGMOID) SB_CASE(SB_EW_TANH) SB_CASE(SB_EW_EXP) SB_CASE(SB_EW_LOG)
      SB_CASE(SB_EW_SIGMOID_BWD) SB_CASE(SB_EW_TANH_BWD)
#undef SB_CASE
      default: break;
    }
  }
  return a;
}

// ---- path 0: contiguous --------------------------------------------------------------------------------
template <class Op, typename CT, class IO, int UNROLL>
__global__ void __launch_bounds__(kEwThreads) ew_contig_kernel(EwParams p) {
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const int64_t nvec = p.numel / kEwVec;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * (kEwThreads * UNROLL) + threadIdx.x;
  CT in[3][UNROLL][kEwVec];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kEwThreads;
    if (v < nvec) {
#pragma unroll
      for (int k = 0; k < Op::arity; ++k) IO::template load<CT, kEwVec>(p.data[k + 1], v * kEwVec, p.dtype[k + 1], in[k][u]);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t v = base + static_cast<int64_t>(u) * kEwThreads;
    if (v < nvec) {
      CT out[kEwVec];
#pragma unroll
      for (int e = 0; e < kEwVec; ++e) out[e] = Op::apply(in[0][u][e], in[1][u][e], in[2][u][e], sc);
      IO::template store<CT, kEwVec>(p.data[0], v * kEwVec, p.dtype[0], out);
    }
  }
  // scalar tail, handled by the last block
  if (blockIdx.x == gridDim.x - 1) {
    for (int64_t i = nvec * kEwVec + threadIdx.x; i < p.numel; i += kEwThreads) {
      CT a[3][1] = {};
#pragma unroll
      for (int k = 0; k < Op::arity; ++k) IO::template load<CT, 1>(p.data[k + 1], i, p.dtype[k + 1], a[k]);
      CT o[1] = {Op::apply(a[0][0], a[1][0], a[2][0], sc)};
      IO::template store<CT, 1>(p.data[0], i, p.dtype[0], o);
    }
  }
}

// ---- path 1: rows -------------------------------------------------------------------------------------------
// Block = bx threads along the row x by rows; blockIdx.x = row_block * row_chunks + chunk.  A thread
// decomposes its row index once and then walks its share of the row, UNROLL vectors in flight, so the
// index arithmetic is amortised over the whole row.  BCAST: some input is constant along the row
// (stride 0 on the fastest dimension) and is fetched as one scalar.
template <class Op, typename CT, class IO, int UNROLL, bool BCAST>
__global__ void __launch_bounds__(kEwThreads) ew_rows_kernel(EwParams p) {
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const uint32_t bx = p.bx;
  const uint32_t by = kEwThreads / bx;
  const uint32_t tx = threadIdx.x & (bx - 1);
  const uint32_t ty = threadIdx.x / bx;
  const uint32_t row_block = blockIdx.x / p.row_chunks;
  const uint32_t chunk = blockIdx.x - row_block * p.row_chunks;
  const uint32_t row = row_block * by + ty;
  if (row >= p.rows) return;
  uint32_t r = row;
  const uint32_t i1 = r % p.sizes[1];
  r /= p.sizes[1];
  const uint32_t i2 = r % p.sizes[2];
  const uint32_t i3 = r / p.sizes[2];
  int64_t off[4];
  CT bval[3];
#pragma unroll
  for (int k = 0; k <= Op::arity; ++k) off[k] = i1 * p.strides[k][1] + i2 * p.strides[k][2] + i3 * p.strides[k][3];
  if (BCAST) {
#pragma unroll
    for (int k = 0; k < Op::arity; ++k) {
      bval[k] = CT();
      if (p.strides[k + 1][0] == 0) {
        CT one[1];
        IO::template load<CT, 1>(p.data[k + 1], off[k + 1], p.dtype[k + 1], one);
        bval[k] = one[0];
      }
    }
  }
  const uint32_t n0 = p.sizes[0];
  const uint32_t nfull = n0 / kEwVec;                 // complete vectors in a row
  const uint32_t v_begin = chunk * p.span;            // this block's share of the row, in vectors
  const uint32_t v_end = min(v_begin + p.span, nfull);
  // One pass = UNROLL vectors per thread.  `load_pass` / `store_pass` are instantiated with and without
  // bounds checks: full passes issue all their loads back to back, only the last pass of a row is guarded.
  auto do_pass = [&](uint32_t v0, auto guarded) {
    constexpr bool kGuard = decltype(guarded)::value;
    CT in[3][UNROLL][kEwVec];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint32_t v = v0 + u * bx;
      if (!kGuard || v < v_end) {
#pragma unroll
        for (int k = 0; k < Op::arity; ++k) {
          if (BCAST && p.strides[k + 1][0] == 0) {
#pragma unroll
            for (int e = 0; e < kEwVec; ++e) in[k][u][e] = bval[k];
          } else {
            IO::template load<CT, kEwVec>(p.data[k + 1], off[k + 1] + static_cast<int64_t>(v) * kEwVec, p.dtype[k + 1], in[k][u]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint32_t v = v0 + u * bx;
      if (!kGuard || v < v_end) {
        CT out[kEwVec];
#pragma unroll
        for (int e = 0; e < kEwVec; ++e) out[e] = Op::apply(in[0][u][e], in[1][u][e], in[2][u][e], sc);
        IO::template store<CT, kEwVec>(p.data[0], off[0] + static_cast<int64_t>(v) * kEwVec, p.dtype[0], out);
      }
    }
  };
  uint32_t v0 = v_begin + tx;
  for (; v0 + (UNROLL - 1) * bx < v_end; v0 += bx * UNROLL) do_pass(v0, std::false_type{});
  if (v0 < v_end) do_pass(v0, std::true_type{});
  // ragged end of the row: the last chunk's first threads take one element each
  if (chunk == p.row_chunks - 1) {
    for (uint32_t e = nfull * kEwVec + tx; e < n0; e += bx) {
      CT a[3][1] = {};
#pragma unroll
      for (int k = 0; k < Op::arity; ++k)
        IO::template load<CT, 1>(p.data[k + 1], off[k + 1] + (p.strides[k + 1][0] == 0 ? 0 : e), p.dtype[k + 1], a[k]);
      CT o[1] = {Op::apply(a[0][0], a[1][0], a[2][0], sc)};
      IO::template store<CT, 1>(p.data[0], off[0] + e, p.dtype[0], o);
    }
  }
}

// ---- path 1, outer-broadcast form -----------------------------------------------------------------------------
// Binary op whose inputs are each constant along a different one of dims 1 and 2 (out[i2][i1][:] =
// x[i2][:] op y[i1][:], the shape of `a[:, None, :] + b[None, :, :]`).  A thread owns one vector position of
// the row and an R2 x R1 tile of (i2, i1): it loads R2 + R1 vectors and produces R2 * R1, so each input
// vector is fetched once per tile instead of once per output row.  KX = which input is constant along dim1.
template <class Op, typename CT, class IO, int R1, int R2, int KX>
__global__ void __launch_bounds__(kEwThreads) ew_outer_kernel(EwParams p, uint32_t tiles1, uint32_t tiles2) {
  constexpr int KY = 1 - KX;
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const uint32_t nv = p.sizes[0] / kEwVec;
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * kEwThreads + threadIdx.x;
  const uint32_t v = static_cast<uint32_t>(item % nv);
  uint64_t t = item / nv;
  const uint32_t t1 = static_cast<uint32_t>(t % tiles1);
  t /= tiles1;
  const uint32_t t2 = static_cast<uint32_t>(t % tiles2);
  const uint64_t i3 = t / tiles2;
  if (i3 >= p.sizes[3]) return;
  const uint32_t i1 = t1 * R1, i2 = t2 * R2;
  const int64_t col = static_cast<int64_t>(v) * kEwVec;
  const int64_t base_x = col + i3 * p.strides[KX + 1][3], base_y = col + i3 * p.strides[KY + 1][3];
  CT x[R2][kEwVec], y[R1][kEwVec];
#pragma unroll
  for (int r = 0; r < R2; ++r)
    if (i2 + r < p.sizes[2]) IO::template load<CT, kEwVec>(p.data[KX + 1], base_x + (i2 + r) * p.strides[KX + 1][2], p.dtype[KX + 1], x[r]);
#pragma unroll
  for (int r = 0; r < R1; ++r)
    if (i1 + r < p.sizes[1]) IO::template load<CT, kEwVec>(p.data[KY + 1], base_y + (i1 + r) * p.strides[KY + 1][1], p.dtype[KY + 1], y[r]);
  const int64_t base_o = col + i3 * p.strides[0][3];
#pragma unroll
  for (int r2 = 0; r2 < R2; ++r2) {
#pragma unroll
    for (int r1 = 0; r1 < R1; ++r1) {
      if (i2 + r2 < p.sizes[2] && i1 + r1 < p.sizes[1]) {
        CT o[kEwVec];
#pragma unroll
        for (int e = 0; e < kEwVec; ++e)
          o[e] = KX == 0 ? Op::apply(x[r2][e], y[r1][e], y[r1][e], sc) : Op::apply(y[r1][e], x[r2][e], x[r2][e], sc);
        IO::template store<CT, kEwVec>(p.data[0], base_o + (i2 + r2) * p.strides[0][2] + (i1 + r1) * p.strides[0][1], p.dtype[0], o);
      }
    }
  }
}

// The outer-broadcast form for add / sub (alpha = 1) / mul with all three operands of one 16-bit floating type, on packed
// pairs without widening.  The result is bit for bit the one of the fp32 route (widen, operate, round): the product of two
// such values is exact in fp32, and so is their sum whenever the exponents are close enough for the smaller operand to
// reach the rounding position of the result (more than 13 binades apart for fp16, 16 for bf16, the smaller one cannot
// change the rounded result either way), so the fp32 route rounds once as well.  Four packed instructions per 16-byte result
// instead of eight conversions, eight fp32 operations and four packs.
template <typename S, int OPK>
__device__ __forceinline__ uint32_t native16_pair(uint32_t a, uint32_t b) {
  if constexpr (std::is_same<S, __half>::value) {
    const __half2 x = *reinterpret_cast<const __half2*>(&a), y = *reinterpret_cast<const __half2*>(&b);
    const __half2 r = OPK == 0 ? __hadd2(x, y) : (OPK == 1 ? __hmul2(x, y) : __hsub2(x, y));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&a), y = *reinterpret_cast<const __nv_bfloat162*>(&b);
    const __nv_bfloat162 r = OPK == 0 ? __hadd2(x, y) : (OPK == 1 ? __hmul2(x, y) : __hsub2(x, y));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}
// OPK: 0 add, 1 mul, 2 sub (first operand minus second).  KX as in ew_outer_kernel.
template <typename S, int OPK, int R1, int R2, int KX>
__global__ void __launch_bounds__(kEwThreads) ew_outer_native16_kernel(EwParams p, uint32_t tiles1, uint32_t tiles2) {
  static_assert(sizeof(S) == 2 && kEwVec == 8, "one 16-byte vector of eight 16-bit values");
  constexpr int KY = 1 - KX;
  const uint32_t nv = p.sizes[0] / kEwVec;
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * kEwThreads + threadIdx.x;
  const uint32_t v = static_cast<uint32_t>(item % nv);
  uint64_t t = item / nv;
  const uint32_t t1 = static_cast<uint32_t>(t % tiles1);
  t /= tiles1;
  const uint32_t t2 = static_cast<uint32_t>(t % tiles2);
  const uint64_t i3 = t / tiles2;
  if (i3 >= p.sizes[3]) return;
  const uint32_t i1 = t1 * R1, i2 = t2 * R2;
  const int64_t col = static_cast<int64_t>(v) * kEwVec;
  const S* xs = static_cast<const S*>(p.data[KX + 1]) + col + i3 * p.strides[KX + 1][3];
  const S* ys = static_cast<const S*>(p.data[KY + 1]) + col + i3 * p.strides[KY + 1][3];
  S* os = static_cast<S*>(p.data[0]) + col + i3 * p.strides[0][3];
  uint4 x[R2], y[R1];
#pragma unroll
  for (int r = 0; r < R2; ++r)
    if (i2 + r < p.sizes[2]) x[r] = *reinterpret_cast<const uint4*>(xs + (i2 + r) * p.strides[KX + 1][2]);
#pragma unroll
  for (int r = 0; r < R1; ++r)
    if (i1 + r < p.sizes[1]) y[r] = *reinterpret_cast<const uint4*>(ys + (i1 + r) * p.strides[KY + 1][1]);
#pragma unroll
  for (int r2 = 0; r2 < R2; ++r2) {
#pragma unroll
    for (int r1 = 0; r1 < R1; ++r1) {
      if (i2 + r2 < p.sizes[2] && i1 + r1 < p.sizes[1]) {
        // operand order: input 0 op input 1
        const uint4& a = KX == 0 ? x[r2] : y[r1];
        const uint4& b = KX == 0 ? y[r1] : x[r2];
        uint4 o;
        o.x = native16_pair<S, OPK>(a.x, b.x);
        o.y = native16_pair<S, OPK>(a.y, b.y);
        o.z = native16_pair<S, OPK>(a.z, b.z);
        o.w = native16_pair<S, OPK>(a.w, b.w);
        st_stream_u4(os + (i2 + r2) * p.strides[0][2] + (i1 + r1) * p.strides[0][1], o);
      }
    }
  }
}

// ---- path 2: tiled transpose ------------------------------------------------------------------------------
// 32 x 32 tile over (dim0, dim1); dims 2.. are walked by blockIdx.z (flattened).  Operands whose unit
// stride lies along dim1 are read with threads along dim1 and turned through shared memory.
template <typename CT>
__global__ void __launch_bounds__(256) ew_transpose_kernel(EwGenericParams p, uint32_t transposed_mask) {
  __shared__ CT tile[3][32][33];
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
  const uint32_t n0 = p.sizes[0], n1 = p.sizes[1];
  const uint32_t t0 = blockIdx.x * 32, t1 = blockIdx.y * 32;
  // outer offset from blockIdx.z
  int64_t outer[SB_MAX_OPERANDS] = {0, 0, 0, 0};
  {
    uint32_t r = blockIdx.z;
    for (int d = 2; d < p.ndim; ++d) {
      const uint32_t i = r % p.sizes[d];
      r /= p.sizes[d];
      for (int k = 0; k < p.noperands; ++k) outer[k] += i * p.strides[k][d];
    }
  }
  const int nin = p.noperands - 1;
  // stage transposed operands: threads along dim1
  for (int k = 0; k < nin; ++k) {
    if (!(transposed_mask >> k & 1)) continue;
    for (int j = ty; j < 32; j += 8) {
      const uint32_t i0 = t0 + j, i1 = t1 + tx;
      if (i0 < n0 && i1 < n1) {
        CT v[1];
        DynamicIO::load<CT, 1>(p.data[k + 1], outer[k + 1] + i0 * p.strides[k + 1][0] + i1 * p.strides[k + 1][1],
                               p.dtype[k + 1], v);
        tile[k][j][tx] = v[0];
      }
    }
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const uint32_t i0 = t0 + tx, i1 = t1 + j;
    if (i0 < n0 && i1 < n1) {
      CT a[3] = {};
      for (int k = 0; k < nin; ++k) {
        if (transposed_mask >> k & 1) {
          a[k] = tile[k][tx][j];
        } else {
          CT v[1];
          DynamicIO::load<CT, 1>(p.data[k + 1], outer[k + 1] + i0 * p.strides[k + 1][0] + i1 * p.strides[k + 1][1],
                                 p.dtype[k + 1], v);
          a[k] = v[0];
        }
      }
      CT o[1] = {ew_apply_runtime<CT>(p.op, a[0], a[1], a[2], sc)};
      DynamicIO::store<CT, 1>(p.data[0], outer[0] + i0 * p.strides[0][0] + i1 * p.strides[0][1], p.dtype[0], o);
    }
  }
}

// Vector form of the tile kernel: 64 x 64 tile, 4 elements per access on both sides.  Needs sizes[0] and
// sizes[1] to be multiples of 4 and every operand 4-element aligned along its unit-stride dimension.
// All global loads of a tile (the transposed operands and the straight ones) are issued before anything
// waits on them; interior tiles (kGuard = false) carry no bounds checks.
template <typename CT, class IO, bool kGuard>
__device__ __forceinline__ void ew_transpose_tile(const EwGenericParams& p, uint32_t transposed_mask, CT (*tile)[64][65],
                                                  const int64_t* outer, uint32_t t0, uint32_t t1) {
  constexpr int T = 64, V = 4, PASSES = T / 16, KMAX = 2;  // at most two inputs (the classifier guarantees it)
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const uint32_t n0 = p.sizes[0], n1 = p.sizes[1];
  const int nin = p.noperands - 1;
  const uint32_t lane_v = threadIdx.x % (T / V);   // vector position along the unit-stride direction
  const uint32_t lane_r = threadIdx.x / (T / V);   // 0..15: row inside a pass
  // Operand k as loaded: vectors along dim1 for a transposed operand, along dim0 (like the output) otherwise.
  // Every index below is a compile-time constant after unrolling, so the arrays stay in registers.
  CT held[KMAX][PASSES][V];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    if (k >= nin) continue;
    const bool tr = transposed_mask >> k & 1;
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
      const uint32_t ia = lane_r + 16 * pass, ib = lane_v * V;
      const uint32_t i0 = t0 + (tr ? ia : ib), i1 = t1 + (tr ? ib : ia);
      if (!kGuard || (i0 < n0 && i1 < n1)) {
        if (!tr && p.strides[k + 1][0] == 0) {
          CT one[1];
          IO::template load<CT, 1>(p.data[k + 1], outer[k + 1] + static_cast<int64_t>(i1) * p.strides[k + 1][1], p.dtype[k + 1], one);
#pragma unroll
          for (int j = 0; j < V; ++j) held[k][pass][j] = one[0];
        } else {
          const int64_t off = tr ? static_cast<int64_t>(i0) * p.strides[k + 1][0] + i1 : i0 + static_cast<int64_t>(i1) * p.strides[k + 1][1];
          IO::template load<CT, V>(p.data[k + 1], outer[k + 1] + off, p.dtype[k + 1], held[k][pass]);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    if (k >= nin || !(transposed_mask >> k & 1)) continue;
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
#pragma unroll
      for (int j = 0; j < V; ++j) tile[k][lane_v * V + j][lane_r + 16 * pass] = held[k][pass][j];
    }
  }
  __syncthreads();
#pragma unroll
  for (int pass = 0; pass < PASSES; ++pass) {
    const uint32_t l1 = lane_r + 16 * pass;
    const uint32_t i1 = t1 + l1, i0 = t0 + lane_v * V;
    if (!kGuard || (i0 < n0 && i1 < n1)) {
      CT a[KMAX][V];
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
#pragma unroll
        for (int j = 0; j < V; ++j) a[k][j] = (k < nin && (transposed_mask >> k & 1)) ? tile[k][l1][lane_v * V + j] : held[k][pass][j];
      }
      CT o[V];
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = ew_apply_runtime<CT>(p.op, a[0][j], a[1][j], a[1][j], sc);
      IO::template store<CT, V>(p.data[0], outer[0] + i0 + static_cast<int64_t>(i1) * p.strides[0][1], p.dtype[0], o);
    }
  }
}

template <typename CT, class IO>
__global__ void __launch_bounds__(256, 5) ew_transpose_vec_kernel(EwGenericParams p, uint32_t transposed_mask) {
  constexpr int T = 64;
  // one [T][T + 1] slot per input (only the transposed ones are used); sized by the launch
  extern __shared__ __align__(16) unsigned char tile_raw[];
  CT (*tile)[T][T + 1] = reinterpret_cast<CT (*)[T][T + 1]>(tile_raw);
  const uint32_t t0 = blockIdx.x * T, t1 = blockIdx.y * T;
  int64_t outer[SB_MAX_OPERANDS] = {0, 0, 0, 0};
  {
    uint32_t r = blockIdx.z;
    for (int d = 2; d < p.ndim; ++d) {
      const uint32_t i = r % p.sizes[d];
      r /= p.sizes[d];
#pragma unroll
      for (int k = 0; k < 3; ++k) outer[k] += i * p.strides[k][d];  // strides of absent operands are zero
    }
  }
  if (t0 + T <= p.sizes[0] && t1 + T <= p.sizes[1]) ew_transpose_tile<CT, IO, false>(p, transposed_mask, tile, outer, t0, t1);
  else ew_transpose_tile<CT, IO, true>(p, transposed_mask, tile, outer, t0, t1);
}

// ---- path 3: generic ------------------------------------------------------------------------------------------
template <typename CT>
__global__ void __launch_bounds__(256) ew_generic_kernel(EwGenericParams p) {
  const OpScalars<CT> sc = make_scalars<CT>(p);
  const int nin = p.noperands - 1;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; idx < p.numel;
       idx += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t off[SB_MAX_OPERANDS] = {0, 0, 0, 0};
    uint64_t r = static_cast<uint64_t>(idx);
    for (int d = 0; d < p.ndim; ++d) {
      uint64_t i;
      if (r >> 32) {
        i = r % p.sizes[d];
        r /= p.sizes[d];
      } else {
        const uint32_t r32 = static_cast<uint32_t>(r);
        i = r32 % p.sizes[d];
        r = r32 / p.sizes[d];
      }
      for (int k = 0; k < p.noperands; ++k) off[k] += static_cast<int64_t>(i) * p.strides[k][d];
    }
    CT a[3] = {};
    for (int k = 0; k < nin; ++k) {
      CT v[1];
      DynamicIO::load<CT, 1>(p.data[k + 1], off[k + 1], p.dtype[k + 1], v);
      a[k] = v[0];
    }
    CT o[1] = {ew_apply_runtime<CT>(p.op, a[0], a[1], a[2], sc)};
    DynamicIO::store<CT, 1>(p.data[0], off[0], p.dtype[0], o);
  }
}

// ---- host-side plan --------------------------------------------------------------------------------------------
enum EwCompute { kCtBool = 0, kCtI32 = 1, kCtI64 = 2, kCtF32 = 3, kCtF64 = 4 };

struct EwPlan {
  int path;             // 0..3
  int compute;          // EwCompute
  bool fast;            // single-MUFU approximations allowed (bf16 result)
  int static_dtype;     // dtype code when every operand shares a dtype with a typed kernel, else -1
  uint32_t transposed_mask;
  bool transpose_vec;   // path 2: every operand allows 4-element accesses
  int outer;            // path 1: 1 or 2 = input 0 / input 1 is constant along dim1 and the other along dim2, else 0
};

int ew_make_plan(const sb_ew_desc* d, EwPlan* plan);

// Launchers per compute type (one translation unit each, to keep compile times parallel).
int ew_launch_f32(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st);
int ew_launch_f64(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st);
int ew_launch_int(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st);

// Fills the kernel parameter blocks from a descriptor.
void ew_fill_params(const sb_ew_desc* d, EwParams* p);
void ew_fill_generic(const sb_ew_desc* d, EwGenericParams* p);
// Launch geometry helpers (defined in elementwise.cu).
int ew_rows_geometry(const sb_ew_desc* d, EwParams* p, unsigned* grid);

// ---- templated launch glue used by the per-compute-type translation units --------------------------
template <int OP, typename CT, bool FAST, class IO>
int ew_launch_vector(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st) {
  using Op = EwOp<OP, CT, FAST>;
  EwParams p;
  ew_fill_params(d, &p);
  if (plan.path == 0) {
    constexpr int kUnroll = 2;
    const int64_t nvec = p.numel / kEwVec;
    const int64_t per_block = static_cast<int64_t>(kEwThreads) * kUnroll;
    int64_t blocks = (nvec + per_block - 1) / per_block;
    if (blocks == 0) blocks = 1;
    if (blocks > 0x7fffffffLL) return SB_ERR_TOO_LARGE;
    ew_contig_kernel<Op, CT, IO, kUnroll><<<static_cast<unsigned>(blocks), kEwThreads, 0, st>>>(p);
    return launch_status();
  }
  if constexpr (Op::arity == 2) {
    if (plan.outer) {
      constexpr int R1 = 4, R2 = 4;
      const uint32_t tiles1 = (p.sizes[1] + R1 - 1) / R1, tiles2 = (p.sizes[2] + R2 - 1) / R2;
      const uint64_t items = static_cast<uint64_t>(p.sizes[0] / kEwVec) * tiles1 * tiles2 * p.sizes[3];
      const uint64_t blocks = (items + kEwThreads - 1) / kEwThreads;
      if (blocks > 0x7fffffffULL) return SB_ERR_TOO_LARGE;
      if constexpr (!IO::kDynamic && std::is_same<CT, float>::value && (OP == SB_EW_ADD || OP == SB_EW_SUB || OP == SB_EW_MUL)) {
        using S = typename IO::storage;
        if constexpr (std::is_same<S, __half>::value || std::is_same<S, __nv_bfloat16>::value) {
          if (OP == SB_EW_MUL || p.alpha == 1.0) {  // the packed route has no alpha
            constexpr int kOpk = OP == SB_EW_ADD ? 0 : (OP == SB_EW_MUL ? 1 : 2);
            if (plan.outer == 1) ew_outer_native16_kernel<S, kOpk, R1, R2, 0><<<static_cast<unsigned>(blocks), kEwThreads, 0, st>>>(p, tiles1, tiles2);
            else ew_outer_native16_kernel<S, kOpk, R1, R2, 1><<<static_cast<unsigned>(blocks), kEwThreads, 0, st>>>(p, tiles1, tiles2);
            return launch_status();
          }
        }
      }
      if (plan.outer == 1) ew_outer_kernel<Op, CT, IO, R1, R2, 0><<<static_cast<unsigned>(blocks), kEwThreads, 0, st>>>(p, tiles1, tiles2);
      else ew_outer_kernel<Op, CT, IO, R1, R2, 1><<<static_cast<unsigned>(blocks), kEwThreads, 0, st>>>(p, tiles1, tiles2);
      return launch_status();
    }
  }
  unsigned grid = 0;
  int rc = ew_rows_geometry(d, &p, &grid);
  if (rc != SB_OK) return rc;
  if (p.bcast) {
    if (p.unroll == 4) ew_rows_kernel<Op, CT, IO, 4, true><<<grid, kEwThreads, 0, st>>>(p);
    else ew_rows_kernel<Op, CT, IO, 2, true><<<grid, kEwThreads, 0, st>>>(p);
  } else {
    if (p.unroll == 4) ew_rows_kernel<Op, CT, IO, 4, false><<<grid, kEwThreads, 0, st>>>(p);
    else ew_rows_kernel<Op, CT, IO, 2, false><<<grid, kEwThreads, 0, st>>>(p);
  }
  return launch_status();
}

template <typename CT>
int ew_launch_scalar_paths(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st) {
  EwGenericParams g;
  ew_fill_generic(d, &g);
  if (plan.path == 2) {
    uint64_t outer = 1;
    for (int i = 2; i < d->ndim; ++i) outer *= static_cast<uint64_t>(d->sizes[i]);
    if (outer > 65535) return SB_ERR_TOO_LARGE;  // the classifier never selects path 2 in that case
    if constexpr (sizeof(CT) <= 4) {
      if (plan.transpose_vec) {
        dim3 grid((g.sizes[0] + 63) / 64, (g.sizes[1] + 63) / 64, static_cast<unsigned>(outer));
        // shared memory: slots up to the last transposed input (at most two inputs reach this kernel)
        const size_t smem = ((plan.transposed_mask & 2u) ? 2 : 1) * sizeof(CT) * 64 * 65;
        if constexpr (std::is_same<CT, float>::value) {
          switch (plan.static_dtype) {
            case SB_F32: ew_transpose_vec_kernel<CT, StaticIO<float>><<<grid, 256, smem, st>>>(g, plan.transposed_mask); break;
            case SB_BF16: ew_transpose_vec_kernel<CT, StaticIO<__nv_bfloat16>><<<grid, 256, smem, st>>>(g, plan.transposed_mask); break;
            case SB_F16: ew_transpose_vec_kernel<CT, StaticIO<__half>><<<grid, 256, smem, st>>>(g, plan.transposed_mask); break;
            default: ew_transpose_vec_kernel<CT, DynamicIO><<<grid, 256, smem, st>>>(g, plan.transposed_mask); break;
          }
        } else {
          ew_transpose_vec_kernel<CT, DynamicIO><<<grid, 256, smem, st>>>(g, plan.transposed_mask);
        }
        return launch_status();
      }
    }
    {
      dim3 grid((g.sizes[0] + 31) / 32, (g.sizes[1] + 31) / 32, static_cast<unsigned>(outer));
      ew_transpose_kernel<CT><<<grid, 256, 0, st>>>(g, plan.transposed_mask);
    }
    return launch_status();
  }
  int64_t blocks = (g.numel + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  ew_generic_kernel<CT><<<static_cast<unsigned>(blocks), 256, 0, st>>>(g);
  return launch_status();
}

}  // namespace sb

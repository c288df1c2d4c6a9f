// Parameter block and row arithmetic shared by the cross-entropy kernel variants.
#pragma once

#include "common.cuh"

namespace sb {

struct CEParams {
  const void* logits;
  void* grad;                // nullable
  const int64_t* target;
  float* row_loss;
  float* row_lse;            // nullable
  const float* row_grad_out; // nullable
  const double* acc;         // {loss_sum, valid_count}
  int64_t rows;
  int64_t classes;
  int64_t ignore_index;
  float label_smoothing;
  float grad_scale;
  int reduction;
  int dtype;
  int32_t* status;           // nullable
  const float* class_weight; // nullable: fp32 [classes]; multiplies the loss and the gradient of a row by w[target]
  uint32_t flags;            // SB_CE_FLAG_* of sb_ce_args
};

// loss of one non-ignored row; sum_x is the plain sum of the row's logits.
__device__ __forceinline__ float ce_row_loss(float lse, float x_target, float sum_x, float eps, float eps_over_c) {
  if (eps == 0.f) return lse - x_target;  // logf(row_sum) + row_max - row_input[target]
  return lse - (1.f - eps) * x_target - eps_over_c * sum_x;
}

// Factor applied to (softmax - smoothed one-hot) of a row.
__device__ __forceinline__ float ce_row_scale(const CEParams& p, int64_t row, int64_t target) {
  float scale = p.grad_scale;
  if (p.reduction == SB_REDUCTION_MEAN) scale = static_cast<float>(static_cast<double>(scale) / p.acc[1]);
  if (p.row_grad_out) scale *= p.row_grad_out[row];
  if (p.class_weight) scale *= p.class_weight[target];
  return scale;
}

__device__ __forceinline__ void ce_store_loss(double loss_sum, double count, int reduction, void* out, int dtype) {
  double v = loss_sum;
  if (reduction == SB_REDUCTION_MEAN) v = count > 0.0 ? loss_sum / count : CUDART_NAN;
  switch (dtype) {
    case SB_F32: *static_cast<float*>(out) = static_cast<float>(v); break;
    case SB_BF16: *static_cast<__nv_bfloat16*>(out) = __float2bfloat16_rn(static_cast<float>(v)); break;
    case SB_F16: *static_cast<__half*>(out) = __float2half_rn(static_cast<float>(v)); break;
    case SB_F64: *static_cast<double*>(out) = v; break;
    default: break;
  }
}

// ---- L2 residency hints for rows that are read twice --------------------------------------------------------------------
// A two-sweep kernel reads a row, reduces it and reads it again.  The first read asks L2 to keep the lines (evict_last); the
// second one, and everything read once, releases them (evict_first).
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ld_hint_u4(const void* p, uint64_t policy) {
  uint4 r;
  asm volatile("ld.global.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(policy));
  return r;
}
// 16-byte vector load with a policy; other widths load plainly.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec_hint(const T* p, uint64_t policy) {
  if constexpr (sizeof(T) * N == 16) {
    const uint4 raw = ld_hint_u4(p, policy);
    return *reinterpret_cast<const Vec<T, N>*>(&raw);
  } else {
    return load_vec<T, N>(p);
  }
}

// Kernel families (defined in cross_entropy.cu, cross_entropy_rows.cu and cross_entropy_tma.cu).
int ce_launch_generic(const CEParams& p, cudaStream_t st);
int ce_launch_resident(const CEParams& p, cudaStream_t st, int variant, bool pdl);
// Rows of less than 16 KB held in registers (one warp or one 128-thread group per row): one read and one write
// per logit.  rows_reg_applies says whether the shape and the pointers qualify.
bool rows_reg_applies(int dtype, int64_t classes, const void* logits, const void* grad);
// Rows of 256 B to 32 KB with a 16-byte aligned pitch, a warp (part of one, or four) per row on a ring of shared-memory slots fed by
// bulk copies.
bool ring_rows_applies(int dtype, int64_t classes, const void* logits, const void* grad);
int ce_launch_ring_rows(const CEParams& p, cudaStream_t st, bool pdl);
int lsm_launch_ring(const void* in, void* out, int dtype, int64_t rows, int64_t dim, int mode, cudaStream_t st);
int red_set_warp_row_bytes(int n);  // tuning: longest row one warp reduces (0 = vector row kernels off, 4096..262144)
int ring_set_max_bytes(int n);  // tuning: longest row the slot-ring kernel takes (16384..65536)
int ring_set_warps(int n);  // tuning: consumer warps per CTA of the slot-ring kernel (0 = automatic)
int ce_launch_rows_reg(const CEParams& p, cudaStream_t st);
// Chooses the resident family for a shape: 0 none, 1/2/4 = resident in shared memory of a 1/2/4-CTA cluster.
int ce_choose_variant(int dtype, int64_t rows, int64_t classes, const void* logits, const void* grad);
// What ce_dispatch will run: 0 generic two-sweep rows, 1/2/4 resident, 8 rows in registers.
int ce_choose_family(const CEParams& p);
int ce_dispatch(const CEParams& p, cudaStream_t st);
int xchg_set_timeout_ms(int ms);  // limit of the waits of the exchange kernels
// log_softmax (mode 1) or softmax (mode 2) over rows of `dim` elements through the resident pipeline; SB_ERR_UNSUPPORTED
// if the shape does not qualify.
int lsm_launch_resident(const void* in, void* out, int dtype, int64_t rows, int64_t dim, int mode, cudaStream_t st);

}  // namespace sb

// Cross entropy with class-probability targets, forward and backward in one kernel (the counterpart of
// cross_entropy_prob_kernel, torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:532-576, which
// computes the forward only).
//
// With q_c = t_c (1 - eps) + eps / C and per-class weights w (1 when absent):
//   loss_i  = sum_c w_c q_ic (lse_i - x_ic) = A_i lse_i - B_i,   A_i = sum_c w_c q_ic,  B_i = sum_c w_c q_ic x_ic
//   grad_ic = (exp(x_ic - lse_i) A_i - w_c q_ic) * scale_i
// One CTA per row, grid-stride over rows: the first sweep streams the logits and the target row together (online
// max / sum of exponentials, A, B), the second forms the gradient; the second read of both rows is served by L2 (the first
// read asks it to keep the lines, the second releases them).  16-byte accesses when the row pitch allows it.
#include "ce_common.cuh"

namespace sb {

namespace {

struct ProbParams {
  const void* logits;
  const void* target;
  void* grad;
  float* row_loss;
  const float* row_grad_out;
  const float* class_weight;
  int64_t rows, classes;
  float eps, grad_scale, loss_scale;
};

template <typename T, int VEC, int THREADS>
__global__ void __launch_bounds__(THREADS) ce_prob_rows_kernel(ProbParams p) {
  constexpr bool kAccurate = sizeof(T) == 4;
  __shared__ float s_m[THREADS / 32], s_s[THREADS / 32], s_a[THREADS / 32], s_b[THREADS / 32];
  __shared__ float s_out[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t C = p.classes;
  const int64_t nvec = C / VEC;  // VEC > 1 only when C % VEC == 0
  const float keep = 1.f - p.eps;
  const float eps_c = p.eps / static_cast<float>(C);

  const uint64_t l2_keep = l2_policy_keep(), l2_stream = l2_policy_stream();
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* x = static_cast<const T*>(p.logits) + row * C;
    const T* tq = static_cast<const T*>(p.target) + row * C;
    float m = -CUDART_INF_F, s = 0.f, a = 0.f, b = 0.f;
    for (int64_t i = tid; i < nvec; i += THREADS) {
      // the gradient sweep reads both rows again: ask L2 to keep them (without a gradient they are read once)
      const Vec<T, VEC> v = load_vec_hint<T, VEC>(x + i * VEC, p.grad ? l2_keep : l2_stream);
      const Vec<T, VEC> tv = load_vec_hint<T, VEC>(tq + i * VEC, p.grad ? l2_keep : l2_stream);
      float f[VEC];
      float vmax = -CUDART_INF_F;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        f[k] = to_float(v.v[k]);
        vmax = fmaxf(vmax, f[k]);
      }
      if (vmax > m) {
        s *= kAccurate ? exp_accurate(m - vmax) : exp_fast(m - vmax);
        m = vmax;
      }
      const float mm = (m == -CUDART_INF_F) ? 0.f : m;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        s += kAccurate ? exp_accurate(f[k] - mm) : exp_fast(f[k] - mm);
        float q = fmaf(to_float(tv.v[k]), keep, eps_c);
        if (p.class_weight) q *= p.class_weight[i * VEC + k];
        a += q;
        b = fmaf(q, f[k], b);
      }
    }
    MaxSum ms = warp_merge(MaxSum{m, s});
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) {
      s_m[warp] = ms.m;
      s_s[warp] = ms.s;
      s_a[warp] = a;
      s_b[warp] = b;
    }
    __syncthreads();
    if (warp == 0) {
      MaxSum r{lane < THREADS / 32 ? s_m[lane] : -CUDART_INF_F, lane < THREADS / 32 ? s_s[lane] : 0.f};
      float ra = lane < THREADS / 32 ? s_a[lane] : 0.f;
      float rb = lane < THREADS / 32 ? s_b[lane] : 0.f;
      r = warp_merge(r);
      ra = warp_sum(ra);
      rb = warp_sum(rb);
      if (lane == 0) {
        const float lse = r.m + logf(r.s);
        s_out[0] = lse;
        s_out[1] = ra;
        p.row_loss[row] = (ra * lse - rb) * p.loss_scale;
      }
    }
    __syncthreads();
    if (p.grad) {
      const float lse = s_out[0];
      float scale = p.grad_scale;
      if (p.row_grad_out) scale *= p.row_grad_out[row];
      const float pa = s_out[1] * scale;  // what the softmax is multiplied by
      T* g = static_cast<T*>(p.grad) + row * C;
      for (int64_t i = tid; i < nvec; i += THREADS) {
        const Vec<T, VEC> v = load_vec_hint<T, VEC>(x + i * VEC, l2_stream);
        const Vec<T, VEC> tv = load_vec_hint<T, VEC>(tq + i * VEC, l2_stream);
        Vec<T, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const float d = to_float(v.v[k]) - lse;
          const float pr = kAccurate ? exp_accurate(d) : exp_fast(d);
          float q = fmaf(to_float(tv.v[k]), keep, eps_c);
          if (p.class_weight) q *= p.class_weight[i * VEC + k];
          o.v[k] = from_float<T>(fmaf(pr, pa, -q * scale));
        }
        store_vec<T, VEC>(g + i * VEC, o);
      }
    }
    __syncthreads();  // s_out is rewritten by the next row
  }
}

template <typename T>
int launch_prob(const ProbParams& p, cudaStream_t st) {
  constexpr int kVec = 16 / sizeof(T);
  constexpr int kThreads = 512;
  const int64_t max_grid = static_cast<int64_t>(sm_count()) * 4;
  const int grid = static_cast<int>(p.rows < max_grid ? p.rows : max_grid);
  const auto al = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  const bool aligned = (p.classes % kVec == 0) && al(p.logits) && al(p.target) && (p.grad == nullptr || al(p.grad));
  if (aligned) ce_prob_rows_kernel<T, kVec, kThreads><<<grid, kThreads, 0, st>>>(p);
  else ce_prob_rows_kernel<T, 1, kThreads><<<grid, kThreads, 0, st>>>(p);
  return launch_status();
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" int sb_ce_prob_forward_backward(const sb_ce_prob_args* a, sb_stream_t stream) {
  if (!a || a->rows < 0 || a->classes < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->rows == 0) return SB_OK;
  if (a->classes == 0 || !a->logits || !a->target || !a->row_loss) return SB_ERR_INVALID_ARGUMENT;
  if (a->dtype != SB_F32 && a->dtype != SB_BF16 && a->dtype != SB_F16) return SB_ERR_UNSUPPORTED;
  if (!(a->label_smoothing >= 0.f && a->label_smoothing <= 1.f)) return SB_ERR_INVALID_ARGUMENT;
  if (a->grad_logits && (a->grad_logits == a->logits || a->grad_logits == a->target)) return SB_ERR_INVALID_ARGUMENT;
  const size_t es = dtype_size(a->dtype);
  if (reinterpret_cast<uintptr_t>(a->logits) % es || reinterpret_cast<uintptr_t>(a->target) % es ||
      reinterpret_cast<uintptr_t>(a->grad_logits) % es)
    return SB_ERR_MISALIGNED;
  ProbParams p;
  p.logits = a->logits;
  p.target = a->target;
  p.grad = a->grad_logits;
  p.row_loss = a->row_loss;
  p.row_grad_out = a->row_grad_out;
  p.class_weight = a->class_weight;
  p.rows = a->rows;
  p.classes = a->classes;
  p.eps = a->label_smoothing;
  p.grad_scale = a->grad_scale;
  p.loss_scale = a->loss_scale;
  switch (a->dtype) {
    case SB_F32: return launch_prob<float>(p, as_stream(stream));
    case SB_BF16: return launch_prob<__nv_bfloat16>(p, as_stream(stream));
    default: return launch_prob<__half>(p, as_stream(stream));
  }
}

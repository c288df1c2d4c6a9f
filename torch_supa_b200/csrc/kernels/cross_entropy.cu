// Fused cross entropy forward + backward for class-index targets: generic row kernels and the
// small bookkeeping kernels (valid-row count, deterministic loss sum, finish, gradient rescale).
//
// Row math (the same as cross_entropy_index_mean_kernel of the reference,
// torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:121-162, extended with label
// smoothing and the gradient): with lse = max + log(sum exp(x - max)),
//   loss_i = lse - (1 - eps) * x[t_i] - (eps / C) * sum_c x_c            (0 when t_i == ignore_index)
//   grad_ic = (exp(x_c - lse) - (1 - eps) * [c == t_i] - eps / C) * scale  (0 when t_i == ignore_index)
// where scale = upstream / |V| for `mean` (|V| = rows that are not ignored), upstream otherwise.
//
// Kernels in this file read each row twice (statistics sweep, gradient sweep); the second read is
// served by L1/L2 because a CTA (or warp) re-reads the row it has just streamed.  The variant that keeps
// the row in shared memory lives in cross_entropy_tma.cu; ce_dispatch() chooses between them.
#include "ce_common.cuh"

namespace sb {

// ---------------------------------------------------------------------------------------------
// One CTA per row, grid-stride over rows.  VEC elements per 16-byte access when the row pitch and
// the base pointers allow it, else VEC = 1.
// ---------------------------------------------------------------------------------------------
//
// WS (class weights together with label smoothing; the arithmetic of the upstream composite the reference falls
// back to, CrossEntropyLoss.cpp:50): the smoothing term weights every class c of a row by w[c],
//   loss_i  = (1 - eps) w[t_i] (lse - x[t_i]) + (eps / C) (W lse - sum_c w[c] x_c),  W = sum_c w[c]
//   grad_ic = (p_c ((1 - eps) w[t_i] + eps W / C) - (1 - eps) w[t_i] [c == t_i] - (eps / C) w[c]) * scale
// with scale = upstream / sum_i w[t_i] for `mean`.  The weights are read along the row in both sweeps.
template <typename T, int VEC, int THREADS, bool WS = false>
__global__ void __launch_bounds__(THREADS) ce_rows_cta_kernel(CEParams p) {
  constexpr bool kAccurate = sizeof(T) == 4;
  __shared__ float s_m[THREADS / 32];
  __shared__ float s_s[THREADS / 32];
  __shared__ float s_x[THREADS / 32];
  __shared__ float s_w[THREADS / 32];
  __shared__ float s_out[4];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int64_t C = p.classes;
  const int64_t nvec = C / VEC;  // VEC > 1 only when C % VEC == 0
  const float eps = p.label_smoothing;
  const float eps_c = eps / static_cast<float>(C);

  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* x = static_cast<const T*>(p.logits) + row * C;
    T* g = p.grad ? static_cast<T*>(p.grad) + row * C : nullptr;
    const int64_t t = p.target[row];
    bool ignored = (t == p.ignore_index);
    if (!ignored && (t < 0 || t >= C)) {
      if (tid == 0 && p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
      ignored = true;
    }
    if (ignored) {  // uniform over the CTA
      if (tid == 0) {
        p.row_loss[row] = 0.f;
        if (p.row_lse) p.row_lse[row] = 0.f;
      }
      if (g) {
        Vec<T, VEC> z;
#pragma unroll
        for (int k = 0; k < VEC; ++k) z.v[k] = from_float<T>(0.f);
        for (int64_t i = tid; i < nvec; i += THREADS) store_vec<T, VEC>(g + i * VEC, z);
      }
      continue;
    }

    // ---- sweep 1: online (max, sum exp) and sum x ------------------------------------------
    float m = -CUDART_INF_F, s = 0.f, sx = 0.f, sw = 0.f;  // WS: sx = sum w x, sw = sum w
    for (int64_t i = tid; i < nvec; i += THREADS) {
      Vec<T, VEC> v = load_vec<T, VEC>(x + i * VEC);
      float f[VEC];
      float vmax = -CUDART_INF_F;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        f[k] = to_float(v.v[k]);
        vmax = fmaxf(vmax, f[k]);
      }
      if (vmax > m) {
        s *= kAccurate ? exp_accurate(m - vmax) : exp_fast(m - vmax);  // m = -inf: s is 0, exp(-inf) = 0
        m = vmax;
      }
      const float mm = (m == -CUDART_INF_F) ? 0.f : m;  // keep exp(-inf - -inf) out of the sum
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        s += kAccurate ? exp_accurate(f[k] - mm) : exp_fast(f[k] - mm);
        if (WS) {
          const float wc = p.class_weight[i * VEC + k];
          sx = fmaf(wc, f[k], sx);
          sw += wc;
        } else {
          sx += f[k];
        }
      }
    }
    MaxSum ms = warp_merge(MaxSum{m, s});
    sx = warp_sum(sx);
    if (WS) sw = warp_sum(sw);
    if (lane == 0) {
      s_m[warp] = ms.m;
      s_s[warp] = ms.s;
      s_x[warp] = sx;
      if (WS) s_w[warp] = sw;
    }
    __syncthreads();
    if (warp == 0) {
      MaxSum a{lane < THREADS / 32 ? s_m[lane] : -CUDART_INF_F, lane < THREADS / 32 ? s_s[lane] : 0.f};
      float b = lane < THREADS / 32 ? s_x[lane] : 0.f;
      float wsum = (WS && lane < THREADS / 32) ? s_w[lane] : 0.f;
      a = warp_merge(a);
      b = warp_sum(b);
      if (WS) wsum = warp_sum(wsum);
      if (lane == 0) {
        const float lse = a.m + logf(a.s);
        const float xt = to_float(x[t]);
        s_out[0] = lse;
        if (WS) {
          const float wt = p.class_weight[t];
          s_out[1] = (1.f - eps) * wt * (lse - xt) + eps_c * (wsum * lse - b);
          s_out[2] = (1.f - eps) * wt + eps_c * wsum;  // what the softmax is multiplied by
          s_out[3] = (1.f - eps) * wt;                 // what the class of the target gets subtracted
        } else {
          s_out[1] = ce_row_loss(lse, xt, b, eps, eps_c) * (p.class_weight ? p.class_weight[t] : 1.f);
        }
      }
    }
    __syncthreads();
    const float lse = s_out[0];
    if (tid == 0) {
      p.row_loss[row] = s_out[1];
      if (p.row_lse) p.row_lse[row] = lse;
    }

    // ---- sweep 2: gradient ---------------------------------------------------------------------
    if (g) {
      float scale, sub_all, sub_t, base = 0.f;
      if (WS) {
        base = p.grad_scale;  // the row's scale without w[target]: the weights enter term by term
        if (p.reduction == SB_REDUCTION_MEAN) base = static_cast<float>(static_cast<double>(base) / p.acc[1]);
        if (p.row_grad_out) base *= p.row_grad_out[row];
        scale = s_out[2] * base;
        sub_all = 0.f;
        sub_t = s_out[3] * base;
      } else {
        scale = ce_row_scale(p, row, t);
        sub_all = eps_c * scale;
        sub_t = (1.f - eps) * scale;
      }
      const float wsub = eps_c * base;
      for (int64_t i = tid; i < nvec; i += THREADS) {
        Vec<T, VEC> v = load_vec<T, VEC>(x + i * VEC);
        Vec<T, VEC> o;
        const int64_t c0 = i * VEC;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const float d = to_float(v.v[k]) - lse;
          const float pr = kAccurate ? exp_accurate(d) : exp_fast(d);
          float gv = WS ? fmaf(pr, scale, -wsub * p.class_weight[c0 + k]) : fmaf(pr, scale, -sub_all);
          if (c0 + k == t) gv -= sub_t;
          o.v[k] = from_float<T>(gv);
        }
        store_vec<T, VEC>(g + c0, o);
      }
    }
    __syncthreads();  // s_out is rewritten by the next row
  }
}

// ---------------------------------------------------------------------------------------------
// One warp per row for short rows (classes <= 1024): the reference keeps a family of special
// kernels for C <= 64 (CrossEntropyLossKernel.cu:228-530); one warp-per-row kernel covers them.
// ---------------------------------------------------------------------------------------------
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) ce_rows_warp_kernel(CEParams p) {
  constexpr bool kAccurate = sizeof(T) == 4;
  const int lane = threadIdx.x & 31;
  const int64_t warps_per_grid = static_cast<int64_t>(gridDim.x) * (THREADS / 32);
  const int64_t C = p.classes;
  const float eps = p.label_smoothing;
  const float eps_c = eps / static_cast<float>(C);

  for (int64_t row = static_cast<int64_t>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5); row < p.rows;
       row += warps_per_grid) {
    const T* x = static_cast<const T*>(p.logits) + row * C;
    T* g = p.grad ? static_cast<T*>(p.grad) + row * C : nullptr;
    const int64_t t = p.target[row];
    bool ignored = (t == p.ignore_index);
    if (!ignored && (t < 0 || t >= C)) {
      if (lane == 0 && p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
      ignored = true;
    }
    if (ignored) {
      if (lane == 0) {
        p.row_loss[row] = 0.f;
        if (p.row_lse) p.row_lse[row] = 0.f;
      }
      if (g)
        for (int64_t c = lane; c < C; c += 32) g[c] = from_float<T>(0.f);
      continue;
    }
    float m = -CUDART_INF_F, sx = 0.f;
    for (int64_t c = lane; c < C; c += 32) {
      const float f = to_float(x[c]);
      m = fmaxf(m, f);
      sx += f;
    }
    m = warp_max(m);
    sx = warp_sum(sx);
    const float mm = (m == -CUDART_INF_F) ? 0.f : m;
    float s = 0.f;
    for (int64_t c = lane; c < C; c += 32) {
      const float d = to_float(x[c]) - mm;
      s += kAccurate ? exp_accurate(d) : exp_fast(d);
    }
    s = warp_sum(s);
    const float lse = m + logf(s);
    if (lane == 0) {
      p.row_loss[row] = ce_row_loss(lse, to_float(x[t]), sx, eps, eps_c) * (p.class_weight ? p.class_weight[t] : 1.f);
      if (p.row_lse) p.row_lse[row] = lse;
    }
    if (g) {
      __syncwarp();  // x[t] has been read before an in-place gradient overwrites it
      const float scale = ce_row_scale(p, row, t);
      const float sub_all = eps_c * scale;
      const float sub_t = (1.f - eps) * scale;
      for (int64_t c = lane; c < C; c += 32) {
        const float d = to_float(x[c]) - lse;
        const float pr = kAccurate ? exp_accurate(d) : exp_fast(d);
        float gv = fmaf(pr, scale, -sub_all);
        if (c == t) gv -= sub_t;
        g[c] = from_float<T>(gv);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Bookkeeping kernels.
// ---------------------------------------------------------------------------------------------
// acc[1] += number of rows in this CTA's slice whose target is not ignore_index.  The sum of
// integer-valued doubles below 2^53 is exact, so the atomic order does not change the result.
__global__ void __launch_bounds__(256) ce_count_valid_kernel(const int64_t* __restrict__ target, int64_t rows,
                                                             int64_t classes, int64_t ignore_index, double* acc,
                                                             int32_t* status) {
  __shared__ unsigned int s_cnt[8];
  unsigned int cnt = 0;
  bool bad = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < rows;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t t = target[i];
    if (t != ignore_index) {
      if (t < 0 || t >= classes) bad = true;
      else ++cnt;
    }
  }
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  const bool any_bad = __any_sync(0xffffffffu, bad);
  if ((threadIdx.x & 31) == 0) {
    s_cnt[threadIdx.x >> 5] = cnt;
    if (any_bad && status) atomicOr(status, SB_STATUS_TARGET_OUT_OF_RANGE);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int total = 0;
    for (int w = 0; w < 8; ++w) total += s_cnt[w];
    if (total) atomicAdd(acc + 1, static_cast<double>(total));
  }
}

// ---- exchange of one double between the ranks of a row-sharded job (see sb_xchg) --------------------------------
struct XchgSlot {
  double value;
  unsigned long long seq;
};
static_assert(sizeof(XchgSlot) == 16, "slot layout is part of the C ABI");

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Called by the 32 lanes of one warp: lane r publishes `local` in rank r's slot array and collects rank r's partial from
// this GPU's own array; the sum runs in rank order, so every rank computes the same bits.  The wait is bounded by time
// and by an iteration count; when it runs out the missing partials count as zero and SB_STATUS_KERNEL_TIMEOUT is set.
__device__ double xchg_all_sum(const sb_xchg& x, double local, int32_t* status, unsigned long long limit_ns) {
  const int lane = threadIdx.x & 31;
  const unsigned row = static_cast<unsigned>(x.seq % SB_XCHG_DEPTH) * SB_XCHG_MAX_RANKS;
  double v = 0.0;
  if (lane < x.nranks) {
    XchgSlot* dst = static_cast<XchgSlot*>(x.slots[lane]) + row + x.rank;
    *reinterpret_cast<volatile double*>(&dst->value) = local;
    st_release_sys(&dst->seq, x.seq);  // a reader that sees the number sees the value
    const XchgSlot* src = static_cast<const XchgSlot*>(x.slots[x.rank]) + row + lane;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long max_polls = limit_ns / 128 + 1024;
    bool ok = false;
    for (unsigned long long i = 0; i < max_polls; ++i) {
      if (ld_acquire_sys(&src->seq) == x.seq) {
        ok = true;
        break;
      }
      if (global_timer_ns() - t0 > limit_ns) break;
      __nanosleep(128);
    }
    if (ok) {
      v = *reinterpret_cast<const volatile double*>(&src->value);
    } else {
      v = lane == x.rank ? local : 0.0;
      if (status) atomicOr(status, SB_STATUS_KERNEL_TIMEOUT);
    }
  }
  double total = 0.0;
  for (int r = 0; r < x.nranks; ++r) total += __shfl_sync(0xffffffffu, v, r);
  return total;
}

// acc[1] = number of rows that count (w == null) or the sum of w[target] over them, added in a fixed order by one CTA
// (thread k adds rows k, k + 1024, ... then a tree); acc[0] = 0.  add_existing: the local value is already in acc[1]
// (counted by the many-CTA kernel above for very long target arrays).  has_x: sum the local values over the ranks.
__global__ void __launch_bounds__(1024) ce_count_kernel(const int64_t* __restrict__ target, const float* __restrict__ w, int64_t rows,
                                                        int64_t classes, int64_t ignore_index, double* acc, int32_t* status,
                                                        sb_xchg x, int has_x, int add_existing, unsigned long long limit_ns) {
  grid_dep_launch();  // the sweep that follows may start its loads: it waits for acc[1] itself
  __shared__ double s_part[32];
  double a = 0.0;
  bool bad = false;
  for (int64_t i = threadIdx.x; i < rows; i += 1024) {
    const int64_t t = target[i];
    if (t != ignore_index) {
      if (t < 0 || t >= classes) bad = true;
      else a += w ? static_cast<double>(w[t]) : 1.0;
    }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0 && status) atomicOr(status, SB_STATUS_TARGET_OUT_OF_RANGE);
  a = warp_sum(a);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x < 32) {
    double b = warp_sum(s_part[threadIdx.x]);
    if (add_existing) b += acc[1];
    if (has_x) b = xchg_all_sum(x, b, status, limit_ns);
    if (threadIdx.x == 0) {
      acc[0] = 0.0;
      acc[1] = b;
    }
  }
}

// Fixed-order sum of row_loss in double: thread k adds elements k, k+1024, ... then a tree.  has_x: the local sums are
// added over the ranks before the division.  Always launched as a programmatic dependent: nothing is read before
// grid_dep_wait returns.
template <bool FINISH>
__global__ void __launch_bounds__(1024) ce_loss_sum_kernel(const float* __restrict__ row_loss, int64_t rows, double* acc,
                                                           int reduction, void* out, int out_dtype, int32_t* status, sb_xchg x,
                                                           int has_x, unsigned long long limit_ns) {
  grid_dep_wait();
  __shared__ double s_part[32];
  double a = 0.0;
  for (int64_t i = threadIdx.x; i < rows; i += 1024) a += static_cast<double>(row_loss[i]);
  a = warp_sum(a);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x < 32) {
    double b = warp_sum(s_part[threadIdx.x]);
    if (has_x) b = xchg_all_sum(x, b, status, limit_ns);
    if (threadIdx.x == 0) {
      acc[0] = b;
      if (FINISH) ce_store_loss(b, acc[1], reduction, out, out_dtype);
    }
  }
}

__global__ void ce_loss_finish_kernel(const double* acc, int reduction, void* out, int out_dtype) {
  if (threadIdx.x == 0 && blockIdx.x == 0) ce_store_loss(acc[0], acc[1], reduction, out, out_dtype);
}

template <typename T>
__device__ __forceinline__ float load_scalar_as_float(const void* p) {
  return to_float(*static_cast<const T*>(p));
}

// dst = src * (*scale / *applied_in) (the divisor is 1 when applied_in is null).  In place, a factor of exactly 1 skips
// the sweep; block 0 records *applied_out = *scale when asked to.  The two words differ, so every CTA reads the old
// factor whenever it runs.  A stored factor of zero has wiped the gradient: NaN and SB_STATUS_GRADIENT_LOST, unless the
// new factor is zero as well.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) ce_rescale_kernel(const T* src, T* dst, int64_t numel, const void* scale, int scale_dtype,
                                                         const float* applied_in, float* applied_out, int32_t* status) {
  float sc;
  switch (scale_dtype) {
    case SB_F32: sc = load_scalar_as_float<float>(scale); break;
    case SB_BF16: sc = load_scalar_as_float<__nv_bfloat16>(scale); break;
    case SB_F16: sc = load_scalar_as_float<__half>(scale); break;
    default: sc = load_scalar_as_float<double>(scale); break;
  }
  float factor = sc;
  if (applied_in) {
    const float was = *applied_in;
    if (was == 0.f) {
      factor = sc == 0.f ? 0.f : CUDART_NAN_F;
      if (sc != 0.f && blockIdx.x == 0 && threadIdx.x == 0 && status) atomicOr(status, SB_STATUS_GRADIENT_LOST);
    } else {
      factor = sc / was;
    }
  }
  if (applied_out && blockIdx.x == 0 && threadIdx.x == 0) *applied_out = sc;
  if (factor == 1.f && src == dst) return;
  const int64_t nvec = numel / VEC;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    Vec<T, VEC> v = load_vec<T, VEC>(src + i * VEC);
#pragma unroll
    for (int k = 0; k < VEC; ++k) v.v[k] = from_float<T>(to_float(v.v[k]) * factor);
    store_vec<T, VEC>(dst + i * VEC, v);
  }
  if (blockIdx.x == 0)
    for (int64_t i = nvec * VEC + threadIdx.x; i < numel; i += 256) dst[i] = from_float<T>(to_float(src[i]) * factor);
}

// ---------------------------------------------------------------------------------------------
// Host side.
// ---------------------------------------------------------------------------------------------
template <typename T>
static int launch_generic(const CEParams& p, cudaStream_t st) {
  constexpr int kVec = 16 / sizeof(T);
  const int sms = sm_count();
  const bool ws = p.class_weight && p.label_smoothing != 0.f;
  if (p.classes <= 1024 && !ws) {
    constexpr int kThreads = 256;
    const int64_t ctas = (p.rows + kThreads / 32 - 1) / (kThreads / 32);
    const int grid = static_cast<int>(ctas < static_cast<int64_t>(sms) * 8 ? ctas : static_cast<int64_t>(sms) * 8);
    ce_rows_warp_kernel<T, kThreads><<<grid, kThreads, 0, st>>>(p);
    return launch_status();
  }
  constexpr int kThreads = 512;
  const int64_t max_grid = static_cast<int64_t>(sms) * 4;
  const int grid = static_cast<int>(p.rows < max_grid ? p.rows : max_grid);
  const bool aligned = (p.classes % kVec == 0) && (reinterpret_cast<uintptr_t>(p.logits) % 16 == 0) &&
                       (p.grad == nullptr || reinterpret_cast<uintptr_t>(p.grad) % 16 == 0);
  if (ws) {
    if (aligned) ce_rows_cta_kernel<T, kVec, kThreads, true><<<grid, kThreads, 0, st>>>(p);
    else ce_rows_cta_kernel<T, 1, kThreads, true><<<grid, kThreads, 0, st>>>(p);
  } else if (aligned) {
    ce_rows_cta_kernel<T, kVec, kThreads><<<grid, kThreads, 0, st>>>(p);
  } else {
    ce_rows_cta_kernel<T, 1, kThreads><<<grid, kThreads, 0, st>>>(p);
  }
  return launch_status();
}

int ce_launch_generic(const CEParams& p, cudaStream_t st) {
  switch (p.dtype) {
    case SB_F32: return launch_generic<float>(p, st);
    case SB_BF16: return launch_generic<__nv_bfloat16>(p, st);
    case SB_F16: return launch_generic<__half>(p, st);
    default: return SB_ERR_UNSUPPORTED;
  }
}

namespace {
int g_xchg_timeout_ms = 10000;

bool xchg_ok(const sb_xchg* x) {
  if (!x) return true;
  if (x->nranks < 1 || x->nranks > SB_XCHG_MAX_RANKS || x->rank < 0 || x->rank >= x->nranks || x->seq == 0) return false;
  for (int r = 0; r < x->nranks; ++r)
    if (!x->slots[r] || reinterpret_cast<uintptr_t>(x->slots[r]) % 16) return false;
  return true;
}

// One-CTA launch with the programmatic-dependent attribute (the kernel begins with grid_dep_wait).
template <class K, class... Args>
int launch_dependent(K kernel, cudaStream_t st, Args... args) {
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(1024);
  cfg.stream = st;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess) {
    cudaGetLastError();
    return SB_ERR_CUDA;
  }
  return SB_OK;
}

int launch_count(const int64_t* target, const float* w, int64_t rows, int64_t classes, int64_t ignore_index, double* acc,
                 int32_t* status, const sb_xchg* x, cudaStream_t st) {
  const unsigned long long limit_ns = static_cast<unsigned long long>(g_xchg_timeout_ms) * 1000000ULL;
  const sb_xchg xv = x ? *x : sb_xchg{};
  // One CTA reads up to half a million targets (4 MB) in a few microseconds; beyond that the unweighted count is spread
  // over many CTAs first (exact in any order) and the one-CTA kernel only finishes it.
  if (!w && rows > (1 << 19)) {
    if (cudaMemsetAsync(acc, 0, 2 * sizeof(double), st) != cudaSuccess) return SB_ERR_CUDA;
    const int64_t ctas = (rows + 255) / 256;
    const int grid = static_cast<int>(ctas < 4 * sm_count() ? ctas : 4 * sm_count());
    ce_count_valid_kernel<<<grid, 256, 0, st>>>(target, rows, classes, ignore_index, acc, status);
    if (launch_status() != SB_OK) return SB_ERR_CUDA;
    ce_count_kernel<<<1, 1024, 0, st>>>(target, nullptr, 0, classes, ignore_index, acc, status, xv, x ? 1 : 0, 1, limit_ns);
    return launch_status();
  }
  ce_count_kernel<<<1, 1024, 0, st>>>(target, w, rows, classes, ignore_index, acc, status, xv, x ? 1 : 0, 0, limit_ns);
  return launch_status();
}
}  // namespace

int xchg_set_timeout_ms(int ms) {
  g_xchg_timeout_ms = ms;
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_ce_count_valid(const int64_t* target, int64_t rows, int64_t classes, int64_t ignore_index, double* acc,
                      int32_t* status, sb_stream_t stream) {
  if (rows < 0 || classes < 0 || !acc || (rows > 0 && !target)) return SB_ERR_INVALID_ARGUMENT;
  return launch_count(target, nullptr, rows, classes, ignore_index, acc, status, nullptr, as_stream(stream));
}

int sb_ce_count_weighted(const int64_t* target, const float* class_weight, int64_t rows, int64_t classes, int64_t ignore_index,
                         double* acc, int32_t* status, sb_stream_t stream) {
  if (rows < 0 || classes < 0 || !acc || !class_weight || (rows > 0 && !target)) return SB_ERR_INVALID_ARGUMENT;
  return launch_count(target, class_weight, rows, classes, ignore_index, acc, status, nullptr, as_stream(stream));
}

int sb_ce_count_exchange(const int64_t* target, const float* class_weight, int64_t rows, int64_t classes, int64_t ignore_index,
                         double* acc, int32_t* status, const sb_xchg* x, sb_stream_t stream) {
  if (rows < 0 || classes < 0 || !acc || (rows > 0 && !target) || !xchg_ok(x)) return SB_ERR_INVALID_ARGUMENT;
  return launch_count(target, class_weight, rows, classes, ignore_index, acc, status, x, as_stream(stream));
}

// Argument checks of the fused sweep, shared with the entry point that brings its own scratch.
static int ce_check_args(const sb_ce_args* a, bool need_row_loss) {
  if (!a) return SB_ERR_INVALID_ARGUMENT;
  if (a->rows < 0 || a->classes < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->rows == 0) return SB_OK;
  if (a->classes == 0) return SB_ERR_INVALID_ARGUMENT;
  if (!a->logits || !a->target || (need_row_loss && !a->row_loss)) return SB_ERR_INVALID_ARGUMENT;
  if (a->dtype != SB_F32 && a->dtype != SB_BF16 && a->dtype != SB_F16) return SB_ERR_UNSUPPORTED;
  if (a->reduction < SB_REDUCTION_NONE || a->reduction > SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  if (!(a->label_smoothing >= 0.f && a->label_smoothing <= 1.f)) return SB_ERR_INVALID_ARGUMENT;
  if (a->flags & ~SB_CE_FLAG_AFTER_COUNT) return SB_ERR_INVALID_ARGUMENT;
  const size_t es = dtype_size(a->dtype);
  if (reinterpret_cast<uintptr_t>(a->logits) % es || reinterpret_cast<uintptr_t>(a->grad_logits) % es)
    return SB_ERR_MISALIGNED;
  return SB_OK;
}

int sb_ce_forward_backward(const sb_ce_args* a, sb_stream_t stream) {
  const int rc = ce_check_args(a, true);
  if (rc != SB_OK) return rc;
  if (a->rows == 0) return SB_OK;
  if (a->grad_logits && a->reduction == SB_REDUCTION_MEAN && !a->acc) return SB_ERR_INVALID_ARGUMENT;
  CEParams p;
  p.logits = a->logits;
  p.grad = a->grad_logits;
  p.target = a->target;
  p.row_loss = a->row_loss;
  p.row_lse = a->row_lse;
  p.row_grad_out = a->row_grad_out;
  p.acc = a->acc;
  p.rows = a->rows;
  p.classes = a->classes;
  p.ignore_index = a->ignore_index;
  p.label_smoothing = a->label_smoothing;
  p.grad_scale = a->grad_scale;
  p.reduction = a->reduction;
  p.dtype = a->dtype;
  p.status = a->status;
  p.class_weight = a->class_weight;
  p.flags = a->flags;
  return ce_dispatch(p, as_stream(stream));
}

static bool loss_dtype_ok(int dt) { return dt == SB_F32 || dt == SB_BF16 || dt == SB_F16 || dt == SB_F64; }

int sb_ce_loss_sum(const float* row_loss, int64_t rows, double* acc, sb_stream_t stream) {
  if (rows < 0 || !acc || (rows > 0 && !row_loss)) return SB_ERR_INVALID_ARGUMENT;
  return launch_dependent(ce_loss_sum_kernel<false>, as_stream(stream), row_loss, rows, acc, 0, static_cast<void*>(nullptr), 0,
                          static_cast<int32_t*>(nullptr), sb_xchg{}, 0, 0ULL);
}

int sb_ce_loss_finish(const double* acc, int32_t reduction, void* out, int32_t dtype, sb_stream_t stream) {
  if (!acc || !out) return SB_ERR_INVALID_ARGUMENT;
  if (!loss_dtype_ok(dtype)) return SB_ERR_UNSUPPORTED;
  if (reduction != SB_REDUCTION_MEAN && reduction != SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  ce_loss_finish_kernel<<<1, 32, 0, as_stream(stream)>>>(acc, reduction, out, dtype);
  return launch_status();
}

int sb_ce_loss_sum_finish(const float* row_loss, int64_t rows, double* acc, int32_t reduction, void* out, int32_t dtype,
                          sb_stream_t stream) {
  return sb_ce_loss_exchange(row_loss, rows, acc, reduction, out, dtype, nullptr, nullptr, stream);
}

int sb_ce_loss_exchange(const float* row_loss, int64_t rows, double* acc, int32_t reduction, void* out, int32_t dtype, int32_t* status,
                        const sb_xchg* x, sb_stream_t stream) {
  if (rows < 0 || !acc || !out || (rows > 0 && !row_loss) || !xchg_ok(x)) return SB_ERR_INVALID_ARGUMENT;
  if (!loss_dtype_ok(dtype)) return SB_ERR_UNSUPPORTED;
  if (reduction != SB_REDUCTION_MEAN && reduction != SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  const unsigned long long limit_ns = static_cast<unsigned long long>(g_xchg_timeout_ms) * 1000000ULL;
  return launch_dependent(ce_loss_sum_kernel<true>, as_stream(stream), row_loss, rows, acc, static_cast<int>(reduction), out,
                          static_cast<int>(dtype), status, x ? *x : sb_xchg{}, x ? 1 : 0, limit_ns);
}

int sb_ce_rescale_grad(const void* src, void* dst, int32_t dtype, int64_t numel, const void* scale, int32_t scale_dtype,
                       const float* applied_in, float* applied_out, int32_t* status, sb_stream_t stream) {
  if (numel < 0 || !scale || (applied_out && applied_in == applied_out) || (numel > 0 && (!src || !dst))) return SB_ERR_INVALID_ARGUMENT;
  if (!loss_dtype_ok(scale_dtype)) return SB_ERR_UNSUPPORTED;
  cudaStream_t st = as_stream(stream);
  const int64_t want = (numel / 8 + 255) / 256 + 1;
  const int grid = static_cast<int>(want < 8LL * sm_count() ? want : 8LL * sm_count());
  const bool al = reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
#define SB_RESCALE(T, V) \
  ce_rescale_kernel<T, V><<<grid, 256, 0, st>>>(static_cast<const T*>(src), static_cast<T*>(dst), numel, scale, scale_dtype, applied_in, applied_out, status)
  switch (dtype) {
    case SB_F32:
      if (al) SB_RESCALE(float, 4);
      else SB_RESCALE(float, 1);
      break;
    case SB_BF16:
      if (al) SB_RESCALE(__nv_bfloat16, 8);
      else SB_RESCALE(__nv_bfloat16, 1);
      break;
    case SB_F16:
      if (al) SB_RESCALE(__half, 8);
      else SB_RESCALE(__half, 1);
      break;
    default: return SB_ERR_UNSUPPORTED;
  }
#undef SB_RESCALE
  return launch_status();
}

// ---- cross entropy with library-owned scratch ------------------------------------------------------------
// Layout of the static array: bytes [0, 16) = the accumulator {loss sum, valid rows} as two doubles, bytes
// [256, 256 + 4 * rows) = the per-row losses.  Host code cannot use the symbol as a pointer; the device
// address is looked up once per device with cudaGetSymbolAddress while that device is current.
static __device__ __align__(256) unsigned char g_ce_static_scratch[SB_CE_STATIC_MAX_ROWS * sizeof(float) + 256];

namespace {
constexpr int kStaticMaxDevices = 64;
void* g_ce_static_ptr[kStaticMaxDevices];  // device address of g_ce_static_scratch per device, once resolved

int ce_static_scratch(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return SB_ERR_CUDA;
  void* p = __atomic_load_n(&g_ce_static_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_ce_static_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return SB_ERR_CUDA;
    }
    __atomic_store_n(&g_ce_static_ptr[dev], p, __ATOMIC_RELEASE);  // every thread resolves the same address
  }
  *out = static_cast<unsigned char*>(p);
  return SB_OK;
}
}  // namespace

int sb_ce_loss_static_scratch(const sb_ce_args* a, void* loss_out, sb_stream_t stream) {
  if (!a || !loss_out) return SB_ERR_INVALID_ARGUMENT;
  if (a->reduction != SB_REDUCTION_MEAN && a->reduction != SB_REDUCTION_SUM) return SB_ERR_INVALID_ARGUMENT;
  if (a->row_loss || a->row_lse || a->row_grad_out || a->acc) return SB_ERR_INVALID_ARGUMENT;
  if (a->rows < 0) return SB_ERR_INVALID_ARGUMENT;
  if (a->rows > SB_CE_STATIC_MAX_ROWS) return SB_ERR_TOO_LARGE;
  // every check of the sweep runs before the first launch: an invalid call must not touch the shared array
  int rc = ce_check_args(a, false);
  if (rc != SB_OK) return rc;
  if (a->rows > 0 && (!a->target || a->classes <= 0)) return SB_ERR_INVALID_ARGUMENT;
  unsigned char* scratch = nullptr;
  rc = ce_static_scratch(&scratch);
  if (rc != SB_OK) return rc;
  double* acc = reinterpret_cast<double*>(scratch);
  float* row_loss = reinterpret_cast<float*>(scratch + 256);
  // The count kernel writes both accumulator words; the sweep writes row_loss[0 .. rows) before the sum reads it.
  rc = a->class_weight ? sb_ce_count_weighted(a->target, a->class_weight, a->rows, a->classes, a->ignore_index, acc, a->status, stream)
                       : sb_ce_count_valid(a->target, a->rows, a->classes, a->ignore_index, acc, a->status, stream);
  if (rc != SB_OK) return rc;
  sb_ce_args full = *a;
  full.row_loss = row_loss;
  full.acc = acc;
  full.flags = 0;
  rc = sb_ce_forward_backward(&full, stream);
  if (rc != SB_OK) return rc;
  return sb_ce_loss_sum_finish(row_loss, a->rows, acc, a->reduction, loss_out, a->dtype, stream);
}

}  // extern "C"

/*
 * oracle.c -- CPU restatement of the operator hot path, used ONLY as the checker.
 *
 * TEST INFRASTRUCTURE.  Nothing under torch_supa_b200/ loads, links or calls this file; the tests,
 * the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Every function restates, in plain C with double accumulation, the arithmetic of one piece of the
 * torch-supa operator path.  Paths are relative to the torch-supa source tree.  The reference's
 * device code cannot be compiled outside its vendor toolchain, and its tests hold no stored vectors:
 * they compare with PyTorch's CPU kernels (torch_supa/testing/common_utils.py:151-168,
 * test/test_loss.py:235-276).  This restatement is therefore pinned against fixtures produced by
 * those same PyTorch CPU kernels (tests/golden/).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#define ORACLE_API __attribute__((visibility("default")))

enum { RED_NONE = 0, RED_MEAN = 1, RED_SUM = 2 };

/* Row statistics as in cross_entropy_index_mean_kernel
 * (torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:144-160): a max pass,
 * a sum-of-exp pass, lse = log(sum) + max. */
static double row_lse(const float* x, int64_t classes, double* sum_x) {
  double m = -INFINITY, s = 0.0, sx = 0.0;
  for (int64_t c = 0; c < classes; ++c)
    if ((double)x[c] > m) m = (double)x[c];
  for (int64_t c = 0; c < classes; ++c) {
    s += exp((double)x[c] - m);
    sx += (double)x[c];
  }
  if (sum_x) *sum_x = sx;
  return log(s) + m;
}

/* Cross entropy with class-index targets.
 *   forward : loss_i = lse_i - x[i, t_i] (CrossEntropyLossKernel.cu:157), rows with
 *             t_i == ignore_index give 0 and do not count (:134-141); mean = sum / count, NaN when the
 *             count is 0 (:164-195); label smoothing as in the upstream composite the reference defers
 *             to (torch_supa/csrc/aten/ops/CrossEntropyLoss.cpp:50):
 *             loss_i = (1 - eps) * (lse_i - x[i, t_i]) + eps / C * sum_c (lse_i - x[i, c]).
 *   backward: the chain nll_loss_backward -> _log_softmax_backward_data of
 *             CrossEntropyLoss.cpp:94-135, which is
 *             grad[i, c] = (softmax[i, c] - (1 - eps) [c == t_i] - eps / C) * g / count (mean) or * g.
 * `loss` holds 1 double (mean, sum) or `rows` doubles (none); `row_grad_out` is the per-row upstream
 * gradient for none (NULL = 1); `grad` may be NULL.  Returns the number of out-of-range targets
 * (those rows are treated as ignored). */
ORACLE_API int64_t oracle_cross_entropy(const float* logits, const int64_t* target, int64_t rows, int64_t classes,
                                        int64_t ignore_index, double label_smoothing, int reduction, double grad_out,
                                        const double* row_grad_out, double* loss, double* grad) {
  int64_t bad = 0;
  double count = 0.0, total = 0.0;
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t t = target[i];
    if (t != ignore_index && t >= 0 && t < classes) count += 1.0;
  }
  for (int64_t i = 0; i < rows; ++i) {
    const float* x = logits + i * classes;
    const int64_t t = target[i];
    int ignored = (t == ignore_index);
    if (!ignored && (t < 0 || t >= classes)) {
      ++bad;
      ignored = 1;
    }
    double li = 0.0;
    if (!ignored) {
      double sx;
      const double lse = row_lse(x, classes, &sx);
      li = (1.0 - label_smoothing) * (lse - (double)x[t]) + label_smoothing / (double)classes * ((double)classes * lse - sx);
      if (grad) {
        double scale = grad_out;
        if (reduction == RED_MEAN) scale /= count;
        if (reduction == RED_NONE && row_grad_out) scale *= row_grad_out[i];
        for (int64_t c = 0; c < classes; ++c) {
          double g = exp((double)x[c] - lse) - label_smoothing / (double)classes;
          if (c == t) g -= 1.0 - label_smoothing;
          grad[i * classes + c] = g * scale;
        }
      }
    } else if (grad) {
      for (int64_t c = 0; c < classes; ++c) grad[i * classes + c] = 0.0;
    }
    if (reduction == RED_NONE) loss[i] = li;
    else total += li;
  }
  if (reduction == RED_MEAN) loss[0] = count > 0.0 ? total / count : NAN;
  else if (reduction == RED_SUM) loss[0] = total;
  return bad;
}

/* log_softmax over the middle dimension of [outer, dim, inner]: x - max - log(sum exp(x - max)),
 * the operator behind at::log_softmax at CrossEntropyLoss.cpp:76. */
ORACLE_API void oracle_log_softmax(const float* x, int64_t outer, int64_t dim, int64_t inner, double* out) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float* p = x + o * dim * inner + i;
      double m = -INFINITY, s = 0.0;
      for (int64_t d = 0; d < dim; ++d)
        if ((double)p[d * inner] > m) m = (double)p[d * inner];
      for (int64_t d = 0; d < dim; ++d) s += exp((double)p[d * inner] - m);
      const double lse = m + log(s);
      for (int64_t d = 0; d < dim; ++d) out[o * dim * inner + d * inner + i] = (double)p[d * inner] - lse;
    }
}

/* _log_softmax_backward_data (CrossEntropyLoss.cpp:132): grad_in = g - exp(y) * sum_dim(g). */
ORACLE_API void oracle_log_softmax_backward(const float* g, const float* y, int64_t outer, int64_t dim, int64_t inner,
                                            double* grad_in) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t base = o * dim * inner + i;
      double s = 0.0;
      for (int64_t d = 0; d < dim; ++d) s += (double)g[base + d * inner];
      for (int64_t d = 0; d < dim; ++d)
        grad_in[base + d * inner] = (double)g[base + d * inner] - exp((double)y[base + d * inner]) * s;
    }
}

/* softmax and its backward over the middle dimension of [outer, dim, inner] (exercised by the reference's
 * test/test_softmax.py and test/test_persistent_softmax.py; the kernels live in its external native-op library):
 * y = exp(x - max) / sum exp(x - max);  grad_in = y * (g - sum_dim(g * y)). */
ORACLE_API void oracle_softmax(const float* x, int64_t outer, int64_t dim, int64_t inner, double* out) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float* p = x + o * dim * inner + i;
      double m = -INFINITY, s = 0.0;
      for (int64_t d = 0; d < dim; ++d)
        if ((double)p[d * inner] > m) m = (double)p[d * inner];
      for (int64_t d = 0; d < dim; ++d) s += exp((double)p[d * inner] - m);
      for (int64_t d = 0; d < dim; ++d) out[o * dim * inner + d * inner + i] = exp((double)p[d * inner] - m) / s;
    }
}

ORACLE_API void oracle_softmax_backward(const float* g, const float* y, int64_t outer, int64_t dim, int64_t inner, double* grad_in) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t base = o * dim * inner + i;
      double s = 0.0;
      for (int64_t d = 0; d < dim; ++d) s += (double)g[base + d * inner] * (double)y[base + d * inner];
      for (int64_t d = 0; d < dim; ++d) grad_in[base + d * inner] = (double)y[base + d * inner] * ((double)g[base + d * inner] - s);
    }
}

/* nll_loss_forward (CrossEntropyLoss.cpp:79): -w[t] x[i, t]; total_weight = sum of w[t] over counted rows. */
ORACLE_API void oracle_nll_loss(const float* logp, const int64_t* target, const float* weight, int64_t rows,
                                int64_t classes, int64_t ignore_index, int reduction, double* out, double* total_weight) {
  double tot = 0.0, tw = 0.0;
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t t = target[i];
    double v = 0.0;
    if (t != ignore_index && t >= 0 && t < classes) {
      const double w = weight ? (double)weight[t] : 1.0;
      v = -w * (double)logp[i * classes + t];
      tw += w;
    }
    if (reduction == RED_NONE) out[i] = v;
    else tot += v;
  }
  if (reduction == RED_MEAN) out[0] = tot / tw;
  else if (reduction == RED_SUM) out[0] = tot;
  *total_weight = tw;
}

/* nll_loss_backward (CrossEntropyLoss.cpp:127). */
ORACLE_API void oracle_nll_loss_backward(const double* grad_out, const int64_t* target, const float* weight, int64_t rows,
                                         int64_t classes, int64_t ignore_index, int reduction, double total_weight,
                                         double* grad_in) {
  for (int64_t i = 0; i < rows * classes; ++i) grad_in[i] = 0.0;
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t t = target[i];
    if (t == ignore_index || t < 0 || t >= classes) continue;
    const double w = weight ? (double)weight[t] : 1.0;
    double g = reduction == RED_NONE ? grad_out[i] : grad_out[0];
    if (reduction == RED_MEAN) g /= total_weight;
    grad_in[i * classes + t] = -w * g;
  }
}

/* nll_loss2d_forward / nll_loss2d_backward: the same rule per sample (n, i) of log-probabilities laid out
 * [outer, classes, inner] with targets [outer, inner] (inner = H * W for the 4-D form exercised by the
 * reference's test/test_loss.py:24,150-233; the kernels themselves live in its external native-op library). */
ORACLE_API void oracle_nll_loss_nd(const float* logp, const int64_t* target, const float* weight, int64_t outer,
                                   int64_t classes, int64_t inner, int64_t ignore_index, int reduction, double* out,
                                   double* total_weight) {
  double tot = 0.0, tw = 0.0;
  for (int64_t n = 0; n < outer; ++n)
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t t = target[n * inner + i];
      double v = 0.0;
      if (t != ignore_index && t >= 0 && t < classes) {
        const double w = weight ? (double)weight[t] : 1.0;
        v = -w * (double)logp[(n * classes + t) * inner + i];
        tw += w;
      }
      if (reduction == RED_NONE) out[n * inner + i] = v;
      else tot += v;
    }
  if (reduction == RED_MEAN) out[0] = tot / tw;
  else if (reduction == RED_SUM) out[0] = tot;
  *total_weight = tw;
}

ORACLE_API void oracle_nll_loss_nd_backward(const double* grad_out, const int64_t* target, const float* weight, int64_t outer,
                                            int64_t classes, int64_t inner, int64_t ignore_index, int reduction,
                                            double total_weight, double* grad_in) {
  for (int64_t i = 0; i < outer * classes * inner; ++i) grad_in[i] = 0.0;
  for (int64_t n = 0; n < outer; ++n)
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t t = target[n * inner + i];
      if (t == ignore_index || t < 0 || t >= classes) continue;
      const double w = weight ? (double)weight[t] : 1.0;
      double g = reduction == RED_NONE ? grad_out[n * inner + i] : grad_out[0];
      if (reduction == RED_MEAN) g /= total_weight;
      grad_in[(n * classes + t) * inner + i] = -w * g;
    }
}

/* binary_cross_entropy_with_logits, unreduced (torch_supa/csrc/aten/ops/kernels/elementwise/
 * BinaryCrossEntropyWithLogitsKernel.cu:16-36): (1 - t) x + lw (max(-x, 0) + log(exp(-max) + exp(-x - max))),
 * lw = (pw - 1) t + 1; weight multiplies the result (:53-60).  pos_weight / weight may be NULL; all arrays are
 * already broadcast to n elements.  grad = d loss / d x = (lw sigmoid(x) - pw t) * weight. */
ORACLE_API void oracle_bce_with_logits(const float* x, const float* t, const float* pos_weight, const float* weight, int64_t n,
                                       double* loss, double* grad) {
  for (int64_t i = 0; i < n; ++i) {
    const double xi = (double)x[i], ti = (double)t[i];
    const double pw = pos_weight ? (double)pos_weight[i] : 1.0, w = weight ? (double)weight[i] : 1.0;
    const double max_val = xi < 0.0 ? -xi : 0.0;
    const double lw = (pw - 1.0) * ti + 1.0;
    const double sp = max_val + log(exp(-max_val) + exp(-xi - max_val));
    loss[i] = ((1.0 - ti) * xi + lw * sp) * w;
    const double sg = 1.0 / (1.0 + exp(-xi));
    grad[i] = (lw * sg - pw * ti) * w;
  }
}

/* Row reductions with a wide accumulator (sum_functor / MeanOps / MaxNanFunctor of
 * torch_supa/csrc/aten/ops/kernels/reduce/ReduceSumKernel.cu:80-100, ReduceMomentKernel.cu:16-35).
 * op: 0 sum, 1 mean, 2 amax (NaN propagates), 3 amin. */
ORACLE_API void oracle_reduce_rows(const float* x, int64_t rows, int64_t len, int op, double* out) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* p = x + r * len;
    if (op <= 1) {
      double s = 0.0;
      for (int64_t i = 0; i < len; ++i) s += (double)p[i];
      out[r] = op == 1 ? s / (double)len : s;
    } else {
      double m = op == 2 ? -INFINITY : INFINITY;
      int nan = 0;
      for (int64_t i = 0; i < len; ++i) {
        const double v = (double)p[i];
        if (v != v) nan = 1;
        if (op == 2 ? v > m : v < m) m = v;
      }
      out[r] = nan ? NAN : m;
    }
  }
}

/* Cross entropy with class weights, label smoothing and class-index targets: the arithmetic of the upstream composite the
 * reference reaches for every weighted call (torch_supa/csrc/aten/ops/CrossEntropyLoss.cpp:23-33,50): the nll part is
 * weighted by w[t_i], the smoothing part weights every class c by w[c]; mean divides both by sum_i w[t_i].
 *   loss_i  = (1 - eps) w[t_i] (lse_i - x[i, t_i]) + eps / C * sum_c w[c] (lse_i - x[i, c])
 *   grad_ic = softmax_ic ((1 - eps) w[t_i] + eps / C * W) - (1 - eps) w[t_i] [c == t_i] - eps / C * w[c],  W = sum_c w[c]
 * weight == NULL means all ones (then this equals oracle_cross_entropy). */
ORACLE_API int64_t oracle_cross_entropy_weighted(const float* logits, const int64_t* target, const float* weight, int64_t rows,
                                                 int64_t classes, int64_t ignore_index, double label_smoothing, int reduction,
                                                 double grad_out, const double* row_grad_out, double* loss, double* grad) {
  int64_t bad = 0;
  double denom = 0.0, total = 0.0, wsum = 0.0;
  for (int64_t c = 0; c < classes; ++c) wsum += weight ? (double)weight[c] : 1.0;
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t t = target[i];
    if (t != ignore_index && t >= 0 && t < classes) denom += weight ? (double)weight[t] : 1.0;
  }
  for (int64_t i = 0; i < rows; ++i) {
    const float* x = logits + i * classes;
    const int64_t t = target[i];
    int ignored = (t == ignore_index);
    if (!ignored && (t < 0 || t >= classes)) {
      ++bad;
      ignored = 1;
    }
    double li = 0.0;
    if (!ignored) {
      const double lse = row_lse(x, classes, NULL);
      const double wt = weight ? (double)weight[t] : 1.0;
      double swx = 0.0;
      for (int64_t c = 0; c < classes; ++c) swx += (weight ? (double)weight[c] : 1.0) * (double)x[c];
      li = (1.0 - label_smoothing) * wt * (lse - (double)x[t]) + label_smoothing / (double)classes * (wsum * lse - swx);
      if (grad) {
        double scale = grad_out;
        if (reduction == RED_MEAN) scale /= denom;
        if (reduction == RED_NONE && row_grad_out) scale *= row_grad_out[i];
        const double pfac = (1.0 - label_smoothing) * wt + label_smoothing / (double)classes * wsum;
        for (int64_t c = 0; c < classes; ++c) {
          double g = exp((double)x[c] - lse) * pfac - label_smoothing / (double)classes * (weight ? (double)weight[c] : 1.0);
          if (c == t) g -= (1.0 - label_smoothing) * wt;
          grad[i * classes + c] = g * scale;
        }
      }
    } else if (grad) {
      for (int64_t c = 0; c < classes; ++c) grad[i * classes + c] = 0.0;
    }
    if (reduction == RED_NONE) loss[i] = li;
    else total += li;
  }
  if (reduction == RED_MEAN) loss[0] = denom > 0.0 ? total / denom : NAN;
  else if (reduction == RED_SUM) loss[0] = total;
  return bad;
}

/* Cross entropy with class-probability targets (cross_entropy_prob_kernel,
 * torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:545-564, with the smoothing and the weights
 * of the composite): q_c = t_c (1 - eps) + eps / C,
 *   loss_i = sum_c w[c] q_ic (lse_i - x[i, c]);  mean divides by the number of rows;
 *   grad_ic = softmax_ic * sum_k w[k] q_ik - w[c] q_ic. */
ORACLE_API void oracle_cross_entropy_prob(const float* logits, const float* target, const float* weight, int64_t rows, int64_t classes,
                                          double label_smoothing, int reduction, double grad_out, const double* row_grad_out,
                                          double* loss, double* grad) {
  double total = 0.0;
  for (int64_t i = 0; i < rows; ++i) {
    const float* x = logits + i * classes;
    const float* t = target + i * classes;
    const double lse = row_lse(x, classes, NULL);
    double a = 0.0, li = 0.0;
    for (int64_t c = 0; c < classes; ++c) {
      const double q = ((double)t[c] * (1.0 - label_smoothing) + label_smoothing / (double)classes) * (weight ? (double)weight[c] : 1.0);
      a += q;
      li += q * (lse - (double)x[c]);
    }
    if (grad) {
      double scale = grad_out;
      if (reduction == RED_MEAN) scale /= (double)rows;
      if (reduction == RED_NONE && row_grad_out) scale *= row_grad_out[i];
      for (int64_t c = 0; c < classes; ++c) {
        const double q = ((double)t[c] * (1.0 - label_smoothing) + label_smoothing / (double)classes) * (weight ? (double)weight[c] : 1.0);
        grad[i * classes + c] = (exp((double)x[c] - lse) * a - q) * scale;
      }
    }
    if (reduction == RED_NONE) loss[i] = li;
    else total += li;
  }
  if (reduction == RED_MEAN) loss[0] = rows > 0 ? total / (double)rows : NAN;
  else if (reduction == RED_SUM) loss[0] = total;
}

/* Extremum and its index along the middle dimension of [outer, len, inner] (the reduce family behind argmax / max.dim,
 * torch_supa/csrc/aten/ops/kernels/reduce/Reduce.cuh:1040-1333, with the index rules of the CPU golden): the first of
 * equal extrema; NaN wins over every number, for max and for min, the first NaN if there are several. */
ORACLE_API void oracle_arg_reduce(const double* x, int64_t outer, int64_t len, int64_t inner, int is_max, double* values,
                                  int64_t* indices) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const double* p = x + o * len * inner + i;
      double best = p[0];
      int64_t at = 0;
      for (int64_t k = 1; k < len; ++k) {
        const double v = p[k * inner];
        if (best != best) break;
        if (v != v || (is_max ? v > best : v < best)) {
          best = v;
          at = k;
        }
      }
      values[o * inner + i] = best;
      indices[o * inner + i] = at;
    }
}

/* Variance / standard deviation with a correction and the mean, along the middle dimension of [outer, len, inner]
 * (torch_supa/csrc/aten/ops/StdVar.cpp:34-63): two passes in double, M2 / max(0, len - correction). */
ORACLE_API void oracle_moments(const double* x, int64_t outer, int64_t len, int64_t inner, double correction, int take_sqrt,
                               double* out, double* mean_out) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const double* p = x + o * len * inner + i;
      double m = 0.0, m2 = 0.0;
      for (int64_t k = 0; k < len; ++k) m += p[k * inner];
      m /= (double)len;
      for (int64_t k = 0; k < len; ++k) m2 += (p[k * inner] - m) * (p[k * inner] - m);
      const double denom = (double)len - correction > 0.0 ? (double)len - correction : 0.0;
      const double v = m2 / denom;
      out[o * inner + i] = take_sqrt ? sqrt(v) : v;
      if (mean_out) mean_out[o * inner + i] = m;
    }
}

/* div with a rounding mode on integers (BinaryDivTruncKernel.cu, BinaryDivFloorKernel.cu): C division, and the same
 * rounded towards minus infinity.  The floating forms are cases 38 / 39 of oracle_ew_scalar. */
ORACLE_API void oracle_div_int(const int64_t* a, const int64_t* b, int64_t n, int floor_mode, int64_t* out) {
  for (int64_t i = 0; i < n; ++i) {
    if (b[i] == 0) {
      out[i] = 0;
      continue;
    }
    int64_t q = a[i] / b[i];
    if (floor_mode && (a[i] % b[i] != 0) && ((a[i] < 0) != (b[i] < 0))) q -= 1;
    out[i] = q;
  }
}

/* Elementwise functors in double.  Codes follow the kernel library's sb_ew_op numbering.
 * add/mul: UfuncCUDA_add.cu:13-16 (self + alpha * other), BinaryInternal.h:16-29; the activations are
 * the formulas of the ATen kernels the reference links from its native-op library. */
static double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }
ORACLE_API double oracle_ew_scalar(int op, double a, double b, double c, double alpha) {
  const double kBeta = 0.79788456080286535588, kKappa = 0.044715;
  switch (op) {
    case 0: return a;
    case 2: return a + alpha * b;
    case 3: return a * b;
    case 4: return a - alpha * b;
    case 5: return a / b;
    case 6: return a * 0.5 * (1.0 + erf(a * 0.70710678118654752440));
    case 7: return 0.5 * a * (1.0 + tanh(kBeta * (a + kKappa * a * a * a)));
    case 8: return a * sigmoid_d(a);
    case 9: return a * sigmoid_d(b);
    case 10: {
      const double cdf = 0.5 * (1.0 + erf(b * 0.70710678118654752440));
      const double pdf = exp(-0.5 * b * b) * 0.39894228040143267794;
      return a * (cdf + b * pdf);
    }
    case 11: {
      const double inner = kBeta * (b + kKappa * b * b * b);
      const double th = tanh(inner);
      return a * (0.5 * (1.0 + th) + 0.5 * b * (1.0 - th * th) * kBeta * (1.0 + 3.0 * kKappa * b * b));
    }
    case 12: {
      const double s = sigmoid_d(b);
      return a * s * (1.0 + b * (1.0 - s));
    }
    case 13: return sigmoid_d(b) * a;
    case 14: {
      const double s = sigmoid_d(b);
      return (1.0 - s) * s * a * c;
    }
    case 17: return -a;
    /* 38 / 39: rounding modes of div, in the operands' own precision (fp32 here): 3.0f / 0.3f is exactly 10 in fp32 and
     * just below 10 in double, and the quotient is what gets truncated */
    case 38: return (double)truncf((float)a / (float)b);
    case 39: {  /* c10::div_floor_floating */
      const float fa = (float)a, fb = (float)b;
      if (fb == 0.f) return (double)(fa / fb);
      const float mod = fmodf(fa, fb);
      float div = (fa - mod) / fb;
      if (mod != 0.f && (fb < 0.f) != (mod < 0.f)) div -= 1.f;
      if (div != 0.f) {
        float fl = floorf(div);
        if (div - fl > 0.5f) fl += 1.f;
        return (double)fl;
      }
      return (double)copysignf(0.f, fa / fb);
    }
    default: return NAN;
  }
}
ORACLE_API void oracle_elementwise(int op, const double* a, const double* b, const double* c, double alpha, int64_t n,
                                   double* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_ew_scalar(op, a ? a[i] : 0.0, b ? b[i] : 0.0, c ? c[i] : 0.0, alpha);
}

// Cross entropy for rows shorter than 16 KB: the whole row sits in the registers of one warp (rows up to 2 KB) or of
// one 128-thread group (up to 16 KB), so every logit is read once and its gradient written once, as in the
// shared-memory pipeline of cross_entropy_tma.cu, whose per-row barriers and bulk copies would not pay for rows this
// short.  The reference keeps a family of small-class kernels for the same reason
// (torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:228-530).
//
// A row is fetched as the 16-byte aligned superset of its bytes with 16-byte loads (TPR threads x VPT vectors), so
// any class count and any element-aligned base address qualify; the elements of the first and last vector that
// belong to the neighbouring rows are masked in registers, and those two vectors are written back element by
// element so that a neighbour's bytes are never touched.  The superset stays inside the 16-byte granules that hold
// the row's own first and last byte, hence inside the same allocation.
//
// Arithmetic as in the resident kernel: base-2 online statistics with ex2.approx, fp32 accumulation, the class of the
// target patched from fp32; one named barrier per row and group (none for a warp).
#include "ce_common.cuh"

namespace sb {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kRowsRegThreads = 256;  // per CTA: 8 warps = 8 warp rows or 2 group rows at a time

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max_nan(float a, float b) {
  float d;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ void merge2(float& m, float& s, float om, float os) {
  const float nm = max_nan(m, om);
  const float a = (m == -CUDART_INF_F) ? 0.f : s * ex2f(m - nm);
  const float b = (om == -CUDART_INF_F) ? 0.f : os * ex2f(om - nm);
  m = nm;
  s = a + b;
}

// Element k of a 16-byte vector held in registers, without indexing the registers dynamically.
template <typename T>
__device__ __forceinline__ float extract_elem(const uint4& r, uint32_t k) {
  const uint32_t w = k * sizeof(T) / 4;
  const uint32_t word = w == 0 ? r.x : (w == 1 ? r.y : (w == 2 ? r.z : r.w));
  if constexpr (sizeof(T) == 4) {
    return __uint_as_float(word);
  } else {
    const unsigned short h = static_cast<unsigned short>((k & 1) ? (word >> 16) : (word & 0xffffu));
    T v;
    *reinterpret_cast<unsigned short*>(&v) = h;
    return to_float(v);
  }
}

// 16 bytes of T as fp32.
template <typename T> struct Lanes;
template <> struct Lanes<float> {
  static constexpr int E = 4;
  __device__ static __forceinline__ void unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
  __device__ static __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <> struct Lanes<__nv_bfloat16> {
  static constexpr int E = 8;
  __device__ static __forceinline__ void unpack(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Lanes<__half> {
  static constexpr int E = 8;
  __device__ static __forceinline__ void unpack(const uint4& r, float (&f)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  __device__ static __forceinline__ uint4 pack(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// TPR threads share a row: 8, 16 or 32 (part of a warp or a whole one; reductions by shuffles) or 128 (four warps, named
// barrier 1 + group index).
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(kRowsRegThreads, VPT <= 2 ? 4 : (VPT == 4 ? 3 : 2)) ce_rows_reg_kernel(CEParams p) {
  constexpr int E = Lanes<T>::E;
  constexpr int kGroupsPerCta = kRowsRegThreads / TPR;
  constexpr int kWarpsPerRow = TPR >= 32 ? TPR / 32 : 1;
  constexpr int kShuffleFrom = TPR >= 32 ? 16 : TPR / 2;
  __shared__ float s_part[2][TPR >= 32 ? kGroupsPerCta : 1][kWarpsPerRow][4];

  const int tid = threadIdx.x, lane = tid & 31;
  const int grp = tid / TPR, gt = tid % TPR, gw = gt >> 5;
  const int64_t group0 = static_cast<int64_t>(blockIdx.x) * kGroupsPerCta + grp;
  const int64_t group_stride = static_cast<int64_t>(gridDim.x) * kGroupsPerCta;
  const uint64_t row_bytes = static_cast<uint64_t>(p.classes) * sizeof(T);
  const uintptr_t in_base = reinterpret_cast<uintptr_t>(p.logits);
  const float eps = p.label_smoothing;
  const float eps_c = eps / static_cast<float>(p.classes);
  float base_scale = p.grad_scale;
  if (p.grad && p.reduction == SB_REDUCTION_MEAN) base_scale = static_cast<float>(static_cast<double>(base_scale) / p.acc[1]);
  unsigned par = 0;

  // Where a row lies: its aligned superset starts head_e elements before the row and spans `span` vectors.
  struct Geom {
    int64_t t;
    bool ignored;
    uint32_t head_b, head_e, span, tail_e;  // tail_e: elements of the last vector that are the row's; 0 = all
    const uint4* src;
  };
  auto geom_of = [&](int64_t row, int64_t t) -> Geom {
    Geom g;
    g.t = t;
    g.ignored = g.t == p.ignore_index || g.t < 0 || g.t >= p.classes;
    const uintptr_t a0 = in_base + static_cast<uint64_t>(row) * row_bytes;
    g.head_b = static_cast<uint32_t>(a0 & 15);
    g.head_e = g.head_b / sizeof(T);
    const uint64_t total = g.head_b + row_bytes;
    g.span = static_cast<uint32_t>((total + 15) >> 4);
    g.tail_e = static_cast<uint32_t>(total & 15) / sizeof(T);
    g.src = reinterpret_cast<const uint4*>(a0 - g.head_b);
    return g;
  };
  auto load_row = [&](const Geom& g, uint4 (&dst)[VPT]) {
    if (g.ignored) return;  // never read
#pragma unroll
    for (int q = 0; q < VPT; ++q) {
      const uint32_t v = q * TPR + gt;
      if (v < g.span) dst[q] = ld_stream_u4(g.src + v);
    }
  };

  // The loads of the next row are issued before the current one is worked on (two rows per group in flight), and targets
  // run two rows ahead: whether a row is loaded at all depends on its target, and that load must not wait for a target
  // that was asked for only then.
  uint4 r[VPT], nxt[VPT];
  Geom cur{}, ahead{};
  int64_t t_ahead = group0 + group_stride < p.rows ? p.target[group0 + group_stride] : 0;
  if (group0 < p.rows) {
    cur = geom_of(group0, p.target[group0]);
    load_row(cur, r);
  }
  for (int64_t row = group0;; row += group_stride) {
    // Rows that share a warp (TPR < 32) run out at different times: the warp goes on while any of them has a row, and a
    // group without one only takes part in the shuffles.
    const bool active = row < p.rows;
    if (TPR >= 32 ? !active : !__any_sync(0xffffffffu, active)) break;
    const bool has_next = row + group_stride < p.rows;
    if (has_next) {
      ahead = geom_of(row + group_stride, t_ahead);
      load_row(ahead, nxt);
      if (row + 2 * group_stride < p.rows) t_ahead = p.target[row + 2 * group_stride];
    }
    const int64_t t = cur.t;
    const bool ignored = cur.ignored || !active;
    if (active && cur.ignored && t != p.ignore_index && gt == 0 && p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    const uint32_t head_b = cur.head_b, head_e = cur.head_e, span = cur.span, tail_e = cur.tail_e;
    const uint32_t t_vec = ignored ? 0xffffffffu : (static_cast<uint32_t>(t) + head_e) / E;  // the target's vector and element in it
    const uint32_t t_el = ignored ? 0 : (static_cast<uint32_t>(t) + head_e) % E;
    // an edge vector holds elements of a neighbouring row: [lo, hi) are this row's
    auto edge_of = [&](uint32_t v, uint32_t& lo, uint32_t& hi) -> bool {
      lo = (v == 0) ? head_e : 0;
      hi = (v == span - 1 && tail_e) ? tail_e : E;
      return lo != 0 || hi != E;
    };

    float m2 = -CUDART_INF_F, s = 0.f, sx = 0.f, xt = 0.f;
    if (!ignored) {
      // pass 1 over the registers: maximum, sum of the logits, x[target]; foreign elements of edge vectors become -inf
      float vm = -CUDART_INF_F;
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        if (v < span) {
          float f[E];
          Lanes<T>::unpack(r[q], f);
          uint32_t lo, hi;
          if (edge_of(v, lo, hi)) {
#pragma unroll
            for (int k = 0; k < E; ++k) {
              if (static_cast<uint32_t>(k) < lo || static_cast<uint32_t>(k) >= hi) f[k] = -CUDART_INF_F;
              else sx += f[k];
            }
            r[q] = Lanes<T>::pack(f);
          } else {
#pragma unroll
            for (int k = 0; k < E; ++k) sx += f[k];
          }
#pragma unroll
          for (int k = 0; k < E; ++k) vm = max_nan(vm, f[k]);
          if (v == t_vec) {
#pragma unroll
            for (int k = 0; k < E; ++k)
              if (static_cast<uint32_t>(k) == t_el) xt = f[k];  // from registers: an in-place gradient may already overwrite the row
          }
        }
      }
      m2 = vm * kLog2e;
      const float mm = (m2 == -CUDART_INF_F) ? 0.f : m2;
      // pass 2: sum of exponentials relative to the thread's maximum (masked elements: 2^-inf = 0)
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        if (v < span) {
          float f[E];
          Lanes<T>::unpack(r[q], f);
#pragma unroll
          for (int k = 0; k < E; ++k) s += ex2f(fmaf(f[k], kLog2e, -mm));
        }
      }
#pragma unroll
      for (int o = kShuffleFrom; o > 0; o >>= 1) {
        merge2(m2, s, __shfl_xor_sync(0xffffffffu, m2, o), __shfl_xor_sync(0xffffffffu, s, o));
        sx += __shfl_xor_sync(0xffffffffu, sx, o);
        xt += __shfl_xor_sync(0xffffffffu, xt, o);  // one thread holds it, the others add 0
      }
    } else if (TPR < 32) {
      // part of a warp: the other rows of the warp run the shuffles above, every lane must take part
#pragma unroll
      for (int o = kShuffleFrom; o > 0; o >>= 1) {
        __shfl_xor_sync(0xffffffffu, m2, o);
        __shfl_xor_sync(0xffffffffu, s, o);
        __shfl_xor_sync(0xffffffffu, sx, o);
        __shfl_xor_sync(0xffffffffu, xt, o);
      }
    }
    if (kWarpsPerRow > 1) {
      // every thread of the group takes the same branch (`ignored` is a property of the row)
      if (lane == 0) {
        s_part[par][grp][gw][0] = m2;
        s_part[par][grp][gw][1] = s;
        s_part[par][grp][gw][2] = sx;
        s_part[par][grp][gw][3] = xt;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(TPR) : "memory");
      m2 = -CUDART_INF_F;
      s = 0.f;
      sx = 0.f;
      xt = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsPerRow; ++w) {
        merge2(m2, s, s_part[par][grp][w][0], s_part[par][grp][w][1]);
        sx += s_part[par][grp][w][2];
        xt += s_part[par][grp][w][3];
      }
      par ^= 1;  // the next row writes the other set; a set is rewritten two barriers after its last read
    }

    float lse = 0.f, scale = 0.f;
    if (!ignored) {
      lse = (m2 + log2f(s)) * kLn2;
      const float wt = p.class_weight ? p.class_weight[t] : 1.f;
      if (gt == 0) {
        p.row_loss[row] = ce_row_loss(lse, xt, sx, eps, eps_c) * wt;
        if (p.row_lse) p.row_lse[row] = lse;
      }
      scale = base_scale * wt;
      if (p.grad && p.row_grad_out) scale *= p.row_grad_out[row];
      if (lse != lse) scale = lse;
    } else if (gt == 0 && active) {
      p.row_loss[row] = 0.f;
      if (p.row_lse) p.row_lse[row] = 0.f;
    }

    if (p.grad && active) {
      const float sub_all = eps_c * scale;
      const float sub_t = (1.f - eps) * scale;
      const float neg_lse2 = -lse * kLog2e;
      T* grow = static_cast<T*>(p.grad) + row * p.classes;  // element 0 of the row
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uintptr_t>(grow) - head_b);
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        if (v < span) {
          uint4 o = make_uint4(0u, 0u, 0u, 0u);
          if (!ignored) {
            float f[E];
            Lanes<T>::unpack(r[q], f);
#pragma unroll
            for (int k = 0; k < E; ++k) f[k] = fmaf(ex2f(fmaf(f[k], kLog2e, neg_lse2)), scale, -sub_all);
            if (v == t_vec) {
#pragma unroll
              for (int k = 0; k < E; ++k)
                if (static_cast<uint32_t>(k) == t_el) f[k] -= sub_t;
            }
            o = Lanes<T>::pack(f);
          }
          uint32_t lo, hi;
          if (!edge_of(v, lo, hi)) {
            st_stream_u4(dst + v, o);
          } else {  // an edge vector: only this row's elements are written
            const T* oe = reinterpret_cast<const T*>(&o);
            T* de = reinterpret_cast<T*>(dst + v);
#pragma unroll
            for (int k = 0; k < E; ++k)
              if (static_cast<uint32_t>(k) >= lo && static_cast<uint32_t>(k) < hi) de[k] = oe[k];
          }
        }
      }
    }
    if (has_next) {
      cur = ahead;
#pragma unroll
      for (int q = 0; q < VPT; ++q) r[q] = nxt[q];
    }
  }
}

template <typename T, int TPR, int VPT>
int launch_rows_reg_cfg(const CEParams& p, cudaStream_t st) {
  constexpr int kGroupsPerCta = kRowsRegThreads / TPR;
  const int64_t want = (p.rows + kGroupsPerCta - 1) / kGroupsPerCta;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;  // a few CTAs of 256 threads per SM, each group walking many rows
  ce_rows_reg_kernel<T, TPR, VPT><<<static_cast<int>(want < cap ? want : cap), kRowsRegThreads, 0, st>>>(p);
  return launch_status();
}

// Vectors of the widest aligned superset of a row: exactly row_bytes / 16 when the pitch and the base are multiples of 16
// bytes, one more when a row may start inside a vector.
uint64_t superset_units(int dtype, int64_t classes, const void* logits) {
  const uint64_t es = static_cast<uint64_t>(dtype_size(dtype));
  const uint64_t row_bytes = static_cast<uint64_t>(classes) * es;
  if (row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(logits) % 16 == 0) return row_bytes / 16;
  return (row_bytes + (16 - es) + 15) / 16;
}

template <typename T>
int launch_rows_reg(const CEParams& p, cudaStream_t st) {
  const uint64_t units = superset_units(p.dtype, p.classes, p.logits);
  if (units <= 8) return launch_rows_reg_cfg<T, 8, 1>(p, st);
  if (units <= 16) return launch_rows_reg_cfg<T, 16, 1>(p, st);
  if (units <= 32) return launch_rows_reg_cfg<T, 32, 1>(p, st);
  if (units <= 64) return launch_rows_reg_cfg<T, 32, 2>(p, st);
  if (units <= 128) return launch_rows_reg_cfg<T, 32, 4>(p, st);
  if (units <= 256) return launch_rows_reg_cfg<T, 128, 2>(p, st);
  if (units <= 512) return launch_rows_reg_cfg<T, 128, 4>(p, st);
  if (units <= 1024) return launch_rows_reg_cfg<T, 128, 8>(p, st);
  return SB_ERR_INVALID_ARGUMENT;
}

}  // namespace

bool rows_reg_applies(int dtype, int64_t classes, const void* logits, const void* grad) {
  const uint64_t es = static_cast<uint64_t>(dtype_size(dtype));
  if (es == 0 || classes <= 0) return false;
  if (superset_units(dtype, classes, logits) > 1024) return false;
  const uintptr_t a = reinterpret_cast<uintptr_t>(logits), b = reinterpret_cast<uintptr_t>(grad);
  if (a % es) return false;
  // the gradient is stored at the input's position within a 16-byte vector
  return grad == nullptr || (b % 16) == (a % 16);
}

int ce_launch_rows_reg(const CEParams& p, cudaStream_t st) {
  switch (p.dtype) {
    case SB_F32: return launch_rows_reg<float>(p, st);
    case SB_BF16: return launch_rows_reg<__nv_bfloat16>(p, st);
    case SB_F16: return launch_rows_reg<__half>(p, st);
    default: return SB_ERR_UNSUPPORTED;
  }
}

}  // namespace sb

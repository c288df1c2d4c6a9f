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
constexpr int kRowsRegThreads = 512;  // per CTA: 16 warps = 16 warp rows or 4 group rows at a time

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

// TPR threads share a row: 32 (a warp) or 128 (four warps, named barrier 1 + group index).
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(kRowsRegThreads) ce_rows_reg_kernel(CEParams p) {
  constexpr int E = 16 / sizeof(T);
  constexpr int kGroupsPerCta = kRowsRegThreads / TPR;
  constexpr int kWarpsPerRow = TPR / 32;
  __shared__ float s_part[2][kGroupsPerCta][kWarpsPerRow][4];

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
  auto geom_of = [&](int64_t row) -> Geom {
    Geom g;
    g.t = p.target[row];
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

  // The loads of the next row are issued before the current one is worked on: two rows per group in flight.
  uint4 r[VPT], nxt[VPT];
  Geom cur{}, ahead{};
  if (group0 < p.rows) {
    cur = geom_of(group0);
    load_row(cur, r);
  }
  for (int64_t row = group0; row < p.rows; row += group_stride) {
    const bool has_next = row + group_stride < p.rows;
    if (has_next) {
      ahead = geom_of(row + group_stride);
      load_row(ahead, nxt);
    }
    const int64_t t = cur.t;
    const bool ignored = cur.ignored;
    if (ignored && t != p.ignore_index && gt == 0 && p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    const uint32_t head_b = cur.head_b, head_e = cur.head_e, span = cur.span, tail_e = cur.tail_e;

    float m2 = -CUDART_INF_F, s = 0.f, sx = 0.f, xt = 0.f;
    if (!ignored) {
      const uint32_t t_pos = static_cast<uint32_t>(t) + head_e;  // the target's element in the superset
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        // taken from registers: an in-place gradient may already be overwriting the row in memory
        if (v < span && v == t_pos / E) xt = extract_elem<T>(r[q], t_pos % E);
      }
      // thread maximum over its own elements (foreign elements of the edge vectors masked to -inf in place)
      float vm = -CUDART_INF_F;
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        if (v < span) {
          T* e = reinterpret_cast<T*>(&r[q]);
          const uint32_t lo = v == 0 ? head_e : 0;
          const uint32_t hi = (v == span - 1 && tail_e) ? tail_e : E;
#pragma unroll
          for (int k = 0; k < E; ++k) {
            const bool mine = static_cast<uint32_t>(k) >= lo && static_cast<uint32_t>(k) < hi;
            const float f = to_float(e[k]);
            if (mine) {
              vm = max_nan(vm, f);
              sx += f;
            } else {
              e[k] = from_float<T>(-CUDART_INF_F);
            }
          }
        }
      }
      m2 = vm * kLog2e;
      const float mm = (m2 == -CUDART_INF_F) ? 0.f : m2;
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        const uint32_t v = q * TPR + gt;
        if (v < span) {
          const T* e = reinterpret_cast<const T*>(&r[q]);
#pragma unroll
          for (int k = 0; k < E; ++k) s += ex2f(fmaf(to_float(e[k]), kLog2e, -mm));  // masked elements: 2^-inf = 0
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        merge2(m2, s, __shfl_xor_sync(0xffffffffu, m2, o), __shfl_xor_sync(0xffffffffu, s, o));
        sx += __shfl_xor_sync(0xffffffffu, sx, o);
        xt += __shfl_xor_sync(0xffffffffu, xt, o);  // one thread holds it, the others add 0
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
    } else if (gt == 0) {
      p.row_loss[row] = 0.f;
      if (p.row_lse) p.row_lse[row] = 0.f;
    }

    if (p.grad) {
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
            const T* e = reinterpret_cast<const T*>(&r[q]);
            T* oe = reinterpret_cast<T*>(&o);
            const int64_t c0 = static_cast<int64_t>(v) * E - head_e;  // class of element 0 of this vector
#pragma unroll
            for (int k = 0; k < E; ++k) {
              float g = fmaf(ex2f(fmaf(to_float(e[k]), kLog2e, neg_lse2)), scale, -sub_all);
              if (c0 + k == t) g -= sub_t;
              oe[k] = from_float<T>(g);
            }
          }
          const uint32_t lo = v == 0 ? head_e : 0;
          const uint32_t hi = (v == span - 1 && tail_e) ? tail_e : E;
          if (lo == 0 && hi == E) {
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
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;  // up to 4 CTAs of 512 threads per SM
  ce_rows_reg_kernel<T, TPR, VPT><<<static_cast<int>(want < cap ? want : cap), kRowsRegThreads, 0, st>>>(p);
  return launch_status();
}

// Vectors of the widest aligned superset of a row.
uint64_t superset_units(int dtype, int64_t classes) {
  const uint64_t es = static_cast<uint64_t>(dtype_size(dtype));
  return (static_cast<uint64_t>(classes) * es + (16 - es) + 15) / 16;
}

template <typename T>
int launch_rows_reg(const CEParams& p, cudaStream_t st) {
  const uint64_t units = superset_units(p.dtype, p.classes);
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
  if (superset_units(dtype, classes) > 1024) return false;
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

// Cross entropy for rows of 256 B to 32 KB with a 16-byte aligned pitch: groups of whole rows travel through a ring of
// shared-memory slots, one warp (or 16, 8 or 4 lanes of one, or a team of four warps) per row.
//
// A persistent CTA (one per SM) owns every gridDim.x-th group of R consecutive rows (R rows = about 8 KB: bulk copies of
// a kilobyte or two each cost the copy engine about as much as one of 8 KB, and a row-sized copy per row held these
// shapes at a fixed ~290 ns per row).  Three kinds of warps:
//   * the loader issues one bulk copy (cp.async.bulk global -> shared, completion on the group's mbarrier) per group into
//     the next free slot;
//   * consumer warp w of W takes rows w, w + W, ... of the CTA's sequence.  With the row in shared memory the three passes
//     cost no HBM traffic:
//       pass 0  row maximum (packed maxima for 16-bit logits)
//       pass 1  sum of 2^(x log2e - max2), sum of x (label smoothing); 16-bit logits: the exponentials overwrite the row
//       pass 2  gradient in place: kept exponential * (scale / sum) - eps/C (bf16: one packed FMA per pair), or
//               recomputed from the logits for fp32; the target's class is patched from fp32 arithmetic on the saved
//               x[target]; a row whose target is ignored is overwritten with zeros
//     and arrives on the group's `done` mbarrier;
//   * the storer waits for a group's rows to be done, issues one bulk store (shared -> global) for the group and hands the
//     slot back to the loader when the store has finished reading it (two stores may be in flight).
// One HBM read and one HBM write per logit; the loads of later groups run under the arithmetic of earlier ones without
// occupying registers.  Rows with an ignored target are read with their group.
//
// Every mbarrier wait is bounded; a wait that runs out sets SB_STATUS_KERNEL_TIMEOUT and the warp leaves its loop.
#include "ce_ring.cuh"

namespace sb {

using namespace ring;

namespace {

constexpr int kRingWarps = 16;                         // consumer warps in the CTA (the launch may use fewer: RingParams::nwarps)
constexpr int kRingThreads = (kRingWarps + 2) * 32;    // plus the loader warp and the storer warp
constexpr int kRingMaxSlots = 32;
constexpr uint32_t kRingMinRowBytes = 256;
constexpr uint32_t kRingMaxRowBytes = 32768;            // up to and including
constexpr uint32_t kRingGroupBytes = 8192;             // rows are grouped up to about this size per bulk copy
int g_ring_warps = 0;  // tuning: consumer warps per CTA (0 = automatic)
int g_ring_max_bytes = static_cast<int>(kRingMaxRowBytes);  // tuning: longest row the ring takes

struct RingParams {
  CEParams p;
  uint32_t row_bytes;
  uint32_t units;        // 16-byte units per row
  uint32_t group_rows;   // R: consecutive rows per group (one bulk copy in, one out)
  uint32_t nslots;       // group slots in the ring
  uint32_t nwarps;       // consumer warps that take rows
  int64_t ngroups;       // ceil(rows / R)
};

struct alignas(16) RingTail {
  unsigned long long full[kRingMaxSlots];   // loader -> consumers: the group has landed
  unsigned long long done[kRingMaxSlots];   // consumers -> storer: R arrivals, the group holds its gradients
  unsigned long long empty[kRingMaxSlots];  // storer -> loader: the group's store has finished reading the slot
  // Lap of the ring whose load has been issued into the slot, written by the loader.  A consumer waits on `full` by phase
  // parity, and different warps take different laps of a slot: a warp that came a whole lap early would see the parity of
  // the lap before last and walk through.  It therefore first waits until the slot's lap number is its own; from then on
  // the barrier is in that lap's phase or just past it, and the parity is unambiguous.
  volatile uint32_t lapno[kRingMaxSlots];
  volatile uint32_t abort;  // set by the first wait that runs out: every other wait of the CTA gives up too
  float team[kRingWarps][3][4];  // [team][maximum, sum of exponentials, sum of logits][warp of the team]
  volatile uint32_t team_failed[kRingWarps];
};

constexpr uint32_t kRingMaxPolls = 1u << 20;  // try_wait attempts before a wait gives up (a legitimate wait lasts microseconds)

// Bounded wait on an mbarrier phase that also ends when another warp of the CTA has given up.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort) {
  for (uint32_t i = 0; i < kRingMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 15u) == 15u && *abort) return false;
  }
  return false;
}
// Bounded wait until the slot's lap number is `lap`.
__device__ __forceinline__ bool ring_wait_lap(volatile uint32_t* lapno, uint32_t lap, volatile uint32_t* abort) {
  for (uint32_t i = 0; i < (kRingMaxPolls << 4); ++i) {
    if (*lapno == lap) return true;
    if ((i & 63u) == 63u) {
      if (*abort) return false;
      __nanosleep(64);
    }
  }
  return false;
}

// NaN-propagating maximum over the warp in one instruction (redux.sync on f32: sm_100a).
__device__ __forceinline__ float warp_max_nan(float v) {
  float r;
  asm volatile("redux.sync.max.NaN.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// NIT > 0: a lane holds its NIT units of the row in registers between the passes (rows of up to 32 * NIT units): one
// shared-memory read and one write per unit, exponentials kept for every dtype.  NIT = 0: longer rows, three passes over
// shared memory.
// LPR: lanes per row.  32 = one row per warp; 16 / 8 / 4 = two / four / eight rows per warp side by side (rows of up to
// 1 KB / 512 B / 256 B, where the fixed cost per row, about 250 instructions, outweighs the arithmetic on the logits): each
// group of LPR lanes is a consumer of its own with its own place in the CTA's row sequence, and every warp-level primitive
// is confined to the group.
// TW: warps per row.  Rows of more than 16 KB are swept by a team of TW warps (three passes over shared memory, the two
// reductions finished through a few floats of shared memory and a named barrier per team): a single warp would hold a slot
// for too long, and rows of this length leave only a handful of slots.
// MODE 0: cross entropy (losses and gradient).  MODE 1: log_softmax (x - lse out; no targets, no losses).  MODE 2: softmax
// (the gradient formula with scale 1, nothing subtracted and no target).  In modes 1 and 2 `grad` is the output.
template <typename T, bool kSumX, int NIT, int LPR, int TW, int MODE>
__global__ void __launch_bounds__(kRingThreads, 1) ce_ring_rows_kernel(RingParams rp) {
  static_assert(MODE == 0 || !kSumX, "only the cross entropy needs the sum of the logits");
  static_assert(LPR == 32 || ((LPR == 16 || LPR == 8 || LPR == 4) && NIT > 0), "rows that share a warp stay in registers");
  static_assert(TW == 1 || (NIT == 0 && LPR == 32 && kRingWarps % TW == 0), "teams of warps sweep shared memory");
  using U = Unit<T>;
  constexpr int P = U::kPairs;
  constexpr int E = 16 / static_cast<int>(sizeof(T));
  constexpr bool kKeep = sizeof(T) == 2 && MODE != 1;  // 16-bit logits: one ex2 per logit, the gradient pass rescales
                                                        // (log_softmax needs the logits themselves in its last pass)
  extern __shared__ __align__(128) unsigned char smem[];
  const CEParams& p = rp.p;
  const uint32_t nslots = rp.nslots, units = rp.units, row_bytes = rp.row_bytes, nwarps = rp.nwarps, R = rp.group_rows;
  const uint32_t slot_bytes = R * row_bytes;
  RingTail* tail = reinterpret_cast<RingTail*>(smem + static_cast<size_t>(nslots) * slot_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this CTA's groups: first, first + stride, ...
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int64_t n_local = first < rp.ngroups ? (rp.ngroups - first + stride - 1) / stride : 0;

  grid_dep_launch();
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < nslots; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 1);
      mbar_init(smem_u32(&tail->done[s]), R * TW);  // one arrival per warp that worked on a row of the group
      mbar_init(smem_u32(&tail->empty[s]), 1);
      tail->lapno[s] = 0;
    }
    tail->abort = 0;
    for (int w = 0; w < kRingWarps; ++w) tail->team_failed[w] = 0;
    fence_mbar_init();
  }
  __syncthreads();

  auto give_up = [&]() {
    tail->abort = 1;
    if ((lane & (LPR - 1)) == 0 && p.status) atomicOr(p.status, SB_STATUS_KERNEL_TIMEOUT);
  };
  auto rows_in_group = [&](int64_t group) {
    const int64_t left = p.rows - group * R;
    return static_cast<uint32_t>(left < static_cast<int64_t>(R) ? left : R);
  };

  if (warp == kRingWarps) {
    // ---- loader ------------------------------------------------------------------------------------------------------
    const char* logits = static_cast<const char*>(p.logits);
    uint32_t slot = 0, lap = 0;
    for (int64_t k = 0; k < n_local; ++k) {
      if (lap > 0 && !ring_wait(smem_u32(&tail->empty[slot]), (lap - 1) & 1, &tail->abort)) {
        give_up();
        break;
      }
      if (lane == 0) {
        const int64_t group = first + k * stride;
        const uint32_t bytes = rows_in_group(group) * row_bytes;
        const uint32_t bar = smem_u32(&tail->full[slot]);
        tail->lapno[slot] = lap;  // the previous lap of this slot is over (its store has been read): consumers of this lap may wait
        mbar_expect_tx(bar, bytes);
        bulk_g2s(smem_u32(smem + static_cast<size_t>(slot) * slot_bytes), logits + group * static_cast<int64_t>(slot_bytes), bytes, bar);
      }
      if (++slot == nslots) {
        slot = 0;
        ++lap;
      }
    }
    return;
  }

  if (warp == kRingWarps + 1) {
    // ---- storer ------------------------------------------------------------------------------------------------------
    char* grad = static_cast<char*>(p.grad);
    uint32_t slot = 0, lap = 0;
    int held[2] = {-1, -1};  // slots of the two most recent stores, oldest first
    for (int64_t k = 0; k < n_local; ++k) {
      if (!ring_wait(smem_u32(&tail->done[slot]), lap & 1, &tail->abort)) {
        give_up();
        break;
      }
      if (lane == 0) {
        if (grad) {
          const int64_t group = first + k * stride;
          bulk_s2g(grad + group * static_cast<int64_t>(slot_bytes), smem_u32(smem + static_cast<size_t>(slot) * slot_bytes),
                   rows_in_group(group) * row_bytes);
          bulk_commit();
          if (held[0] >= 0) {
            bulk_wait_read<2>();  // all but the two most recent stores have finished reading shared memory
            mbar_arrive(smem_u32(&tail->empty[held[0]]));
          }
          held[0] = held[1];
          held[1] = static_cast<int>(slot);
        } else {
          mbar_arrive(smem_u32(&tail->empty[slot]));
        }
      }
      if (++slot == nslots) {
        slot = 0;
        ++lap;
      }
    }
    if (lane == 0 && grad) {
      bulk_wait_all();
      if (held[0] >= 0) mbar_arrive(smem_u32(&tail->empty[held[0]]));
      if (held[1] >= 0) mbar_arrive(smem_u32(&tail->empty[held[1]]));
    }
    return;
  }

  // ---- consumers -------------------------------------------------------------------------------------------------------
  if (static_cast<uint32_t>(warp) >= nwarps) return;
  constexpr uint32_t kSubs = 32 / LPR;                        // consumers per warp
  const uint32_t sub = static_cast<uint32_t>(lane) / LPR;     // which of them this lane belongs to
  const uint32_t sl = static_cast<uint32_t>(lane) % LPR;      // lane within the consumer
  const uint32_t gmask = LPR == 32 ? 0xffffffffu : (((1u << (LPR & 31)) - 1u) << (LPR * sub));
  const uint32_t team = static_cast<uint32_t>(warp) / TW, tw_rank = static_cast<uint32_t>(warp) % TW;
  const uint32_t me = team * kSubs + sub, consumers = (nwarps / TW) * kSubs;
  // position and stride of this lane in the sweeps over a row in shared memory
  const uint32_t lane_pos = TW > 1 ? tw_rank * 32 + static_cast<uint32_t>(lane) : sl;
  const uint32_t lane_step = TW > 1 ? 32 * TW : LPR;
  const bool leader = sl == 0 && tw_rank == 0;  // writes the row's loss
  auto valid_target = [&](int64_t t) { return t != p.ignore_index && t >= 0 && t < p.classes; };
  const float eps = p.label_smoothing;
  const float eps_c = eps / static_cast<float>(p.classes);
  float base_scale = p.grad_scale;
  if (p.grad && p.reduction == SB_REDUCTION_MEAN) {
    grid_dep_wait();  // the valid-row count comes from the launch before this one
    base_scale = static_cast<float>(static_cast<double>(p.grad_scale) / p.acc[1]);
  }
  const float2 l2e2 = make_float2(kLog2e, kLog2e);
  // Sequence number i = k * R + j: row j of the CTA's k-th group.  (k, j) advance by the number of consumers per step without
  // a division.
  uint32_t j = me % R;
  int64_t k = me / R;
  const uint32_t step_j = consumers % R, step_k = consumers / R;
  uint32_t slot = static_cast<uint32_t>(k) % nslots, lap = static_cast<uint32_t>(k) / nslots;
  auto row_of = [&](int64_t kk, uint32_t jj) { return (first + kk * stride) * R + jj; };
  auto load_target = [&](int64_t kk, uint32_t jj) -> int64_t {
    if constexpr (MODE != 0) return 0;
    const int64_t r = row_of(kk, jj);
    return (kk < n_local && r < p.rows) ? p.target[r] : p.ignore_index;
  };
  // Targets are fetched one step ahead and must not be looked at before the step that uses them: a use in the step that
  // issued the load would stall the warp for a full trip to HBM per row.
  int64_t t_next = load_target(k, j);
  for (; k < n_local;) {
    const int64_t row = row_of(k, j);
    const int64_t t = t_next;
    // the next step of this warp
    uint32_t nj = j + step_j;
    int64_t nk = k + step_k;
    if (nj >= R) {
      nj -= R;
      ++nk;
    }
    t_next = load_target(nk, nj);

    bool landed = (lap == 0 || ring_wait_lap(&tail->lapno[slot], lap, &tail->abort)) && ring_wait(smem_u32(&tail->full[slot]), lap & 1, &tail->abort);
    if constexpr (TW > 1) {
      // the warps of a team meet at named barriers while they work on a row: they go on, or give up, together
      if (!landed) tail->team_failed[team] = 1;
      named_barrier(1 + team, 32 * TW);
      landed = tail->team_failed[team] == 0;
    }
    if (!landed) {
      give_up();
      break;
    }
    if (row < p.rows) {  // the last group may have fewer than R rows: the missing ones only arrive
      const bool ignored = MODE == 0 && !valid_target(t);
      if (ignored && t != p.ignore_index && leader && p.status) atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
      float wt = 1.f;
      if (p.class_weight && !ignored) wt = p.class_weight[t];
      uint4* buf = reinterpret_cast<uint4*>(smem + static_cast<size_t>(slot) * slot_bytes + static_cast<size_t>(j) * row_bytes);
      if (ignored) {
        if (leader) {
          p.row_loss[row] = 0.f;
          if (p.row_lse) p.row_lse[row] = 0.f;
        }
        if (p.grad) {
          for (uint32_t v = lane_pos; v < units; v += lane_step) buf[v] = make_uint4(0u, 0u, 0u, 0u);
        }
      } else {
        if constexpr (NIT > 0) {
          // ---- the row in registers -------------------------------------------------------------------------------------
          uint4 r[NIT];
          float vm = -CUDART_INF_F;
#pragma unroll
          for (int n = 0; n < NIT; ++n) {
            const uint32_t v = sl + LPR * n;
            if (v < units) {
              r[n] = buf[v];
              vm = max_nan(vm, U::vmax(r[n]));
            }
          }
          // x[target] is read before any lane stores a gradient (the warp-wide reductions below lie in between)
          const float xt = MODE == 0 ? to_float(reinterpret_cast<const T*>(buf)[t]) : 0.f;
          if constexpr (LPR == 32) {
            vm = warp_max_nan(vm);
          } else {
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) vm = max_nan(vm, __shfl_xor_sync(gmask, vm, o));
          }
          const float m2 = vm * kLog2e;
          const float mm = (m2 == -CUDART_INF_F) ? 0.f : m2;
          const float2 negm = make_float2(-mm, -mm);
          float2 s2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          float2 sx2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
          for (int n = 0; n < NIT; ++n) {
            if (sl + LPR * n < units) {
              float2 f[P];
              U::unpack(r[n], f);
#pragma unroll
              for (int q = 0; q < P; ++q) {
                const float2 y = fma2(f[q], l2e2, negm);
                const float2 ex = make_float2(ex2(y.x), ex2(y.y));
                s2[q & 1] = add2(s2[q & 1], ex);
                if (kSumX) sx2[q & 1] = add2(sx2[q & 1], f[q]);
                f[q] = ex;
              }
              if (MODE != 1) r[n] = U::pack(f);  // the exponentials replace the logits (fp32: the same registers)
            }
          }
          float s = (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
          float sx = (sx2[0].x + sx2[0].y) + (sx2[1].x + sx2[1].y);
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) {
            s += __shfl_xor_sync(gmask, s, o);
            if (kSumX) sx += __shfl_xor_sync(gmask, sx, o);
          }
          const float lse2 = m2 + log2f(s);
          const float lse = lse2 * kLn2;
          if (MODE == 0 && sl == 0) {
            p.row_loss[row] = ce_row_loss(lse, xt, sx, eps, eps_c) * wt;
            if (p.row_lse) p.row_lse[row] = lse;
          }
          if (p.grad) {
            float scale = MODE == 0 ? base_scale * wt : 1.f;
            if (MODE == 0 && p.row_grad_out) scale *= p.row_grad_out[row];
            if (lse != lse) scale = lse;  // a NaN row has a NaN gradient
            const float sub_all = MODE == 0 ? eps_c * scale : 0.f;
            const float sub_t = (1.f - eps) * scale;
            const float g_t = fmaf(ex2(fmaf(xt, kLog2e, -lse2)), scale, -sub_all) - sub_t;
            const uint32_t t_vec = static_cast<uint32_t>(t) / E;
            const float factor = scale / s;  // kept value * factor = softmax * scale
            const float2 f2 = make_float2(factor, factor), n2 = make_float2(-sub_all, -sub_all);
#pragma unroll
            for (int n = 0; n < NIT; ++n) {
              const uint32_t v = sl + LPR * n;
              if (v < units) {
                uint4 o;
                if constexpr (MODE == 1) {
                  o = shift_vector<T>(r[n], make_float2(-lse, -lse));
                } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                  o = grad_from_kept_bf16(r[n], __float2bfloat162_rn(factor), __float2bfloat162_rn(-sub_all));
                } else {
                  o = grad_from_kept<T>(r[n], f2, n2);
                }
                buf[v] = o;
              }
            }
            // the target's class, by the lane that has just stored its unit
            if (MODE == 0 && sl == t_vec % LPR) reinterpret_cast<T*>(buf)[t] = from_float<T>(g_t);
          }
        } else {
          // pass 0: the row maximum
          float vm = -CUDART_INF_F;
#pragma unroll 4
          for (uint32_t v = lane_pos; v < units; v += lane_step) vm = max_nan(vm, U::vmax(buf[v]));
          // x[target]: before the reduction, whose synchronisation orders this read before the owner's write in pass 1
          const float xt = MODE == 0 ? to_float(reinterpret_cast<const T*>(buf)[t]) : 0.f;
          vm = warp_max_nan(vm);
          if constexpr (TW > 1) {
            if (lane == 0) tail->team[team][0][tw_rank] = vm;
            named_barrier(1 + team, 32 * TW);
            vm = tail->team[team][0][0];
#pragma unroll
            for (int w = 1; w < TW; ++w) vm = max_nan(vm, tail->team[team][0][w]);
          }
          const float m2 = vm * kLog2e;
          const float mm = (m2 == -CUDART_INF_F) ? 0.f : m2;  // a row of -inf: keep (-inf) - (-inf) out of the arithmetic
          if (kKeep) __syncwarp();  // every lane has read x[target] before its owner overwrites it
          // pass 1: sum of exponentials relative to the row maximum, sum of logits
          const float2 negm = make_float2(-mm, -mm);
          float2 s2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          float2 sx2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll 4
          for (uint32_t v = lane_pos; v < units; v += lane_step) {
            float2 f[P];
            U::unpack(buf[v], f);
#pragma unroll
            for (int q = 0; q < P; ++q) {
              const float2 y = fma2(f[q], l2e2, negm);
              const float2 e = make_float2(ex2(y.x), ex2(y.y));
              s2[q & 1] = add2(s2[q & 1], e);
              if (kSumX) sx2[q & 1] = add2(sx2[q & 1], f[q]);
              if (kKeep) f[q] = e;
            }
            if (kKeep) buf[v] = U::pack(f);
          }
          float s = (s2[0].x + s2[0].y) + (s2[1].x + s2[1].y);
          float sx = (sx2[0].x + sx2[0].y) + (sx2[1].x + sx2[1].y);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, o);
            if (kSumX) sx += __shfl_xor_sync(0xffffffffu, sx, o);
          }
          if constexpr (TW > 1) {
            if (lane == 0) {
              tail->team[team][1][tw_rank] = s;
              tail->team[team][2][tw_rank] = sx;
            }
            named_barrier(1 + team, 32 * TW);
            s = tail->team[team][1][0];
            sx = tail->team[team][2][0];
#pragma unroll
            for (int w = 1; w < TW; ++w) {  // the same order in every warp: all of them get the same bits
              s += tail->team[team][1][w];
              sx += tail->team[team][2][w];
            }
          }
          const float lse2 = m2 + log2f(s);
          const float lse = lse2 * kLn2;
          if (MODE == 0 && leader) {
            p.row_loss[row] = ce_row_loss(lse, xt, sx, eps, eps_c) * wt;
            if (p.row_lse) p.row_lse[row] = lse;
          }
          if (p.grad) {
            float scale = MODE == 0 ? base_scale * wt : 1.f;
            if (MODE == 0 && p.row_grad_out) scale *= p.row_grad_out[row];
            if (lse != lse) scale = lse;  // a NaN row has a NaN gradient
            const float sub_all = MODE == 0 ? eps_c * scale : 0.f;
            const float sub_t = (1.f - eps) * scale;
            // gradient of the target's class from fp32 arithmetic on the saved logit
            const float g_t = fmaf(ex2(fmaf(xt, kLog2e, -lse2)), scale, -sub_all) - sub_t;
            const uint32_t t_vec = MODE == 0 ? static_cast<uint32_t>(t) / E : 0xffffffffu, t_el = static_cast<uint32_t>(t) % E;
            auto patch = [&](uint4 o) {
              T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
              for (int q = 0; q < E; ++q)
                if (static_cast<uint32_t>(q) == t_el) oe[q] = from_float<T>(g_t);
              return o;
            };
            if constexpr (MODE == 1) {
              const float2 nl = make_float2(-lse, -lse);
#pragma unroll 4
              for (uint32_t v = lane_pos; v < units; v += lane_step) buf[v] = shift_vector<T>(buf[v], nl);
            } else if (kKeep) {
              const float factor = scale / s;  // kept value * factor = softmax * scale
              if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                const __nv_bfloat162 f2 = __float2bfloat162_rn(factor), n2 = __float2bfloat162_rn(-sub_all);
#pragma unroll 4
                for (uint32_t v = lane_pos; v < units; v += lane_step) {
                  uint4 o = grad_from_kept_bf16(buf[v], f2, n2);
                  if (v == t_vec) o = patch(o);
                  buf[v] = o;
                }
              } else {
                const float2 f2 = make_float2(factor, factor), n2 = make_float2(-sub_all, -sub_all);
#pragma unroll 4
                for (uint32_t v = lane_pos; v < units; v += lane_step) {
                  uint4 o = grad_from_kept<T>(buf[v], f2, n2);
                  if (v == t_vec) o = patch(o);
                  buf[v] = o;
                }
              }
            } else {
              const float2 nl2 = make_float2(-lse2, -lse2), sc2 = make_float2(scale, scale), n2 = make_float2(-sub_all, -sub_all);
#pragma unroll 4
              for (uint32_t v = lane_pos; v < units; v += lane_step) {
                uint4 o = grad_vector<T>(buf[v], nl2, sc2, n2);
                if (v == t_vec) o = patch(o);
                buf[v] = o;
              }
            }
          }
        }
      }
      if (p.grad) fence_proxy_async();  // this lane's writes to the slot, before the bulk store reads them
    }
    __syncwarp(gmask);
    if (sl == 0) mbar_arrive(smem_u32(&tail->done[slot]));
    slot += static_cast<uint32_t>(nk - k);
    while (slot >= nslots) {
      slot -= nslots;
      ++lap;
    }
    j = nj;
    k = nk;
  }
}

size_t ring_smem_limit() {
  static size_t limit = 0;
  if (limit == 0) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || v <= 0) v = 227 * 1024;
    limit = static_cast<size_t>(v);
  }
  return limit;
}

template <typename T, bool SUMX, int NIT, int LPR, int TW, int MODE>
int launch_ring_cfg(const RingParams& rp, size_t smem, int grid, cudaStream_t st, bool pdl) {
  auto kernel = ce_ring_rows_kernel<T, SUMX, NIT, LPR, TW, MODE>;
  static bool configured = false;  // per instantiation; the attribute is per device, set again after a device change is harmless
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring_smem_limit())) != cudaSuccess) {
      cudaGetLastError();
      return SB_ERR_CUDA;
    }
    configured = true;
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kRingThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, rp) != cudaSuccess) {
    cudaGetLastError();
    return SB_ERR_CUDA;
  }
  return SB_OK;
}

// The instantiation for the row length: lanes per row, units per lane in registers, warps per row.
template <typename T, bool SUMX, int MODE>
int launch_ring_shape(const RingParams& rp, size_t smem, int grid, cudaStream_t st, bool pdl) {
  const uint32_t u = rp.units;
  // Rows of up to 256 B / 512 B / 1 KB: eight / four / two rows per warp (bf16 [131072,512]: 0.71 of the copy peak against 0.54
  // with a warp per row; for rows of 2 KB the same split measured slower, 0.75 against 0.82).  Longer ones: one row per warp,
  // in registers up to 8 KB, in shared memory up to 16 KB; beyond that a team of four warps per row.
  if (u <= 16) return launch_ring_cfg<T, SUMX, 4, 4, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 32) return launch_ring_cfg<T, SUMX, 4, 8, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 64) return launch_ring_cfg<T, SUMX, 4, 16, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 128) return launch_ring_cfg<T, SUMX, 4, 32, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 256) return launch_ring_cfg<T, SUMX, 8, 32, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 512) return launch_ring_cfg<T, SUMX, 16, 32, 1, MODE>(rp, smem, grid, st, pdl);
  if (u <= 1024) return launch_ring_cfg<T, SUMX, 0, 32, 1, MODE>(rp, smem, grid, st, pdl);
  return launch_ring_cfg<T, SUMX, 0, 32, 4, MODE>(rp, smem, grid, st, pdl);
}

template <typename T>
int launch_ring_t(const RingParams& rp, size_t smem, int grid, cudaStream_t st, bool pdl, int mode) {
  if (mode == 1) return launch_ring_shape<T, false, 1>(rp, smem, grid, st, pdl);
  if (mode == 2) return launch_ring_shape<T, false, 2>(rp, smem, grid, st, pdl);
  return rp.p.label_smoothing != 0.f ? launch_ring_shape<T, true, 0>(rp, smem, grid, st, pdl) : launch_ring_shape<T, false, 0>(rp, smem, grid, st, pdl);
}

}  // namespace

int ring_set_max_bytes(int n) {
  if (n < 16384 || n > 65536) return SB_ERR_INVALID_ARGUMENT;
  g_ring_max_bytes = n;
  return SB_OK;
}

int ring_set_warps(int n) {
  if (n < 0 || n > kRingWarps) return SB_ERR_INVALID_ARGUMENT;
  g_ring_warps = n;
  return SB_OK;
}

bool ring_rows_applies(int dtype, int64_t classes, const void* logits, const void* grad) {
  if (dtype != SB_F32 && dtype != SB_BF16 && dtype != SB_F16) return false;
  const uint64_t row_bytes = static_cast<uint64_t>(classes) * dtype_size(dtype);
  if (row_bytes < kRingMinRowBytes || row_bytes > static_cast<uint64_t>(g_ring_max_bytes) || row_bytes % 16) return false;
  return reinterpret_cast<uintptr_t>(logits) % 16 == 0 && reinterpret_cast<uintptr_t>(grad) % 16 == 0;
}

namespace {
int launch_ring(const CEParams& p, cudaStream_t st, bool pdl, int mode) {
  RingParams rp;
  rp.p = p;
  rp.row_bytes = static_cast<uint32_t>(p.classes * dtype_size(p.dtype));
  rp.units = rp.row_bytes / 16;
  uint32_t group_rows = kRingGroupBytes / rp.row_bytes;
  if (group_rows < 1) group_rows = 1;
  if (static_cast<int64_t>(group_rows) > p.rows) group_rows = static_cast<uint32_t>(p.rows);
  rp.group_rows = group_rows;
  rp.ngroups = (p.rows + group_rows - 1) / group_rows;
  const size_t slot_bytes = static_cast<size_t>(group_rows) * rp.row_bytes;
  const size_t room = ring_smem_limit() - sizeof(RingTail) - 128;
  uint32_t nslots = static_cast<uint32_t>(room / slot_bytes);
  if (nslots > kRingMaxSlots) nslots = kRingMaxSlots;
  if (nslots < 3) return SB_ERR_UNSUPPORTED;
  rp.nslots = nslots;
  // Consumer warps: the arithmetic per byte is fixed per dtype, so the warps needed to keep up with HBM do not depend on the
  // row length (measured: about 6 for fp32, 12 for 16-bit logits; more warps than that only take slots away from the loads
  // and stores in flight: fp32 rows of 8 KB run at 0.89 of the copy peak with 6 warps, 0.83 with 16).  Rows under 4 KB add a
  // fixed cost per row and take all 16.  At least four slots' worth of rows stay with the copy engine.
  uint32_t nwarps = rp.row_bytes < 4096 ? kRingWarps : (dtype_size(p.dtype) == 2 ? 12 : 7);
  const uint32_t held_max = nslots * group_rows > 4 * group_rows + 2 ? nslots * group_rows - 4 * group_rows : 2;
  if (nwarps > held_max) nwarps = held_max;
  if (nwarps > static_cast<uint32_t>(kRingWarps)) nwarps = kRingWarps;
  if (nwarps < 2) nwarps = 2;
  if (rp.units > 1024) {
    // rows of more than 16 KB: teams of four warps, one slot each; three slots stay with the copy engine
    uint32_t teams = nslots > 4 ? nslots - 3 : 1;
    if (teams > 4) teams = 4;
    nwarps = teams * 4;
  }
  if (g_ring_warps > 0 && g_ring_warps <= kRingWarps && (rp.units <= 1024 || g_ring_warps % 4 == 0)) nwarps = g_ring_warps;
  rp.nwarps = nwarps;
  const size_t smem = static_cast<size_t>(nslots) * slot_bytes + sizeof(RingTail);
  const int64_t sms = sm_count();
  const int grid = static_cast<int>(rp.ngroups < sms ? rp.ngroups : sms);
  switch (p.dtype) {
    case SB_F32: return launch_ring_t<float>(rp, smem, grid, st, pdl, mode);
    case SB_BF16: return launch_ring_t<__nv_bfloat16>(rp, smem, grid, st, pdl, mode);
    default: return launch_ring_t<__half>(rp, smem, grid, st, pdl, mode);
  }
}
}  // namespace

int ce_launch_ring_rows(const CEParams& p, cudaStream_t st, bool pdl) { return launch_ring(p, st, pdl, 0); }

// log_softmax (mode 1) / softmax (mode 2) over the last dimension of a contiguous [rows, dim] array on the same ring.
// SB_ERR_UNSUPPORTED when the shape does not qualify.
int lsm_launch_ring(const void* in, void* out, int dtype, int64_t rows, int64_t dim, int mode, cudaStream_t st) {
  if (rows <= 0 || !ring_rows_applies(dtype, dim, in, out)) return SB_ERR_UNSUPPORTED;
  CEParams p{};
  p.logits = in;
  p.grad = out;
  p.rows = rows;
  p.classes = dim;
  p.dtype = dtype;
  p.grad_scale = 1.f;
  p.reduction = SB_REDUCTION_NONE;
  return launch_ring(p, st, false, mode);
}

}  // namespace sb

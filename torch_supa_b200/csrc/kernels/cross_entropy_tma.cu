// Cross entropy with the row resident in shared memory: one HBM read and one HBM write per logit.
//
// A persistent CTA (or a cluster of 2 / 4 CTAs that split the row) owns every num_clusters-th row.
// The row slice is cut into chunks of about 8 KB.  The CTA is divided into G warp groups; group g owns
// the chunks c = g, g + G, ... of every row together with a private ring of shared-memory buffers, and
// runs its own little pipeline:
//
//   * the group's first thread streams its chunks in with 1-D bulk copies (cp.async.bulk global ->
//     shared, completion on one mbarrier per buffer) and streams finished chunks out with bulk stores
//     (cp.async.bulk shared -> global, bulk groups);
//   * the group's threads sweep their chunks twice while they sit in shared memory: sweep A
//     accumulates the online (max, sum exp) and sum x as chunks land, sweep B overwrites each chunk in
//     place with the gradient; a group-wide named barrier (not a CTA barrier) precedes each store;
//   * a buffer is handed back to the loader as soon as its store has finished reading it, so the
//     loads of the next rows run under sweep B of the current row and under sweep A of the next.
//
// Groups meet once per row, to combine their statistics.  With a cluster the per-CTA partials
// {max, sum, sum x, x[target]} are exchanged through distributed shared memory (st.shared::cluster into
// every peer, then one cluster barrier per row).
//
// Arithmetic uses the packed fp32 pair instructions of sm_100 (fma/add .f32x2), packed bf16 maxima and
// ex2.approx; the row statistics are in base 2 (max2 = max * log2 e).
//
// Rows whose pitch is not a multiple of 16 bytes (vocabularies such as 50257 or 151643) run the same pipeline
// (kRagged) over the 16-byte units that lie wholly inside the row.  The row may begin inside a unit and end inside
// another: those two edge units, which it shares with its neighbours, travel apart (two 16-byte bulk copies per row into a
// small slot ring of their own) and one thread handles their few elements with scalar arithmetic and ordinary stores,
// so a neighbouring row's bytes are never written and the vector sweeps never see a foreign element.
//
// No TMA multicast is used anywhere: every CTA fetches its own chunks.  Every mbarrier wait is
// bounded; a wait that runs out sets SB_STATUS_KERNEL_TIMEOUT and the kernel still terminates.
#include <type_traits>

#include "ce_ring.cuh"

namespace sb {

using namespace ring;

namespace {

int g_ce_force_variant = -1;  // tuning: -1 automatic, 0 generic, 1/2/4 resident cluster size
int g_ce_keep = 1;  // tuning: 1 = bf16 gradients from kept exponentials (one ex2 per logit), 0 = recompute (two)
int g_ce_window_chunks = -1;  // tuning: chunks of the next row a group may fold while it waits for the exchange; -1 automatic

struct ResidentParams {
  CEParams p;
  uint32_t nch;          // chunks per row slice
  uint32_t nbuf;         // ring buffers (>= nch + 1)
  uint32_t chunk_units;  // 16-byte units per chunk
  uint32_t slice_units;  // 16-byte units per CTA slice (last CTA of a cluster may own fewer)
  uint32_t row_units;    // 16-byte units per row (ragged rows: the most whole units a row can have)
  uint32_t num_clusters;
  int mode;              // 0 cross entropy, 1 log_softmax, 2 softmax
  uint32_t window;       // chunks of the next row a group may fold while the row statistics are exchanged
  uint64_t row_bytes;    // exact bytes of one row (classes * sizeof(T))
};

constexpr int kGroups = 4;          // consumer warp groups per CTA
constexpr int kGroupThreads = 128;  // threads per group
constexpr int kVecPerThread = 4;    // 16-byte vectors a thread handles per chunk
constexpr int kChunkUnits = kGroupThreads * kVecPerThread;  // 512 units = 8 KB per chunk
constexpr int kConsumers = kGroups * kGroupThreads;
constexpr int kResidentThreads = kConsumers + 32 * kGroups;  // plus one copy-engine warp per group
constexpr int kMaxBuffers = 32;
constexpr int kEdgeSlots = kMaxBuffers / kGroups;

// Shared-memory carve-up after the chunk ring.
struct alignas(16) Tail {
  float4 slots[2][4];        // cluster exchange: [row parity][source CTA] = {max2, sum, sum x, x[target]}
  float red[3][32];          // per-warp partials
  float xt_kept;             // kept-exponential mode: x[target] saved by the thread that owns it before it is overwritten
  float xt_edge;             // ragged rows: x[target] when the target lies in an edge unit, saved by the lane that holds it
  unsigned long long full[kMaxBuffers];   // loader -> consumers: chunk has landed
  unsigned long long ready[kMaxBuffers];  // consumers -> loader: chunk holds the gradient (or may be reused)
  // ragged rows: the first and the last 16-byte unit of a row, when the row owns only part of them, for the row in slot
  // (local row number % kEdgeSlots).  A slot is rewritten kEdgeSlots rows later; the loader is never more than
  // kMaxBuffers / kGroups = kEdgeSlots rows ahead of the row being retired.
  uint4 edge[kEdgeSlots][2];
  unsigned long long edge_full[kEdgeSlots];
};

// Where a row lies in 16-byte units.  With an aligned pitch this is the same for every row; with kRagged the row starts
// head_e elements into a unit and owns only tail_e elements of its last one; `span` counts the units wholly inside the
// row, which are what the chunks are cut from.
struct RowGeom {
  uint32_t head_e;    // elements of the unit before the first whole one that belong to the previous row; 0 = no such unit
  uint32_t tail_e;    // elements of the unit after the last whole one that belong to this row; 0 = no such unit
  uint32_t span;      // whole units
  int64_t byte_off;   // byte offset of the first whole unit from the tensor's base pointer
  int64_t class0;     // class index of the first element of the first whole unit
};

// kKeep (cross entropy on 16-bit logits, at most kKeepChunks chunks per group and row): the statistics sweep overwrites
// each chunk with its exponentials 2^(x log2e - m), m being the thread's running maximum at that chunk, and the gradient
// sweep only rescales them: one ex2 per logit instead of two and a third fewer instructions, which is what limits this
// kernel on bf16 (special-function unit, issue slots and, under sustained load, the power cap).  The kept value is
// rounded to bf16 once more than in the two-ex2 form (relative error 2^-8 instead of 2^-9 on the gradient, still far
// inside the 1e-2 the reference allows for bf16, whose own backward starts from bf16 log-probabilities).
constexpr int kKeepChunks = 4;
template <typename T, int CLUSTER, bool kSumX, int MODE, bool kKeep = false, bool kRagged = false>
__global__ void __launch_bounds__(kResidentThreads, 1) ce_resident_kernel(ResidentParams rp) {
  extern __shared__ __align__(128) unsigned char smem[];
  using U = Unit<T>;
  constexpr int E = 2 * U::kPairs;  // elements per 16-byte vector
  constexpr int G = kGroups, TG = kGroupThreads, NV = kVecPerThread;
  constexpr uint32_t kChunkBytes = kChunkUnits * 16;
  const CEParams& p = rp.p;

  // The next kernel of the stream may be scheduled as soon as this one's CTAs are resident (it waits for this
  // kernel's results itself if it was launched as a programmatic dependent; otherwise this changes nothing).
  grid_dep_launch();

  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t cpg = rp.nch / G;   // chunks per group and row
  const uint32_t nbg = rp.nbuf / G;  // ring buffers per group
  Tail* tail = reinterpret_cast<Tail*>(smem + static_cast<size_t>(rp.nbuf) * kChunkBytes);

  const uint32_t cta_rank = CLUSTER > 1 ? cluster_ctarank() : 0;
  const uint32_t cluster_id = blockIdx.x / CLUSTER;
  const int64_t nrows_local = cluster_id < p.rows ? (p.rows - cluster_id + rp.num_clusters - 1) / rp.num_clusters : 0;

  // this CTA's slice of a row, in 16-byte units
  const uint32_t slice_begin = cta_rank * rp.slice_units;
  const uint32_t base_mis = kRagged ? static_cast<uint32_t>(reinterpret_cast<uintptr_t>(p.logits) & 15) : 0;
  auto row_geom = [&](int64_t row) -> RowGeom {
    RowGeom g;
    if constexpr (!kRagged) {
      g.head_e = 0;
      g.tail_e = 0;
      g.span = rp.row_units;
      g.byte_off = row * static_cast<int64_t>(rp.row_bytes);
      g.class0 = 0;
    } else {
      const uint64_t a0 = base_mis + static_cast<uint64_t>(row) * rp.row_bytes;  // the row's address modulo 16 is a0 modulo 16
      const uint32_t head_b = static_cast<uint32_t>(a0 & 15);
      const uint64_t total = head_b + rp.row_bytes;
      const uint32_t touched = static_cast<uint32_t>((total + 15) >> 4);
      g.head_e = head_b / sizeof(T);
      g.tail_e = static_cast<uint32_t>(total & 15) / sizeof(T);
      const uint32_t first = g.head_e ? 1 : 0, last = touched - (g.tail_e ? 1 : 0);
      g.span = last > first ? last - first : 0;
      g.byte_off = row * static_cast<int64_t>(rp.row_bytes) - head_b + first * 16;
      g.class0 = g.head_e ? static_cast<int64_t>(E) - g.head_e : 0;
    }
    return g;
  };
  auto slice_len_of = [&](const RowGeom& g) -> uint32_t {
    return g.span > slice_begin ? min(rp.slice_units, g.span - slice_begin) : 0;
  };
  // Units of chunk `cl` of group `g` that lie in the slice.
  auto chunk_range = [&](uint32_t slice_len, uint32_t g, uint32_t cl, uint32_t& u0, uint32_t& len) {
    u0 = (cl * G + g) * kChunkUnits;
    len = u0 < slice_len ? min(static_cast<uint32_t>(kChunkUnits), slice_len - u0) : 0;
  };

  if (tid == 0) {
    for (uint32_t b = 0; b < rp.nbuf; ++b) {
      mbar_init(smem_u32(&tail->full[b]), 1);
      mbar_init(smem_u32(&tail->ready[b]), TG / 32);
    }
    for (int e = 0; e < kEdgeSlots; ++e) mbar_init(smem_u32(&tail->edge_full[e]), 1);
    tail->xt_kept = 0.f;
    tail->xt_edge = 0.f;
    fence_mbar_init();
  }
  __syncthreads();
  if (CLUSTER > 1) {  // peers must not write our slots before we are resident
    cluster_arrive();
    cluster_wait();
  }

  bool timed_out = false;

  // Buffer numbering: group g owns buffers g * nbg .. g * nbg + nbg - 1; its chunks are numbered
  // i = k * cpg + cl (local row k, cl-th chunk of the group in that row), chunk-in-row c = cl * G + g,
  // buffer j = i % nbg, mbarrier phase parity (i / nbg) & 1.

  if (warp >= kConsumers / 32) {
    // =================== copy-engine warps: one per group; loads, stores, buffer recycling ===================
    // Lane 0 does the work; the whole warp walks the row loop so that it can join the per-row cluster
    // barrier (which counts every thread of every CTA) in step with the consumers.
    const uint32_t g = warp - kConsumers / 32;
    const int64_t per_group = nrows_local * cpg;
    const uint32_t ring_base = smem_u32(smem) + g * nbg * kChunkBytes;
    const uint32_t full_base = smem_u32(&tail->full[g * nbg]);
    const uint32_t ready_base = smem_u32(&tail->ready[g * nbg]);
    int64_t next_load = 0, ld_k = 0;
    uint32_t ld_j = 0, ld_cl = 0;
    bool ld_skip = false;  // the row being loaded is ignored: its logits are never read
    RowGeom ld_geom = row_geom(cluster_id);
    uint32_t ld_slice = slice_len_of(ld_geom);
    int64_t ld_target = (MODE == 0 && lane == 0 && nrows_local > 0) ? p.target[cluster_id] : 0;
    auto load_next = [&]() {  // loads the group's next chunk into the buffer its ring position names
      if (next_load >= per_group) return;
      const int64_t row = cluster_id + ld_k * static_cast<int64_t>(rp.num_clusters);
      if (ld_cl == 0) {
        if (MODE == 0) {
          const int64_t tr = ld_target;  // fetched one row ahead so that the load never waits on it
          ld_skip = tr == p.ignore_index || tr < 0 || tr >= p.classes;  // the consumers' notion of "ignored"
          if (ld_k + 1 < nrows_local) ld_target = p.target[row + rp.num_clusters];
        }
        ld_geom = row_geom(row);
        ld_slice = slice_len_of(ld_geom);
        if (kRagged && g == 0 && cta_rank == 0) {
          // the units the row shares with its neighbours go to the slot ring of their own
          const uint32_t slot = static_cast<uint32_t>(ld_k % kEdgeSlots);
          const uint32_t ebar = smem_u32(&tail->edge_full[slot]);
          const uint32_t nedge = ld_skip ? 0 : (ld_geom.head_e ? 1 : 0) + (ld_geom.tail_e ? 1 : 0);
          if (nedge) {
            const unsigned char* first_whole = static_cast<const unsigned char*>(p.logits) + ld_geom.byte_off;
            mbar_expect_tx(ebar, nedge * 16);
            if (ld_geom.head_e) bulk_g2s(smem_u32(&tail->edge[slot][0]), first_whole - 16, 16, ebar);
            if (ld_geom.tail_e) bulk_g2s(smem_u32(&tail->edge[slot][1]), first_whole + static_cast<size_t>(ld_geom.span) * 16, 16, ebar);
          } else {
            mbar_arrive(ebar);
          }
        }
      }
      const uint32_t u0 = (ld_cl * G + g) * kChunkUnits;
      const uint32_t len = (!ld_skip && u0 < ld_slice) ? min(static_cast<uint32_t>(kChunkUnits), ld_slice - u0) : 0;
      const uint32_t bar = full_base + 8 * ld_j;
      if (len) {
        const unsigned char* src =
            static_cast<const unsigned char*>(p.logits) + ld_geom.byte_off + static_cast<int64_t>(slice_begin + u0) * 16;
        mbar_expect_tx(bar, len * 16);
        bulk_g2s(ring_base + ld_j * kChunkBytes, src, len * 16, bar);
      } else {
        mbar_arrive(bar);
      }
      ++next_load;
      if (++ld_j == nbg) ld_j = 0;
      if (++ld_cl == cpg) {
        ld_cl = 0;
        ++ld_k;
      }
    };
    if (lane == 0)
      for (uint32_t j = 0; j < nbg; ++j) load_next();  // prologue: fill the ring
    uint32_t j = 0, ph = 0;  // ring position / phase parity of the chunk being retired
    bool pending = false;    // a committed store whose buffer has not been recycled yet
    for (int64_t k = 0; k < nrows_local; ++k) {
      if (CLUSTER > 1) {  // the consumers' statistics exchange of row k
        cluster_arrive();
        cluster_wait();
      }
      if (lane == 0) {
        const int64_t row = cluster_id + k * static_cast<int64_t>(rp.num_clusters);
        const RowGeom rg = row_geom(row);
        const uint32_t slice_len = slice_len_of(rg);
        for (uint32_t cl = 0; cl < cpg; ++cl) {
          if (!mbar_wait(ready_base + 8 * j, ph)) timed_out = true;
          if (p.grad) {
            uint32_t u0, len;
            chunk_range(slice_len, g, cl, u0, len);
            if (len) {
              unsigned char* dst =
                  static_cast<unsigned char*>(p.grad) + rg.byte_off + static_cast<int64_t>(slice_begin + u0) * 16;
              bulk_s2g(dst, ring_base + j * kChunkBytes, len * 16);
            }
            bulk_commit();
            bulk_wait_read<1>();  // every store of this thread but the newest has finished reading shared memory
            if (pending) load_next();
            pending = true;
          } else {
            load_next();  // forward only: the buffer is free as soon as the group has read it
          }
          if (++j == nbg) {
            j = 0;
            ph ^= 1;
          }
        }
      }
      __syncwarp();
    }
    if (lane == 0) bulk_wait_all();
    __syncwarp();
    if (CLUSTER > 1) {  // the final cluster barrier
      cluster_arrive();
      cluster_wait();
    }
    if (timed_out && lane == 0 && p.status) atomicOr(p.status, SB_STATUS_KERNEL_TIMEOUT);
    return;
  }

  // =================== consumer warps ===================
  const uint32_t grp = tid / TG, gt = tid - grp * TG;
  unsigned char* ring = smem + static_cast<size_t>(grp) * nbg * kChunkBytes;  // this group's ring
  const uint32_t full0 = smem_u32(&tail->full[grp * nbg]);
  const uint32_t ready0 = smem_u32(&tail->ready[grp * nbg]);

  uint32_t cj = 0, cphase = 0;  // ring position and phase parity of the group's first chunk of the current row
  const float eps = p.label_smoothing;
  const float eps_c = eps / static_cast<float>(p.classes);
  const int64_t elems_per_chunk = static_cast<int64_t>(kChunkUnits) * E;
  const int64_t slice_elem0 = static_cast<int64_t>(slice_begin) * E;
  float base_scale = p.grad_scale;  // gradient scale that does not depend on the row
  // `mean` divides by the valid-row count, which the kernel before this one in the stream produces.  When the launch
  // allows this kernel to start under that one, the copy-engine warps fill the ring in the meantime and the consumers wait
  // here.  (Waiting later, right before the first gradient sweep, put the wait inside the row loop and cost the 16-bit
  // sweeps 4 % on B200.)
  if (p.grad && p.reduction == SB_REDUCTION_MEAN) {
    grid_dep_wait();
    base_scale = static_cast<float>(static_cast<double>(base_scale) / p.acc[1]);
  }

  // Folds the group's chunks [from, cpg) of the row whose first chunk sits at ring position (j0, ph0) into
  // the statistics and returns how many chunks of the row are done.  blocking: wait for every chunk;
  // otherwise stop at the first chunk that has not landed yet (used to fill the wait for the peers'
  // statistics with the next row's work).
  auto fold_chunks = [&](RowStats& st, const RowGeom& rg, uint32_t j0, uint32_t ph0, uint32_t from, uint32_t to, bool skip,
                         bool blocking) -> uint32_t {
    uint32_t j = j0 + from, ph = ph0;
    if (j >= nbg) {  // from < cpg < nbg: one wrap at most
      j -= nbg;
      ph ^= 1;
    }
    const uint32_t slice_len = slice_len_of(rg);
    uint32_t cl = from;
    for (; cl < to; ++cl) {
      const uint32_t bar = full0 + 8 * j;
      if (blocking) {
        if (!mbar_wait(bar, ph)) timed_out = true;
      } else if (!__all_sync(0xffffffffu, mbar_test_wait(bar, ph))) {
        break;
      }
      if (!skip) {
        uint32_t u0, len;
        chunk_range(slice_len, grp, cl, u0, len);
        const uint4* buf = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(j) * kChunkBytes) + gt;
        if (len == kChunkUnits) {
          uint4 r[NV];
#pragma unroll
          for (int q = 0; q < NV; ++q) r[q] = buf[q * TG];
          stats_update<T, NV, kSumX>(st, r);
        } else {
          for (uint32_t v = gt; v < len; v += TG) {  // short last chunk of the slice
            uint4 r[1] = {buf[v - gt]};
            stats_update<T, 1, kSumX>(st, r);
          }
        }
      }
      if (++j == nbg) {
        j = 0;
        ph ^= 1;
      }
    }
    return cl;
  };
  auto is_ignored = [&](int64_t t) { return MODE == 0 && (t == p.ignore_index || t < 0 || t >= p.classes); };

  RowStats st;  // statistics of the row in sweep A; re-initialised as soon as they have been reduced
  st.m2 = -CUDART_INF_F;
  st.s[0] = st.s[1] = st.sx[0] = st.sx[1] = make_float2(0.f, 0.f);
  uint32_t a_done = 0;  // chunks of the current row already folded (during the previous row's exchange)
  uint32_t xpar = 0;    // which pair of exchange slots the row uses; advances with every row that is not ignored

  int64_t t_next = (MODE == 0 && nrows_local > 0) ? p.target[cluster_id] : 0;
  for (int64_t k = 0; k < nrows_local; ++k) {
    const int64_t row = cluster_id + k * static_cast<int64_t>(rp.num_clusters);
    const int64_t t = t_next;
    if (MODE == 0 && k + 1 < nrows_local) t_next = p.target[row + rp.num_clusters];  // in flight during this row's sweeps
    const bool ignored = is_ignored(t);
    if (MODE == 0 && ignored && t != p.ignore_index && tid == 0 && cta_rank == 0 && p.status)
      atomicOr(p.status, SB_STATUS_TARGET_OUT_OF_RANGE);
    const RowGeom rg = row_geom(row);
    const uint32_t slice_len = slice_len_of(rg);
    const int64_t t_slice = t - rg.class0 - slice_elem0;  // element position of the target in this CTA's slice of whole units
    // Ragged rows: the elements of the two edge units (they arrive in a slot ring of their own) are spread over the lanes of
    // warp 0 of the cluster's first CTA, one element per lane: lane l holds element l % E of the head unit (l < E) or of
    // the tail unit.  Each lane folds its element into its own statistics, which the warp reduction below merges anyway.
    const uint32_t edge_slot = static_cast<uint32_t>(k % kEdgeSlots);
    const int64_t tail_class0 = rg.class0 + static_cast<int64_t>(rg.span) * E;  // class of the first element after the whole units
    bool edge_lane = false;      // this thread holds an element of an edge unit that belongs to the row
    const T* edge_elem = nullptr;
    int64_t edge_class = 0;
    if constexpr (kRagged) {
      if (tid < 2 * E && cta_rank == 0) {
        const uint32_t which = tid / E, e = tid % E;
        edge_lane = which == 0 ? (rg.head_e != 0 && e >= rg.head_e) : (e < rg.tail_e);
        edge_elem = reinterpret_cast<const T*>(&tail->edge[edge_slot][which]) + e;
        edge_class = which == 0 ? static_cast<int64_t>(e) - rg.head_e : tail_class0 + e;
      }
      if (warp == 0 && cta_rank == 0 && !ignored && (rg.head_e != 0 || rg.tail_e != 0)) {
        if (!mbar_wait(smem_u32(&tail->edge_full[edge_slot]), static_cast<uint32_t>(k / kEdgeSlots) & 1)) timed_out = true;
        if (edge_lane) {
          const float x = to_float(*edge_elem);
          const float nm = max_nan(st.m2, x * kLog2e);
          const float resc = ex2(nm == -CUDART_INF_F ? 0.f : st.m2 - nm);
          st.s[0] = mul2(st.s[0], make_float2(resc, resc));
          st.s[1] = mul2(st.s[1], make_float2(resc, resc));
          st.m2 = nm;
          st.s[0].x += ex2(fmaf(x, kLog2e, nm == -CUDART_INF_F ? 0.f : -nm));
          if (kSumX) st.sx[0].x += x;
          if (edge_class == t) tail->xt_edge = x;
        }
      }
    }

    // ---- sweep A: statistics as the group's chunks land (the first a_done chunks are folded already) ----
    float mref[kKeepChunks];          // kept mode: the maximum each of the group's chunks was scaled by (per thread)
    uint32_t t_cl = 0xffffffffu, t_off = 0;  // kept mode: chunk of this group and element offset of the target, if this thread owns it
    if constexpr (kKeep) {
      if (!ignored) {
        if (t_slice >= 0 && t_slice < static_cast<int64_t>(slice_len) * E) {
          const uint32_t tu = static_cast<uint32_t>(t_slice) / E;
          const uint32_t c = tu / kChunkUnits, v = tu % kChunkUnits;
          if (c % G == grp && v % TG == gt) {
            t_cl = c / G;
            t_off = static_cast<uint32_t>(t_slice) - c * (kChunkUnits * E);
          }
        }
      }
      uint32_t j = cj, ph = cphase;
#pragma unroll
      for (int cl = 0; cl < kKeepChunks; ++cl) {
        mref[cl] = -CUDART_INF_F;
        if (static_cast<uint32_t>(cl) < cpg) {
          if (!mbar_wait(full0 + 8 * j, ph)) timed_out = true;
          if (!ignored) {
            uint32_t u0, len;
            chunk_range(slice_len, grp, cl, u0, len);
            unsigned char* chunk = ring + static_cast<size_t>(j) * kChunkBytes;
            uint4* buf = reinterpret_cast<uint4*>(chunk) + gt;
            // the logit of the target is needed for the loss: its owner saves it before the chunk is overwritten
            if (static_cast<uint32_t>(cl) == t_cl) tail->xt_kept = to_float(reinterpret_cast<const T*>(chunk)[t_off]);
            if (len == kChunkUnits) {
              uint4 r[NV], e[NV];
#pragma unroll
              for (int q = 0; q < NV; ++q) r[q] = buf[q * TG];
              stats_update<T, NV, kSumX, true>(st, r, e);
#pragma unroll
              for (int q = 0; q < NV; ++q) buf[q * TG] = e[q];
            } else {
              // short last chunk of the slice: one maximum for all of this thread's vectors, then the exponentials
              float vm = -CUDART_INF_F;
              for (uint32_t v = gt; v < len; v += TG) vm = max_nan(vm, U::vmax(buf[v - gt]));
              const float nm = max_nan(st.m2, vm * kLog2e);
              const float resc = ex2(nm == -CUDART_INF_F ? 0.f : st.m2 - nm);
              st.s[0] = mul2(st.s[0], make_float2(resc, resc));
              st.s[1] = mul2(st.s[1], make_float2(resc, resc));
              st.m2 = nm;  // stats_update below finds its maximum already in place: no further rescaling
              for (uint32_t v = gt; v < len; v += TG) {
                uint4 r[1] = {buf[v - gt]}, e[1];
                stats_update<T, 1, kSumX, true>(st, r, e);
                buf[v - gt] = e[0];
              }
            }
            mref[cl] = st.m2;
          }
          if (++j == nbg) {
            j = 0;
            ph ^= 1;
          }
        }
      }
    } else {
      fold_chunks(st, rg, cj, cphase, a_done, cpg, ignored, true);
    }

    // ---- CTA reduce; the other warps go on to the next row's chunks while warp 0 combines ----
    if (!ignored) {
      float m2 = st.m2;
      float s = (st.s[0].x + st.s[0].y) + (st.s[1].x + st.s[1].y);
      float sx = (st.sx[0].x + st.sx[0].y) + (st.sx[1].x + st.sx[1].y);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        merge2(m2, s, __shfl_xor_sync(0xffffffffu, m2, o), __shfl_xor_sync(0xffffffffu, s, o));
        sx += __shfl_xor_sync(0xffffffffu, sx, o);
      }
      if (lane == 0) {
        tail->red[0][warp] = m2;
        tail->red[1][warp] = s;
        tail->red[2][warp] = sx;
      }
      __syncwarp();
      if (warp != 0) {
        named_barrier_arrive(1, kConsumers);  // partials published; no need to wait here
      } else {
        named_barrier(1, kConsumers);
        float wm = lane < kConsumers / 32 ? tail->red[0][lane] : -CUDART_INF_F;
        float wsum = lane < kConsumers / 32 ? tail->red[1][lane] : 0.f;
        float wx = lane < kConsumers / 32 ? tail->red[2][lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          merge2(wm, wsum, __shfl_xor_sync(0xffffffffu, wm, o), __shfl_xor_sync(0xffffffffu, wsum, o));
          wx += __shfl_xor_sync(0xffffffffu, wx, o);
        }
        if (lane == 0) {
          // x[target] if it lies in this CTA's slice: chunk c of the row belongs to group c % G
          float xt = 0.f;
          if (kKeep) {  // saved by its owner during the sweep (ordered by the barrier above); 0 when another CTA holds the target
            xt = tail->xt_kept;
            tail->xt_kept = 0.f;
          } else if (MODE == 0 && t_slice >= 0 && t_slice < static_cast<int64_t>(slice_len) * E) {
            const uint32_t c = static_cast<uint32_t>(t_slice / elems_per_chunk);
            const uint32_t off = static_cast<uint32_t>(t_slice - c * elems_per_chunk);
            const uint32_t og = c % G, ocl = c / G;
            uint32_t oj = cj + ocl, oph = cphase;  // every group is at the same ring position
            if (oj >= nbg) {
              oj -= nbg;
              oph ^= 1;
            }
            // already complete (the owning group passed it before the barrier above): makes the data visible here
            if (!mbar_wait(smem_u32(&tail->full[og * nbg + oj]), oph)) timed_out = true;
            xt = to_float(reinterpret_cast<const T*>(smem + (static_cast<size_t>(og) * nbg + oj) * kChunkBytes)[off]);
          }
          if (kRagged) {  // written by a lane of this warp before the barrier above
            xt += tail->xt_edge;
            tail->xt_edge = 0.f;
          }
          if (CLUSTER > 1) {
            const uint32_t slot = smem_u32(&tail->slots[xpar][cta_rank]);
#pragma unroll
            for (int jj = 0; jj < CLUSTER; ++jj) st_cluster_f4(mapa(slot, jj), wm, wsum, wx, xt);
          } else {
            tail->slots[xpar][0] = make_float4(wm, wsum, wx, xt);
          }
        }
        __syncwarp();
      }
    }
    // Everybody signals that its part of the exchange is done (the cluster barrier is the hardware's; an
    // mbarrier-based exchange with remote arrivals measured 12 % slower), then fills the time until the others
    // have signalled too with whatever part of the next row is already in shared memory (at most rp.window chunks).
    if (CLUSTER > 1) cluster_arrive();  // every thread of the cluster, ignored rows included
    st.m2 = -CUDART_INF_F;
    st.s[0] = st.s[1] = st.sx[0] = st.sx[1] = make_float2(0.f, 0.f);
    a_done = 0;
    if (!kKeep && k + 1 < nrows_local) {
      uint32_t nj = cj + cpg, nph = cphase;
      if (nj >= nbg) {
        nj -= nbg;
        nph ^= 1;
      }
      a_done = fold_chunks(st, row_geom(row + rp.num_clusters), nj, nph, 0, min(cpg, rp.window), is_ignored(t_next), false);
    }
    if (CLUSTER > 1) {
      cluster_wait();
    } else {
      named_barrier(2, kConsumers);  // warp 0 wrote the slot before it started on the next row
    }
    float lse = 0.f, scale = 0.f, xt_all = 0.f;
    if (!p.grad) {
      // forward only: every read of this row's chunks (x[target] included) lies before the barrier above;
      // hand the buffers back, one arrival per warp and chunk
      if (lane == 0) {
        uint32_t j = cj;
        for (uint32_t cl = 0; cl < cpg; ++cl) {
          mbar_arrive(ready0 + 8 * j);
          if (++j == nbg) j = 0;
        }
      }
    }
    if (!ignored) {
      float gm = -CUDART_INF_F, gs = 0.f, gx = 0.f;
#pragma unroll
      for (int jj = 0; jj < CLUSTER; ++jj) {
        const float4 v = tail->slots[xpar][jj];
        merge2(gm, gs, v.x, v.y);
        gx += v.z;
        xt_all += v.w;
      }
      lse = (gm + log2f(gs)) * kLn2;
      const float wt = (MODE == 0 && p.class_weight) ? p.class_weight[t] : 1.f;
      if (MODE == 0 && tid == 0 && cta_rank == 0) {
        p.row_loss[row] = ce_row_loss(lse, xt_all, gx, eps, eps_c) * wt;
        if (p.row_lse) p.row_lse[row] = lse;
      }
      scale = base_scale * wt;
      if (p.grad && p.row_grad_out) scale *= p.row_grad_out[row];
      if (lse != lse) scale = lse;  // a NaN row: every gradient element is NaN, the polynomial pairs included
    } else if (MODE == 0 && tid == 0 && cta_rank == 0) {
      p.row_loss[row] = 0.f;
      if (p.row_lse) p.row_lse[row] = 0.f;
    }

    // ---- sweep B: gradient in place, chunk by chunk; the copy-engine warp streams it out ----
    if (p.grad) {
      const float sub_all = eps_c * scale;
      const float sub_t = (1.f - eps) * scale;
      const float2 neg_lse2 = make_float2(-lse * kLog2e, -lse * kLog2e);
      const float2 scale2 = make_float2(scale, scale);
      const float2 nsub2 = make_float2(-sub_all, -sub_all);
      const float2 neg_lse_nat2 = make_float2(-lse, -lse);
      // The class of the target gets (1 - eps) * scale subtracted: its owner recomputes that one element from
      // x[target] with the same arithmetic and a single rounding.
      const float g_target = fmaf(ex2(fmaf(xt_all, kLog2e, neg_lse2.x)), scale, -sub_all) - sub_t;
      // Edge units of a ragged row: each of their elements is computed by the lane that holds it and written to global
      // memory on its own (the bulk stores cover whole units only, so a neighbouring row's bytes are never touched).
      if constexpr (kRagged) {
        if (edge_lane) {
          float gv = 0.f;
          if (!ignored) {
            const float x = to_float(*edge_elem);
            if (MODE == 1) {
              gv = x - lse;
            } else {
              gv = fmaf(ex2(fmaf(x, kLog2e, neg_lse2.x)), scale, -sub_all);
              if (MODE == 0 && edge_class == t) gv -= sub_t;
            }
          }
          reinterpret_cast<T*>(static_cast<unsigned char*>(p.grad) + row * static_cast<int64_t>(rp.row_bytes))[edge_class] = from_float<T>(gv);
        }
      }
      if constexpr (kKeep) {
        // the chunks hold 2^(x log2e - mref): the gradient is that times 2^(mref - lse2) * scale, minus the smoothing share
        uint32_t j = cj;
#pragma unroll
        for (int cl = 0; cl < kKeepChunks; ++cl) {
          if (static_cast<uint32_t>(cl) < cpg) {
            uint32_t u0, len;
            chunk_range(slice_len, grp, cl, u0, len);
            unsigned char* chunk = ring + static_cast<size_t>(j) * kChunkBytes;
            uint4* buf = reinterpret_cast<uint4*>(chunk) + gt;
            if (!ignored) {
              const float mr = mref[cl] == -CUDART_INF_F ? 0.f : mref[cl];  // the sweep scaled an all -inf chunk by 2^0
              const float factor = ex2(mr + neg_lse2.x) * scale;
              if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                // bf16: one packed FMA per pair (fp16 stays on fp32 pairs: its factor, about 1 / rows, would be subnormal)
                const __nv_bfloat162 fb = __float2bfloat162_rn(factor);
                const __nv_bfloat162 nb = __float2bfloat162_rn(-sub_all);
                if (len == kChunkUnits) {
                  uint4 r[NV];
#pragma unroll
                  for (int q = 0; q < NV; ++q) r[q] = buf[q * TG];
#pragma unroll
                  for (int q = 0; q < NV; ++q) buf[q * TG] = grad_from_kept_bf16(r[q], fb, nb);
                } else {
                  for (uint32_t v = gt; v < len; v += TG) buf[v - gt] = grad_from_kept_bf16(buf[v - gt], fb, nb);
                }
              } else {
                const float2 factor2 = make_float2(factor, factor);
                if (len == kChunkUnits) {
                  uint4 r[NV];
#pragma unroll
                  for (int q = 0; q < NV; ++q) r[q] = buf[q * TG];
#pragma unroll
                  for (int q = 0; q < NV; ++q) buf[q * TG] = grad_from_kept<T>(r[q], factor2, nsub2);
                } else {
                  for (uint32_t v = gt; v < len; v += TG) buf[v - gt] = grad_from_kept<T>(buf[v - gt], factor2, nsub2);
                }
              }
              if (static_cast<uint32_t>(cl) == t_cl) reinterpret_cast<T*>(chunk)[t_off] = from_float<T>(g_target);
            } else {
              for (uint32_t v = gt; v < len; v += TG) buf[v - gt] = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(ready0 + 8 * j);
            if (++j == nbg) j = 0;
          }
        }
      } else {
      uint32_t j = cj;
      for (uint32_t cl = 0; cl < cpg; ++cl) {
        uint32_t u0, len;
        chunk_range(slice_len, grp, cl, u0, len);
        unsigned char* chunk = ring + static_cast<size_t>(j) * kChunkBytes;
        uint4* buf = reinterpret_cast<uint4*>(chunk) + gt;
        if (!ignored) {
          if (len == kChunkUnits) {
            uint4 r[NV];
#pragma unroll
            for (int q = 0; q < NV; ++q) r[q] = buf[q * TG];
#pragma unroll
            for (int q = 0; q < NV; ++q)
              buf[q * TG] = MODE != 1 ? grad_vector<T>(r[q], neg_lse2, scale2, nsub2) : shift_vector<T>(r[q], neg_lse_nat2);
          } else {
            for (uint32_t v = gt; v < len; v += TG)
              buf[v - gt] = MODE != 1 ? grad_vector<T>(buf[v - gt], neg_lse2, scale2, nsub2) : shift_vector<T>(buf[v - gt], neg_lse_nat2);
          }
          // position of the target inside this chunk, in elements
          const int64_t tl = t_slice - static_cast<int64_t>(u0) * E;
          if (MODE == 0 && tl >= 0 && tl < static_cast<int64_t>(len) * E && (static_cast<uint32_t>(tl) / E) % TG == gt)
            reinterpret_cast<T*>(chunk)[tl] = from_float<T>(g_target);
        } else {
          for (uint32_t v = gt; v < len; v += TG) buf[v - gt] = make_uint4(0u, 0u, 0u, 0u);
        }
        // One fence and hand-over per chunk: pairing two chunks per fence and hoisting the target's position out of
        // this loop were both measured slower (the stores start later; more values live across the sweep).
        fence_proxy_async();  // this thread's writes become visible to the bulk-copy engine
        __syncwarp();
        if (lane == 0) mbar_arrive(ready0 + 8 * j);
        if (++j == nbg) j = 0;
      }
      }
    }

    if (!ignored) xpar ^= 1;
    // advance the ring position to the next row
    cj += cpg;
    while (cj >= nbg) {
      cj -= nbg;
      cphase ^= 1;
    }
  }

  if (timed_out && p.status) atomicOr(p.status, SB_STATUS_KERNEL_TIMEOUT);
  if (CLUSTER > 1) {  // do not retire while a peer may still address our shared memory
    cluster_arrive();
    cluster_wait();
  }
}

size_t resident_smem_bytes(uint32_t nbuf) { return static_cast<size_t>(nbuf) * kChunkUnits * 16 + sizeof(Tail); }

// Rows in 16-byte units.  Of a row whose pitch or base address is not a multiple of 16 bytes the units wholly inside it
// are fetched in chunks; the two units it shares with its neighbours travel apart.
struct RowLayout {
  uint64_t row_bytes;
  uint32_t row_units;  // whole 16-byte units of a row (the most, for ragged rows)
  bool ragged;
  bool ok;
};
RowLayout row_layout(int dtype, int64_t classes, const void* logits, const void* out) {
  RowLayout l{};
  const uint64_t es = static_cast<uint64_t>(dtype_size(dtype));
  l.row_bytes = static_cast<uint64_t>(classes) * es;
  const uintptr_t a = reinterpret_cast<uintptr_t>(logits), b = reinterpret_cast<uintptr_t>(out);
  l.ragged = (l.row_bytes % 16) != 0 || (a % 16) != 0;
  // the output is written from the same shared-memory image: it needs the input's position within a unit
  l.ok = es != 0 && a % es == 0 && (out == nullptr || (b % 16) == (a % 16));
  const uint64_t units = l.row_bytes / 16;  // ragged rows: the most 16-byte units that can lie wholly inside a row
  if (units > 0x7fffffffULL) l.ok = false;
  l.row_units = static_cast<uint32_t>(units);
  return l;
}

// Geometry for a row of `row_units` 16-byte units split over `cluster` CTAs.  Returns false when the
// slice does not fit next to at least one spare buffer per group.
bool resident_geometry(const RowLayout& l, int cluster, size_t smem_limit, ResidentParams* rp) {
  const uint32_t row_units = l.row_units;
  const uint32_t slice_units = (row_units + cluster - 1) / cluster;
  uint32_t cpg = (slice_units + kGroups * kChunkUnits - 1) / (kGroups * kChunkUnits);
  if (cpg == 0) cpg = 1;
  if (smem_limit <= sizeof(Tail)) return false;
  uint32_t nbg = static_cast<uint32_t>((smem_limit - sizeof(Tail)) / (static_cast<size_t>(kChunkUnits) * 16)) / kGroups;
  if (nbg * kGroups > kMaxBuffers) nbg = kMaxBuffers / kGroups;
  if (nbg < cpg + 1) return false;
  rp->nch = cpg * kGroups;
  rp->nbuf = nbg * kGroups;
  rp->chunk_units = kChunkUnits;
  rp->slice_units = slice_units;
  rp->row_units = row_units;
  rp->row_bytes = l.row_bytes;
  rp->window = 0;  // set by the launcher, which knows the element type
  return true;
}

// pdl: launch as a programmatic dependent of the kernel before it in the stream (the caller vouches that this kernel is
// the library's own valid-row count, whose only product, acc[1], the kernel reads behind grid_dep_wait).
template <typename T, int CLUSTER, bool SUMX, int MODE, bool KEEP = false, bool RAGGED = false>
int launch_resident_cfg(ResidentParams rp, cudaStream_t st, bool pdl) {
  auto kernel = ce_resident_kernel<T, CLUSTER, SUMX, MODE, KEEP, RAGGED>;
  const size_t smem = resident_smem_bytes(rp.nbuf);
  static thread_local int configured_device = -1;  // per (instantiation, thread): attribute set for this device
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin()) != cudaSuccess)
      return SB_ERR_CUDA;
    configured_device = dev;
  }
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  int clusters = sm_count() / CLUSTER;
  if (CLUSTER > 1) {
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(sm_count() / CLUSTER * CLUSTER);
    probe.blockDim = dim3(kResidentThreads);
    probe.dynamicSmemBytes = smem;
    probe.attrs = attr;
    probe.numAttrs = 1;
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &probe) == cudaSuccess && max_clusters > 0 &&
        max_clusters < clusters)
      clusters = max_clusters;
  }
  if (clusters < 1) clusters = 1;
  if (static_cast<int64_t>(clusters) > rp.p.rows) clusters = static_cast<int>(rp.p.rows);
  rp.num_clusters = clusters;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * CLUSTER);
  cfg.blockDim = dim3(kResidentThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, rp) != cudaSuccess) {
    cudaGetLastError();
    return SB_ERR_CUDA;
  }
  return SB_OK;
}

template <typename T, int CLUSTER, bool RAGGED>
int launch_resident(ResidentParams rp, cudaStream_t st, bool pdl) {
  // Chunks of the next row a group folds while a row's statistics are exchanged.  Measured on B200: with
  // 4-byte elements the sweeps are short next to the memory time and filling the exchange with the next
  // row's statistics gains 8 %; with 2-byte elements the sweeps set the pace and the same reordering only
  // delays the gradient sweep that frees the buffers the next loads need (-5 % per chunk), so it stays off.
  const uint32_t spare = (rp.nbuf - rp.nch) / kGroups;
  rp.window = g_ce_window_chunks >= 0 ? static_cast<uint32_t>(g_ce_window_chunks) : (sizeof(T) == 4 && spare > 1 ? spare - 1 : 0);
  if (rp.mode == 1) return launch_resident_cfg<T, CLUSTER, false, 1, false, RAGGED>(rp, st, false);
  if (rp.mode == 2) return launch_resident_cfg<T, CLUSTER, false, 2, false, RAGGED>(rp, st, false);
  const bool sumx = rp.p.label_smoothing != 0.f;
  if constexpr (sizeof(T) == 2) {
    // 16-bit logits with a gradient: keep the exponentials of the statistics sweep (see ce_resident_kernel); in fp16 a kept
    // value below 2^-14 is subnormal, an absolute error of at most 2^-25 on a probability
    if (g_ce_keep != 0 && rp.p.grad && rp.nch / kGroups <= static_cast<uint32_t>(kKeepChunks)) {
      rp.window = 0;
      return sumx ? launch_resident_cfg<T, CLUSTER, true, 0, true, RAGGED>(rp, st, pdl)
                  : launch_resident_cfg<T, CLUSTER, false, 0, true, RAGGED>(rp, st, pdl);
    }
  }
  return sumx ? launch_resident_cfg<T, CLUSTER, true, 0, false, RAGGED>(rp, st, pdl)
              : launch_resident_cfg<T, CLUSTER, false, 0, false, RAGGED>(rp, st, pdl);
}

template <typename T>
int launch_resident_t(const ResidentParams& rp, cudaStream_t st, int variant, bool ragged, bool pdl) {
  if (ragged) {
    switch (variant) {
      case 1: return launch_resident<T, 1, true>(rp, st, pdl);
      case 2: return launch_resident<T, 2, true>(rp, st, pdl);
      case 4: return launch_resident<T, 4, true>(rp, st, pdl);
      default: return SB_ERR_INVALID_ARGUMENT;
    }
  }
  switch (variant) {
    case 1: return launch_resident<T, 1, false>(rp, st, pdl);
    case 2: return launch_resident<T, 2, false>(rp, st, pdl);
    case 4: return launch_resident<T, 4, false>(rp, st, pdl);
    default: return SB_ERR_INVALID_ARGUMENT;
  }
}

int launch_resident_any(const ResidentParams& rp, int dtype, cudaStream_t st, int variant, bool ragged, bool pdl) {
  switch (dtype) {
    case SB_F32: return launch_resident_t<float>(rp, st, variant, ragged, pdl);
    case SB_BF16: return launch_resident_t<__nv_bfloat16>(rp, st, variant, ragged, pdl);
    case SB_F16: return launch_resident_t<__half>(rp, st, variant, ragged, pdl);
    default: return SB_ERR_UNSUPPORTED;
  }
}

}  // namespace

// 0: no resident kernel for this shape; 1 / 2 / 4: cluster size.  Rows shorter than 16 KB are left to the kernels that
// hold a row in registers (the per-row barriers of this pipeline would dominate them).
int ce_choose_variant(int dtype, int64_t rows, int64_t classes, const void* logits, const void* grad) {
  if (rows <= 0 || classes <= 0) return 0;
  const RowLayout l = row_layout(dtype, classes, logits, grad);
  if (!l.ok) return 0;
  if (l.row_bytes < 16 * 1024) return 0;
  const size_t limit = static_cast<size_t>(max_smem_optin());
  ResidentParams rp;
  const int candidates[3] = {1, 2, 4};
  for (int c : candidates)
    if (resident_geometry(l, c, limit, &rp)) return c;
  return 0;
}

int ce_launch_resident(const CEParams& p, cudaStream_t st, int variant, bool pdl) {
  ResidentParams rp;
  rp.p = p;
  rp.mode = 0;
  const RowLayout l = row_layout(p.dtype, p.classes, p.logits, p.grad);
  if (!l.ok || !resident_geometry(l, variant, static_cast<size_t>(max_smem_optin()), &rp)) return SB_ERR_INVALID_ARGUMENT;
  return launch_resident_any(rp, p.dtype, st, variant, l.ragged, pdl);
}

// log_softmax over the last dimension with the row resident in shared memory (same pipeline as the cross
// entropy, MODE 1).  Returns SB_ERR_UNSUPPORTED when the shape does not qualify; the caller then uses the
// generic kernels.
int lsm_launch_resident(const void* in, void* out, int dtype, int64_t rows, int64_t dim, int mode, cudaStream_t st) {
  if (g_ce_force_variant == 0) return SB_ERR_UNSUPPORTED;
  const int variant = ce_choose_variant(dtype, rows, dim, in, out);
  if (variant == 0) return SB_ERR_UNSUPPORTED;
  ResidentParams rp;
  rp.p = CEParams{};
  rp.p.logits = in;
  rp.p.grad = out;
  rp.p.rows = rows;
  rp.p.classes = dim;
  rp.p.dtype = dtype;
  rp.p.grad_scale = 1.f;
  rp.mode = mode;
  const RowLayout l = row_layout(dtype, dim, in, out);
  if (!l.ok || !resident_geometry(l, variant, static_cast<size_t>(max_smem_optin()), &rp)) return SB_ERR_UNSUPPORTED;
  return launch_resident_any(rp, dtype, st, variant, l.ragged, false);
}

int ce_choose_family(const CEParams& p) {
  // class weights together with label smoothing weight every class of the row: only the two-sweep kernel reads them
  if (p.class_weight && p.label_smoothing != 0.f) return 0;
  if (g_ce_force_variant == 0) return 0;
  const bool forced_resident = g_ce_force_variant >= 1 && g_ce_force_variant <= 4;
  // Aligned rows of up to 32 KB go to the slot ring: below 64 KB the resident kernel has too few chunks per row for its four
  // groups (fp32 rows of 18 / 24 / 32 KB: 0.47 / 0.60 / 0.73 of the copy peak).
  if (!forced_resident && g_ce_force_variant != 8 && ring_rows_applies(p.dtype, p.classes, p.logits, p.grad)) return 16;
  int variant = ce_choose_variant(p.dtype, p.rows, p.classes, p.logits, p.grad);
  if (forced_resident && variant != 0) variant = g_ce_force_variant;  // falls back if it does not fit
  if (variant != 0) return variant;
  if (g_ce_force_variant != 8 && ring_rows_applies(p.dtype, p.classes, p.logits, p.grad)) return 16;
  return rows_reg_applies(p.dtype, p.classes, p.logits, p.grad) ? 8 : 0;
}

int ce_dispatch(const CEParams& p, cudaStream_t st) {
  const int family = ce_choose_family(p);
  if (family == 16) {
    const int rc = ce_launch_ring_rows(p, st, (p.flags & SB_CE_FLAG_AFTER_COUNT) != 0);
    if (rc == SB_OK) return rc;
    return rows_reg_applies(p.dtype, p.classes, p.logits, p.grad) ? ce_launch_rows_reg(p, st) : ce_launch_generic(p, st);
  }
  if (family == 8) return ce_launch_rows_reg(p, st);
  if (family != 0) {
    const int rc = ce_launch_resident(p, st, family, (p.flags & SB_CE_FLAG_AFTER_COUNT) != 0);
    if (rc == SB_OK) return rc;
  }
  return ce_launch_generic(p, st);
}

}  // namespace sb

// Tuning hook for benchmarks: key 1 = force the kernel family (-1 automatic, 0 generic, 1/2/4 resident cluster size, 8 = short rows in
// registers instead of the shared-memory slot ring); key 2 = chunks of the
// next row folded during the statistics exchange (-1 automatic); key 3 = bf16 gradients from kept exponentials (1, default) or
// recomputed (0).
extern "C" int sb_set_tuning(int32_t key, int32_t value) {
  if (key == 1 && (value == -1 || value == 0 || value == 1 || value == 2 || value == 4 || value == 8)) {
    sb::g_ce_force_variant = value;
    return SB_OK;
  }
  if (key == 3 && (value == 0 || value == 1)) {
    sb::g_ce_keep = value;
    return SB_OK;
  }
  if (key == 2 && value >= -1 && value <= 64) {
    sb::g_ce_window_chunks = value;
    return SB_OK;
  }
  if (key == 5 && value >= 1 && value <= 60000) return sb::xchg_set_timeout_ms(value);
  if (key == 6) return sb::ring_set_warps(value);
  if (key == 7) return sb::ring_set_max_bytes(value);
  if (key == 8) return sb::red_set_warp_row_bytes(value);
  return SB_ERR_INVALID_ARGUMENT;
}

extern "C" int sb_ce_kernel_variant(int32_t dtype, int64_t rows, int64_t classes) {
  sb::CEParams p{};
  p.dtype = dtype;
  p.rows = rows;
  p.classes = classes;
  return sb::ce_choose_family(p);
}

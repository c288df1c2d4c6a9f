// Elementwise engine: descriptor validation, path classification and the C entry points.
#include "elementwise.cuh"

namespace sb {

namespace {

int compute_type_of(int dtype) {
  switch (dtype) {
    case SB_BOOL: return kCtBool;
    case SB_U8: case SB_I8: case SB_I16: case SB_I32: return kCtI32;
    case SB_I64: return kCtI64;
    case SB_F16: case SB_BF16: case SB_F32: return kCtF32;
    case SB_F64: return kCtF64;
    default: return -1;
  }
}

// Alignment (bytes) a vector access of kEwVec elements of this dtype needs.
size_t vec_align(int dtype) {
  const size_t bytes = static_cast<size_t>(dtype_size(dtype)) * kEwVec;
  return bytes >= 16 ? 16 : bytes;
}

bool aligned_for_vec(const sb_ew_desc* d, int k) {
  const size_t a = vec_align(d->dtype[k]);
  if (reinterpret_cast<uintptr_t>(d->data[k]) % a) return false;
  const size_t es = dtype_size(d->dtype[k]);
  for (int i = 1; i < d->ndim; ++i)
    if ((static_cast<uint64_t>(d->strides[k][i] < 0 ? -d->strides[k][i] : d->strides[k][i]) * es) % a) return false;
  return true;
}

}  // namespace

int ew_make_plan(const sb_ew_desc* d, EwPlan* plan) {
  if (!d || !plan) return SB_ERR_INVALID_ARGUMENT;
  if (d->op < 0 || d->op >= SB_EW_OP_COUNT) return SB_ERR_INVALID_ARGUMENT;
  if (d->ndim < 1 || d->ndim > SB_MAX_DIMS) return SB_ERR_INVALID_ARGUMENT;
  const int arity = ew_arity(d->op);
  if (d->noperands != arity + 1) return SB_ERR_INVALID_ARGUMENT;
  int64_t numel = 1;
  for (int i = 0; i < d->ndim; ++i) {
    if (d->sizes[i] < 0) return SB_ERR_INVALID_ARGUMENT;
    if (d->sizes[i] != 0 && numel > INT64_MAX / d->sizes[i]) return SB_ERR_TOO_LARGE;
    numel *= d->sizes[i];
  }
  for (int k = 0; k < d->noperands; ++k) {
    if (d->dtype[k] < 0 || d->dtype[k] >= SB_DTYPE_COUNT) return SB_ERR_UNSUPPORTED;
    if (numel > 0 && !d->data[k]) return SB_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(d->data[k]) % dtype_size(d->dtype[k])) return SB_ERR_MISALIGNED;
  }
  plan->compute = compute_type_of(d->common_dtype);
  if (plan->compute < 0) return SB_ERR_UNSUPPORTED;
  if (ew_float_only(d->op) && plan->compute != kCtF32 && plan->compute != kCtF64) return SB_ERR_UNSUPPORTED;
  plan->fast = d->common_dtype == SB_BF16 && d->dtype[0] == SB_BF16;
  plan->static_dtype = -1;
  if (d->common_dtype == SB_F32 || d->common_dtype == SB_BF16 || d->common_dtype == SB_F16) {
    bool same = true;
    for (int k = 0; k < d->noperands; ++k) same = same && d->dtype[k] == d->common_dtype;
    if (same) plan->static_dtype = d->common_dtype;
  }
  plan->transposed_mask = 0;
  plan->transpose_vec = false;
  plan->outer = 0;
  plan->path = 3;
  if (numel == 0) return SB_OK;

  // stride of the output along the fastest dimension must be 1 for the vector and tile paths
  const bool out_unit = d->strides[0][0] == 1 || d->sizes[0] == 1;
  bool sizes_fit32 = true;
  for (int i = 0; i < d->ndim; ++i) sizes_fit32 = sizes_fit32 && d->sizes[i] <= 0xffffffffLL;
  if (!sizes_fit32) {
    // only a dense 1-D run may be that long
    bool dense = d->ndim == 1;
    for (int k = 0; k < d->noperands && dense; ++k) dense = d->strides[k][0] == 1;
    if (!dense) return SB_ERR_TOO_LARGE;
  }

  if (d->ndim == 1) {
    bool all_unit = true, vec_ok = true;
    for (int k = 0; k < d->noperands; ++k) {
      all_unit = all_unit && (d->strides[k][0] == 1 || d->sizes[0] == 1);
      vec_ok = vec_ok && aligned_for_vec(d, k);
    }
    if (all_unit && vec_ok) {
      plan->path = 0;
      return SB_OK;
    }
  }
  if (out_unit && d->ndim <= kEwRowDims && d->sizes[0] <= 0x7fffffffLL) {
    bool ok = aligned_for_vec(d, 0);
    for (int k = 1; k < d->noperands && ok; ++k) {
      const int64_t s0 = d->sizes[0] == 1 ? 1 : d->strides[k][0];
      ok = (s0 == 1 && aligned_for_vec(d, k)) || s0 == 0;
    }
    uint64_t rows = 1;
    for (int i = 1; i < d->ndim; ++i) rows *= static_cast<uint64_t>(d->sizes[i]);
    if (ok && rows <= 0xffffffffULL) {
      plan->path = 1;
      // outer-broadcast form: two inputs, whole vectors only, each input constant along a different one of dims 1, 2
      if (d->noperands == 3 && ew_arity(d->op) == 2 && d->ndim >= 3 && d->sizes[0] % kEwVec == 0 && d->strides[1][0] == 1 &&
          d->strides[2][0] == 1 && d->sizes[1] >= 4 && d->sizes[2] >= 4) {
        if (d->strides[1][1] == 0 && d->strides[2][2] == 0) plan->outer = 1;
        else if (d->strides[2][1] == 0 && d->strides[1][2] == 0) plan->outer = 2;
      }
      return SB_OK;
    }
  }
  if (out_unit && d->ndim >= 2) {
    bool ok = true;
    uint32_t mask = 0;
    for (int k = 1; k < d->noperands; ++k) {
      const int64_t s0 = d->strides[k][0], s1 = d->strides[k][1];
      if (s0 == 1 || s0 == 0) continue;
      if (s1 == 1) mask |= 1u << (k - 1);
      else ok = false;
    }
    uint64_t outer = 1;
    for (int i = 2; i < d->ndim; ++i) outer *= static_cast<uint64_t>(d->sizes[i]);
    if (ok && mask && outer <= 65535 && (d->sizes[1] + 31) / 32 <= 65535 && (d->sizes[0] + 31) / 32 <= 0x7fffffffLL) {
      plan->path = 2;
      plan->transposed_mask = mask;
      // 4-element accesses: sizes multiples of 4 and every access 4-element aligned
      bool vec = d->sizes[0] % 4 == 0 && d->sizes[1] % 4 == 0 && d->noperands <= 3;  // the vector kernel holds two inputs
      for (int k = 0; k < d->noperands && vec; ++k) {
        const size_t es = dtype_size(d->dtype[k]);
        const size_t a = es * 4 >= 16 ? 16 : es * 4;
        vec = reinterpret_cast<uintptr_t>(d->data[k]) % a == 0;
        const bool transposed = k >= 1 && (mask >> (k - 1) & 1);
        for (int i = 0; i < d->ndim && vec; ++i) {
          const bool unit_dim = transposed ? i == 1 : i == 0;
          if (unit_dim) continue;
          const int64_t st = d->strides[k][i] < 0 ? -d->strides[k][i] : d->strides[k][i];
          vec = (static_cast<uint64_t>(st) * es) % a == 0;
        }
      }
      plan->transpose_vec = vec;
      return SB_OK;
    }
  }
  plan->path = 3;
  return SB_OK;
}

void ew_fill_params(const sb_ew_desc* d, EwParams* p) {
  int64_t numel = 1;
  for (int i = 0; i < kEwRowDims; ++i) {
    const int64_t s = i < d->ndim ? d->sizes[i] : 1;
    p->sizes[i] = static_cast<uint32_t>(s);
    numel *= s;
  }
  for (int i = kEwRowDims; i < d->ndim; ++i) numel *= d->sizes[i];
  p->numel = numel;
  for (int k = 0; k < SB_MAX_OPERANDS; ++k) {
    p->data[k] = k < d->noperands ? d->data[k] : nullptr;
    p->dtype[k] = k < d->noperands ? d->dtype[k] : SB_F32;
    for (int i = 0; i < kEwRowDims; ++i)
      p->strides[k][i] = (k < d->noperands && i < d->ndim) ? (d->sizes[i] == 1 && i == 0 ? 1 : d->strides[k][i]) : 0;
  }
  p->row_chunks = 1;
  p->span = 0;
  p->bcast = 0;
  p->rows = 1;
  p->bx = kEwThreads;
  p->unroll = 1;
  p->op = d->op;
  p->alpha = d->alpha;
  p->scalar = d->scalar;
  p->ialpha = d->ialpha;
  p->iscalar = d->iscalar;
}

void ew_fill_generic(const sb_ew_desc* d, EwGenericParams* g) {
  g->ndim = d->ndim;
  g->noperands = d->noperands;
  g->op = d->op;
  int64_t numel = 1;
  for (int i = 0; i < SB_MAX_DIMS; ++i) {
    g->sizes[i] = i < d->ndim ? static_cast<uint32_t>(d->sizes[i]) : 1;
    if (i < d->ndim) numel *= d->sizes[i];
  }
  g->numel = numel;
  for (int k = 0; k < SB_MAX_OPERANDS; ++k) {
    g->data[k] = k < d->noperands ? d->data[k] : nullptr;
    g->dtype[k] = k < d->noperands ? d->dtype[k] : SB_F32;
    for (int i = 0; i < SB_MAX_DIMS; ++i) g->strides[k][i] = (k < d->noperands && i < d->ndim) ? d->strides[k][i] : 0;
  }
  g->alpha = d->alpha;
  g->scalar = d->scalar;
  g->ialpha = d->ialpha;
  g->iscalar = d->iscalar;
}

int ew_rows_geometry(const sb_ew_desc* d, EwParams* p, unsigned* grid) {
  const uint64_t n0 = p->sizes[0];
  const uint64_t nv0 = (n0 + kEwVec - 1) / kEwVec;
  uint64_t rows = 1;
  for (int i = 1; i < d->ndim; ++i) rows *= static_cast<uint64_t>(d->sizes[i]);
  const int arity = ew_arity(d->op);
  const int unroll = arity <= 1 ? 4 : 2;
  // threads along the row: each thread should walk about four passes of `unroll` vectors, so that the row
  // decomposition it does once is amortised; short rows get fewer threads and the block takes several rows
  int bx = 1;
  while (bx < kEwThreads && static_cast<uint64_t>(bx) * 2 * unroll * 4 <= nv0) bx <<= 1;
  if (static_cast<uint64_t>(bx) * unroll < nv0 && bx < 8) bx = 8;
  const uint64_t by = kEwThreads / bx;
  const uint64_t row_blocks = (rows + by - 1) / by;
  // long rows and few of them: cut each row into chunks so that every SM gets work
  uint64_t chunks = 1;
  const uint64_t want_blocks = 4ull * static_cast<uint64_t>(sm_count());
  const uint64_t per_pass = static_cast<uint64_t>(bx) * unroll;
  if (row_blocks < want_blocks && nv0 > 4 * per_pass) {
    chunks = (want_blocks + row_blocks - 1) / row_blocks;
    const uint64_t max_chunks = nv0 / (2 * per_pass);
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
  }
  uint64_t span = (nv0 + chunks - 1) / chunks;
  span = (span + per_pass - 1) / per_pass * per_pass;
  chunks = (nv0 + span - 1) / span;
  const uint64_t blocks = row_blocks * chunks;
  if (blocks > 0x7fffffffULL || rows > 0xffffffffULL) return SB_ERR_TOO_LARGE;
  bool bcast = false;
  for (int k = 1; k < d->noperands; ++k) bcast = bcast || (p->strides[k][0] == 0);
  p->bx = bx;
  p->unroll = unroll;
  p->row_chunks = static_cast<uint32_t>(chunks);
  p->span = static_cast<uint32_t>(span);
  p->rows = static_cast<uint32_t>(rows);
  p->bcast = bcast ? 1 : 0;
  *grid = static_cast<unsigned>(blocks);
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_elementwise(const sb_ew_desc* d, sb_stream_t stream) {
  EwPlan plan;
  int rc = ew_make_plan(d, &plan);
  if (rc != SB_OK) return rc;
  for (int i = 0; i < d->ndim; ++i)
    if (d->sizes[i] == 0) return SB_OK;
  cudaStream_t st = as_stream(stream);
  switch (plan.compute) {
    case kCtF32: return ew_launch_f32(d, plan, st);
    case kCtF64: return ew_launch_f64(d, plan, st);
    default: return ew_launch_int(d, plan, st);
  }
}

int sb_elementwise_path(const sb_ew_desc* d) {
  EwPlan plan;
  int rc = ew_make_plan(d, &plan);
  return rc != SB_OK ? rc : plan.path;
}

}  // extern "C"

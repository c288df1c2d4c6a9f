// Cross-entropy kernel selection (and, below, the shared-memory-resident variant).
#include "ce_common.cuh"

namespace sb {

int ce_choose_variant(int dtype, int64_t rows, int64_t classes, const void* logits, const void* grad) {
  (void)dtype; (void)rows; (void)classes; (void)logits; (void)grad;
  return 0;
}

int ce_launch_resident(const CEParams&, cudaStream_t, int) { return SB_ERR_UNSUPPORTED; }

int ce_dispatch(const CEParams& p, cudaStream_t st) {
  const int variant = ce_choose_variant(p.dtype, p.rows, p.classes, p.logits, p.grad);
  if (variant == 0) return ce_launch_generic(p, st);
  return ce_launch_resident(p, st, variant);
}

}  // namespace sb

extern "C" int sb_ce_kernel_variant(int32_t dtype, int64_t rows, int64_t classes) {
  return sb::ce_choose_variant(dtype, rows, classes, nullptr, nullptr);
}

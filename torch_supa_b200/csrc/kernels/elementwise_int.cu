// Elementwise launchers whose arithmetic runs in an integer type or bool.  Integer results wrap
// (two's complement), which is what the narrower storage types see after truncation.
#include "elementwise.cuh"

namespace sb {

namespace {
template <typename CT>
int launch_ct(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st) {
  if (plan.path >= 2) return ew_launch_scalar_paths<CT>(d, plan, st);
  switch (d->op) {
#define SB_CASE(OPCODE) case OPCODE: return ew_launch_vector<OPCODE, CT, false, DynamicIO>(d, plan, st);
    SB_CASE(SB_EW_COPY) SB_CASE(SB_EW_FILL) SB_CASE(SB_EW_ADD) SB_CASE(SB_EW_MUL) SB_CASE(SB_EW_SUB)
    SB_CASE(SB_EW_ADD_SCALAR) SB_CASE(SB_EW_MUL_SCALAR) SB_CASE(SB_EW_NEG)
    SB_CASE(SB_EW_MAXIMUM) SB_CASE(SB_EW_MINIMUM) SB_CASE(SB_EW_EQ) SB_CASE(SB_EW_NE) SB_CASE(SB_EW_LT) SB_CASE(SB_EW_LE) SB_CASE(SB_EW_GT)
    SB_CASE(SB_EW_GE) SB_CASE(SB_EW_WHERE) SB_CASE(SB_EW_MASKED_FILL) SB_CASE(SB_EW_DIV_TRUNC) SB_CASE(SB_EW_DIV_FLOOR)
#undef SB_CASE
    default: return SB_ERR_UNSUPPORTED;
  }
}
}  // namespace

int ew_launch_int(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st) {
  switch (plan.compute) {
    case kCtBool: return launch_ct<bool>(d, plan, st);
    case kCtI32: return launch_ct<int32_t>(d, plan, st);
    case kCtI64: return launch_ct<int64_t>(d, plan, st);
    default: return SB_ERR_UNSUPPORTED;
  }
}

}  // namespace sb

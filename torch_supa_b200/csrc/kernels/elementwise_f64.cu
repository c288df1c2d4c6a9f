// Elementwise launchers whose arithmetic runs in fp64.
#include "elementwise.cuh"

namespace sb {

int ew_launch_f64(const sb_ew_desc* d, const EwPlan& plan, cudaStream_t st) {
  if (plan.path >= 2) return ew_launch_scalar_paths<double>(d, plan, st);
  switch (d->op) {
#define SB_CASE(OPCODE) case OPCODE: return ew_launch_vector<OPCODE, double, false, DynamicIO>(d, plan, st);
    SB_CASE(SB_EW_COPY) SB_CASE(SB_EW_FILL) SB_CASE(SB_EW_ADD) SB_CASE(SB_EW_MUL) SB_CASE(SB_EW_SUB) SB_CASE(SB_EW_DIV)
    SB_CASE(SB_EW_GELU_ERF) SB_CASE(SB_EW_GELU_TANH) SB_CASE(SB_EW_SILU) SB_CASE(SB_EW_GLU) SB_CASE(SB_EW_GELU_ERF_BWD)
    SB_CASE(SB_EW_GELU_TANH_BWD) SB_CASE(SB_EW_SILU_BWD) SB_CASE(SB_EW_GLU_BWD_A) SB_CASE(SB_EW_GLU_BWD_B)
    SB_CASE(SB_EW_ADD_SCALAR) SB_CASE(SB_EW_MUL_SCALAR) SB_CASE(SB_EW_NEG)
    SB_CASE(SB_EW_BCE_LOGITS) SB_CASE(SB_EW_BCE_LOGITS_PW) SB_CASE(SB_EW_BCE_LOGITS_BWD) SB_CASE(SB_EW_BCE_LOGITS_PW_BWD)
    SB_CASE(SB_EW_SIGMOID) SB_CASE(SB_EW_TANH) SB_CASE(SB_EW_EXP) SB_CASE(SB_EW_LOG) SB_CASE(SB_EW_SIGMOID_BWD) SB_CASE(SB_EW_TANH_BWD)
    SB_CASE(SB_EW_MAXIMUM) SB_CASE(SB_EW_MINIMUM) SB_CASE(SB_EW_EQ) SB_CASE(SB_EW_NE) SB_CASE(SB_EW_LT) SB_CASE(SB_EW_LE) SB_CASE(SB_EW_GT)
    SB_CASE(SB_EW_GE) SB_CASE(SB_EW_WHERE) SB_CASE(SB_EW_MASKED_FILL) SB_CASE(SB_EW_DIV_TRUNC) SB_CASE(SB_EW_DIV_FLOOR)
#undef SB_CASE
    default: return SB_ERR_UNSUPPORTED;
  }
}

}  // namespace sb

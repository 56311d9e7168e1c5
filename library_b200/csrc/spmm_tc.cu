// tcgen05 tensor-core SpMM variant (bf16 A and B, fp32 C).  Placeholder translation unit
// until the kernel lands: reports the variant as not applicable.
#include "asp_internal.h"

namespace asp {
void free_spmm_tc_plan(void*) {}
bool spmm_tc_applicable(alphasparseSpMatDescr_t, alphasparseDnMatDescr_t, alphasparseDnMatDescr_t) {
  return false;
}
alphasparseStatus_t spmm_tc_run(alphasparseHandle_t, alphasparseSpMatDescr_t, alphasparseDnMatDescr_t,
                                alphasparseDnMatDescr_t, float, float, bool) {
  return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
}  // namespace asp

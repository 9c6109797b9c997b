// Tensor-core (tcgen05, kind::tf32) gather-GEMM.  Not built yet: every shape reports "not handled"
// and the caller runs the fp32 kernel instead.
#include "internal.h"

namespace scn {

int gather_gemm_tf32(const float *, int64_t, const int32_t *, int, int64_t, const float *, const float *, float *,
                     int64_t, int64_t, int64_t, int, cudaStream_t, bool *handled) {
  *handled = false;
  return SCN_OK;
}

}  // namespace scn

// One-pass cross-entropy with the row staged in shared memory across a thread-block cluster.
#include "common.cuh"

namespace mdy {

int ce_fused_cluster(const void*, void*, const int64_t*, float*, float*, const float*, float, int64_t,
                     int64_t, int64_t, int, cudaStream_t) {
  return MDY_ERR_UNSUPPORTED;
}

}  // namespace mdy

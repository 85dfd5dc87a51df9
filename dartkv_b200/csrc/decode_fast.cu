// Tensor-core decode kernel for the headline page geometry (placeholder until the kernel lands).
#include "common.cuh"

int dartkv_decode_fast_supported(const dartkv_cache_desc*, int, int) { return 0; }
int dartkv_decode_fast_launch(const dartkv_cache_desc*, const void*, int, int, float, int, int, int, int, int, float*,
                              float*, float*, cudaStream_t) {
  dartkv_set_error("fast decode kernel not built");
  return DARTKV_EINVAL;
}

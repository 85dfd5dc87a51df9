// Page-shaped quantize+pack kernels for the headline geometry (placeholder until the kernels land).
#include "common.cuh"

int dartkv_append_fast_supported(const dartkv_cache_desc*, const dartkv_append_plan*, int64_t) { return 0; }
int dartkv_append_fast(const dartkv_cache_desc*, const dartkv_append_plan*, const void*, const void*, int64_t, int64_t,
                       int64_t, const int32_t*, int32_t*, cudaStream_t) {
  dartkv_set_error("fast append kernels not built");
  return DARTKV_EINVAL;
}

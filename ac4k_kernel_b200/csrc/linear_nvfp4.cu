// placeholder until the tcgen05 GEMM lands
#include "common.cuh"
extern "C" int ac4k_linear_nvfp4(void *, int, const void *, const void *, const float *, const void *,
                                 const void *, const float *, const void *, int, int64_t, int64_t, int64_t,
                                 int, ac4k_stream_t) {
  return ac4k::fail(AC4K_ERR_UNSUPPORTED, "linear_nvfp4 not built yet");
}

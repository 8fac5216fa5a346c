// Library identity, error reporting and the device status word of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace ac4k {

__device__ unsigned int g_device_status = 0;

static thread_local char t_last_error[512] = "";

void set_last_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  snprintf(t_last_error, sizeof(t_last_error), "%s: %s (%s)", what, cudaGetErrorString(e),
           cudaGetErrorName(e));
  return (int)e > 0 ? (int)e : 999;
}

unsigned int *device_status_ptr() {
  static PerDevice<unsigned int *> cache;
  unsigned int *ptr = nullptr;
  const int rc = cache.get(&ptr, [](unsigned int *&v) {
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_device_status);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_device_status)");
    v = static_cast<unsigned int *>(p);
    return 0;
  });
  return rc == 0 ? ptr : nullptr;
}

}  // namespace ac4k

extern "C" const char *ac4k_arch(void) { return "sm100"; }
extern "C" const char *ac4k_arch_description(void) { return "NVIDIA Blackwell (B200/B100)"; }
extern "C" const char *ac4k_backend(void) { return "cuda"; }
extern "C" const char *ac4k_version(void) { return "0.1.0"; }
extern "C" const char *ac4k_last_error(void) { return ac4k::t_last_error; }

extern "C" int ac4k_device_status(uint32_t *status_out, int clear) {
  if (!status_out) return ac4k::fail(AC4K_ERR_NULL, "status_out is NULL");
  unsigned int v = 0;
  AC4K_CUDA_TRY(cudaDeviceSynchronize());
  AC4K_CUDA_TRY(cudaMemcpyFromSymbol(&v, ac4k::g_device_status, sizeof(v)));
  *status_out = v;
  if (clear && v != 0) {
    unsigned int z = 0;
    AC4K_CUDA_TRY(cudaMemcpyToSymbol(ac4k::g_device_status, &z, sizeof(z)));
  }
  if (v >= 0xA1 && v <= 0xA4) {
    static const char *role[] = {"TMA producer", "MMA issuer", "scale warps", "epilogue"};
    return ac4k::fail(AC4K_ERR_TIMEOUT, "a bounded device-side wait expired in a GEMM launched earlier (%s, status 0x%X); "
                                        "the outputs of that launch are undefined", role[v - 0xA1], v);
  }
  return 0;
}

/* A plain C translation unit that uses the library through include/ac4k_b200.h only: the header must
 * be valid C, every declared entry point must link, and argument errors must come back as negative
 * codes with a message.  No GPU is touched (every call below is rejected before any CUDA call). */
#include <stdio.h>
#include <string.h>

#include "ac4k_b200.h"

int main(void) {
  int failures = 0;
  int64_t shape[4] = {1, 1, 16, 64};
  int64_t stride[4] = {0, 0, 64, 1};
  void *fake = (void *)(uintptr_t)4096; /* aligned, never dereferenced */
  void *dsts[2];
  void *ptr = NULL;
  unsigned char handle[64];

  if (strcmp(ac4k_arch(), "sm100") != 0) { printf("arch: %s\n", ac4k_arch()); ++failures; }
  if (strcmp(ac4k_backend(), "cuda") != 0) ++failures;
  if (ac4k_version()[0] == 0 || ac4k_arch_description()[0] == 0) ++failures;

  if (ac4k_quantize_nvfp4(NULL, NULL, NULL, NULL, shape, stride, 0, AC4K_SF_AC4K, NULL) != AC4K_ERR_NULL) ++failures;
  if (strstr(ac4k_last_error(), "NULL") == NULL) ++failures;
  if (ac4k_quantize_nvfp4(fake, fake, fake, (const float *)fake, shape, stride, 0, 7, NULL) != AC4K_ERR_ENUM) ++failures;
  if (ac4k_quantize_fp8(NULL, NULL, NULL, NULL, NULL, NULL, 0, NULL) >= 0) ++failures;
  if (ac4k_quantize_int8(NULL, NULL, NULL, NULL, NULL, NULL, NULL) >= 0) ++failures;
  if (ac4k_global_scale_bf16(NULL, -1, 1.0f, (float *)fake, NULL) != AC4K_ERR_SHAPE) ++failures;
  if (ac4k_linear_nvfp4(fake, AC4K_DT_BF16, fake, fake, (const float *)fake, fake, fake, (const float *)fake, NULL, 0,
                        8, 8, 80, AC4K_SF_TILE128X4, NULL) != AC4K_ERR_SHAPE) ++failures;
  if (ac4k_linear_nvfp4_noalloc(NULL, AC4K_DT_BF16, fake, fake, (const float *)fake, fake, fake, (const float *)fake,
                                NULL, 0, 8, 8, 64, AC4K_SF_TILE128X4, NULL) != AC4K_ERR_NULL) ++failures;
  dsts[0] = fake; dsts[1] = fake;
  if (ac4k_linear_nvfp4_gather(dsts, 9, 64, 0, AC4K_DT_BF16, fake, fake, (const float *)fake, fake, fake,
                               (const float *)fake, NULL, 0, 8, 64, 64, AC4K_SF_TILE128X4, NULL) != AC4K_ERR_SHAPE) ++failures;
  if (ac4k_linear_nvfp4_requant(fake, fake, (const float *)fake, AC4K_SF_TILE128X4, fake, fake, (const float *)fake, fake,
                                fake, (const float *)fake, NULL, 0, 8, 96, 64, AC4K_SF_TILE128X4, NULL) != AC4K_ERR_UNSUPPORTED)
    ++failures;
  if (ac4k_peer_alloc(0, &ptr, handle) != AC4K_ERR_SHAPE) ++failures;
  if (ac4k_peer_open(NULL, &ptr) != AC4K_ERR_NULL) ++failures;
  if (ac4k_peer_close(NULL) != 0 || ac4k_peer_free(NULL) != 0) ++failures;
  /* ac4k_device_status needs a device: only its address is taken here, so that it must link */
  {
    int (*volatile fn)(uint32_t *, int) = ac4k_device_status;
    if (fn == NULL) ++failures;
  }

  printf(failures ? "FAILED: %d\n" : "ok\n", failures);
  return failures;
}

// Test infrastructure, not product code: a pybind11 module around the reference's own quantiser and RoPE kernels
// (its lib/cuda/sm120/quantize_nvfp4.cu, quantize_fp8.cu, quantize_int8.cu and rope3d.cu, compiled unchanged from
// the reference checkout by oracle/build_ref.py for sm_100a; its GEMM and attention kernels use sm_120a-only MMAs
// and cannot be built for a B200).  The functions are the ones its own binding exports (lib/cuda_bindings.cc:61-97,
// declared in include/ac4k_kernel/ops.h:27-66), under the same names, so that a test can run the reference's kernel
// and this repository's on the same device tensors and compare bytes and times.
#include <torch/extension.h>

#include "ac4k_kernel/ops.h"

PYBIND11_MODULE(_ac4k_ref, m) {
  m.doc() = "the reference's quantiser and RoPE kernels, compiled for sm_100a (test-side comparator)";
  m.def("quantize_nvfp4", &ac4k::quantize_nvfp4);
  m.def("quantize_fp8", &ac4k::quantize_fp8);
  m.def("quantize_int8", &ac4k::quantize_int8);
  m.def("rope3d", &ac4k::rope3d);
}

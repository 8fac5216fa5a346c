// The compiled `_cuda_ops` module over the C ABI: the translation unit a maintainer of ac4k_kernel would add
// as lib/cuda/sm100/bindings_sm100.cc.  Same module name, function names, positional signatures and module
// attributes as the reference's lib/cuda_bindings.cc:37-97 (prototypes: include/ac4k_kernel/ops.h:13-54);
// the argument checks are the TORCH_CHECKs of the reference's host launchers, the launch is a call into
// libac4k_b200.so with raw pointers and the current CUDA stream.
//
// Built by ac4k_kernel_b200/build.py (build_pybind) with the host compiler; no CUDA source is involved.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <vector>

#include "ac4k_b200.h"

namespace ac4k {

static int64_t align_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }
static int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

static void check_cuda(const torch::Tensor &t, at::ScalarType dt, const char *name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == dt, "Inconsistency of Tensor type: ", name);
}

// sizes and element strides ordered [outer0, outer1, cross, reduce], rank padded to 4 with leading 1s
// (quantize_nvfp4.cu:226-241)
static std::vector<int> view4(const torch::Tensor &in, uint32_t cross, uint32_t reduce, int64_t shape[4], int64_t stride[4]) {
  std::vector<int> others;
  for (int i = 0; i < in.dim(); ++i)
    if (i != (int)cross && i != (int)reduce) others.push_back(i);
  int o = 2 - (int)others.size();
  for (int i = 0; i < o; ++i) { shape[i] = 1; stride[i] = 0; }
  for (int i : others) { shape[o] = in.size(i); stride[o] = in.stride(i); ++o; }
  shape[2] = in.size(cross);  stride[2] = in.stride(cross);
  shape[3] = in.size(reduce); stride[3] = in.stride(reduce);
  return others;
}

static std::vector<int> check_quant_common(const torch::Tensor &out, const torch::Tensor &in, uint32_t cross_dim,
                                           uint32_t reduce_dim, int reduce_align, int reduce_div, int64_t shape[4],
                                           int64_t stride[4]) {
  TORCH_CHECK(in.dim() >= 2 && in.dim() <= 4, "in must be 2-4D");
  TORCH_CHECK(cross_dim < (uint32_t)in.dim(), "cross_dim must be less than in.dim()");
  TORCH_CHECK(reduce_dim < (uint32_t)in.dim(), "reduce_dim must be less than in.dim()");
  TORCH_CHECK(cross_dim != reduce_dim, "cross_dim and reduce_dim must be different");
  TORCH_CHECK(out.dim() == in.dim(), "out must be the same dim as in");
  std::vector<int> others = view4(in, cross_dim, reduce_dim, shape, stride);
  for (size_t c = 0; c < others.size(); ++c) TORCH_CHECK(out.size(c) == in.size(others[c]), "out must be the same shape as in");
  TORCH_CHECK(out.size(-2) == shape[2], "meet invalid cross dim size");
  TORCH_CHECK(out.size(-1) == align_up(shape[3], reduce_align) / reduce_div, "meet invalid reduce dim size");
  return others;
}

// ops.h:27-29; checks of quantize_nvfp4.cu:171-224
void quantize_nvfp4(torch::Tensor &out, torch::Tensor &sf, torch::Tensor const &in, torch::Tensor const &global_scale,
                    uint32_t cross_dim, uint32_t reduce_dim, bool swizzle) {
  check_cuda(in, at::kBFloat16, "in");
  check_cuda(global_scale, at::kFloat, "global_scale");
  TORCH_CHECK(global_scale.dim() == 0, "global_scale must be a scalar");
  check_cuda(out, at::kByte, "out");
  check_cuda(sf, at::kFloat8_e4m3fn, "sf");
  int64_t shape[4], stride[4];
  std::vector<int> others = check_quant_common(out, in, cross_dim, reduce_dim, 64, 2, shape, stride);
  const int64_t kt = ceil_div(shape[3], 64);
  std::vector<int64_t> want;
  for (int i : others) want.push_back(in.size(i));
  int layout;
  if (sf.dim() == in.dim() + 1) {
    layout = AC4K_SF_AC4K;
    want.insert(want.end(), {kt, align_up(shape[2], 16), 4});
  } else if (sf.dim() == in.dim() + 3) {
    layout = AC4K_SF_TILE128X4;
    want.insert(want.end(), {ceil_div(shape[2], 128), kt, 32, 4, 4});
  } else {
    TORCH_CHECK(false, "meet invalid sf rank");
  }
  TORCH_CHECK(sf.sizes().vec() == want, "meet invalid sf shape");
  c10::cuda::CUDAGuard guard(in.device());
  const int rc = ac4k_quantize_nvfp4(out.data_ptr(), sf.data_ptr(), in.data_ptr(), global_scale.data_ptr<float>(), shape,
                                     stride, swizzle ? 1 : 0, layout, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_quantize_nvfp4: ", ac4k_last_error());
}

// ops.h:31-33; checks of quantize_fp8.cu:196-247
void quantize_fp8(torch::Tensor &out, torch::Tensor &sf, torch::Tensor const &in, torch::Tensor const &scale_max,
                  uint32_t cross_dim, uint32_t reduce_dim, bool swizzle) {
  check_cuda(in, at::kBFloat16, "in");
  check_cuda(scale_max, at::kFloat, "scale_max");
  TORCH_CHECK(scale_max.dim() == 0, "scale_max must be a scalar");
  check_cuda(out, at::kFloat8_e4m3fn, "out");
  check_cuda(sf, at::kFloat, "sf");
  int64_t shape[4], stride[4];
  std::vector<int> others = check_quant_common(out, in, cross_dim, reduce_dim, 16, 1, shape, stride);
  TORCH_CHECK(sf.dim() == in.dim() - 1, "meet invalid sf rank");
  std::vector<int64_t> want;
  for (int i : others) want.push_back(in.size(i));
  want.push_back(align_up(shape[2], 16));
  TORCH_CHECK(sf.sizes().vec() == want, "meet invalid sf shape");
  c10::cuda::CUDAGuard guard(in.device());
  const int rc = ac4k_quantize_fp8(out.data_ptr(), sf.data_ptr<float>(), in.data_ptr(), scale_max.data_ptr<float>(), shape,
                                   stride, swizzle ? 1 : 0, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_quantize_fp8: ", ac4k_last_error());
}

// ops.h:35-37; checks of quantize_int8.cu:179-230
void quantize_int8(torch::Tensor &out, torch::Tensor &sf, torch::Tensor const &in, torch::Tensor const &scale_max,
                   uint32_t cross_dim, uint32_t reduce_dim) {
  check_cuda(in, at::kBFloat16, "in");
  check_cuda(scale_max, at::kInt, "scale_max");
  TORCH_CHECK(scale_max.dim() == 0, "scale_max must be a scalar");
  check_cuda(out, at::kChar, "out");
  check_cuda(sf, at::kFloat, "sf");
  int64_t shape[4], stride[4];
  std::vector<int> others = check_quant_common(out, in, cross_dim, reduce_dim, 16, 1, shape, stride);
  TORCH_CHECK(sf.dim() == in.dim() - 1, "meet invalid sf rank");
  std::vector<int64_t> want;
  for (int i : others) want.push_back(in.size(i));
  want.push_back(align_up(shape[2], 16));
  TORCH_CHECK(sf.sizes().vec() == want, "meet invalid sf shape");
  c10::cuda::CUDAGuard guard(in.device());
  const int rc = ac4k_quantize_int8(out.data_ptr(), sf.data_ptr<float>(), in.data_ptr(), scale_max.data_ptr<int32_t>(), shape,
                                    stride, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_quantize_int8: ", ac4k_last_error());
}

static int dtype_code(at::ScalarType t, const char *what) {
  TORCH_CHECK(t == at::kBFloat16 || t == at::kHalf || t == at::kFloat, what, " must be bfloat16, half or float");
  return t == at::kBFloat16 ? AC4K_DT_BF16 : (t == at::kHalf ? AC4K_DT_FP16 : AC4K_DT_FP32);
}

// ops.h:43-48; checks of linear_nvfp4.cu:759-805
void linear_nvfp4(torch::Tensor &D, torch::Tensor const &A, torch::Tensor const &A_sf, torch::Tensor const &A_global_scale,
                  torch::Tensor const &B, torch::Tensor const &B_sf, torch::Tensor const &B_global_scale,
                  c10::optional<torch::Tensor> const &bias) {
  TORCH_CHECK(D.dim() == 2, "d must be a 2d matrix");
  const int64_t M = D.size(0), N = D.size(1);
  const int d_dt = dtype_code(D.scalar_type(), "d");
  TORCH_CHECK(D.is_cuda() && D.is_contiguous(), "d must be contiguous");
  TORCH_CHECK(A.dim() == 2, "a must be a 2d matrix");
  check_cuda(A, at::kByte, "a");
  TORCH_CHECK(A.size(0) == M, "A size(0) must be ", M, " but see ", A.size(0));
  const int64_t K = A.size(1) * 2;
  TORCH_CHECK(K % 16 == 0, "A size(1)*2 must be multiple of 16 but see ", K);
  TORCH_CHECK(B.dim() == 2, "b must be a 2d matrix");
  check_cuda(B, at::kByte, "b");
  TORCH_CHECK(B.size(0) == N, "B size(0) must be ", N, " but see ", B.size(0));
  TORCH_CHECK(B.size(1) == A.size(1), "B size(1) must equal A size(1)");
  const int64_t kt = ceil_div(K, 64);
  check_cuda(A_sf, at::kFloat8_e4m3fn, "scale_a");
  check_cuda(B_sf, at::kFloat8_e4m3fn, "scale_b");
  int layout;
  if (A_sf.dim() == 3) {
    layout = AC4K_SF_AC4K;
    TORCH_CHECK(A_sf.sizes().vec() == std::vector<int64_t>({kt, align_up(M, 16), 4}), "scale_a has an invalid shape");
    TORCH_CHECK(B_sf.sizes().vec() == std::vector<int64_t>({kt, align_up(N, 16), 4}), "scale_b has an invalid shape");
  } else {
    TORCH_CHECK(A_sf.dim() == 5, "scale_a must be a 3d matrix");
    layout = AC4K_SF_TILE128X4;
    TORCH_CHECK(A_sf.sizes().vec() == std::vector<int64_t>({ceil_div(M, 128), kt, 32, 4, 4}), "scale_a has an invalid shape");
    TORCH_CHECK(B_sf.sizes().vec() == std::vector<int64_t>({ceil_div(N, 128), kt, 32, 4, 4}), "scale_b has an invalid shape");
  }
  check_cuda(A_global_scale, at::kFloat, "global_scale_a");
  TORCH_CHECK(A_global_scale.dim() == 0, "A_global_scale must be a scalar");
  check_cuda(B_global_scale, at::kFloat, "global_scale_b");
  TORCH_CHECK(B_global_scale.dim() == 0, "B_global_scale must be a scalar");
  const void *bias_ptr = nullptr;
  int bias_dt = 0;
  if (bias.has_value()) {
    bias_dt = dtype_code(bias->scalar_type(), "bias");
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous(), "bias must be contiguous");
    TORCH_CHECK(bias->dim() == 2, "bias must be a 2d matrix");
    TORCH_CHECK(bias->size(0) == 1, "bias shape[0] must be 1");
    TORCH_CHECK(bias->size(1) == N, "bias shape[1] must be ", N);
    bias_ptr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(D.device());
  const int rc = ac4k_linear_nvfp4(D.data_ptr(), d_dt, A.data_ptr(), A_sf.data_ptr(), A_global_scale.data_ptr<float>(),
                                   B.data_ptr(), B_sf.data_ptr(), B_global_scale.data_ptr<float>(), bias_ptr, bias_dt, M, N, K,
                                   layout, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_linear_nvfp4: ", ac4k_last_error());
}

// replaces the Triton kernel behind python/ac4k_kernel/ops/quant.py:21-59 (not in the reference's module)
void global_scale_bf16(torch::Tensor &out, torch::Tensor const &x, double max_scale) {
  check_cuda(x, at::kBFloat16, "x");
  check_cuda(out, at::kFloat, "out");
  TORCH_CHECK(out.numel() == 1, "out must hold one float");
  c10::cuda::CUDAGuard guard(x.device());
  const int rc = ac4k_global_scale_bf16(x.data_ptr(), x.numel(), (float)max_scale, out.data_ptr<float>(),
                                        at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_global_scale_bf16: ", ac4k_last_error());
}

// ops.h:13-17; checks of mha_nvfp4.cu:897-1010.  O may be a permuted view ([B, N, H, D] storage): the kernel addresses it
// by strides.  Block scales in the reference's layout [B, H, K/64, align16(rows), 4] or tiled
// [B, H, ceil(rows/128), K/64, 32, 4, 4].
void mha_nvfp4_fwd(torch::Tensor &o, torch::Tensor &q, torch::Tensor &q_sf, torch::Tensor &q_global_scale, torch::Tensor &k,
                   torch::Tensor &k_sf, torch::Tensor &k_global_scale, torch::Tensor &v, torch::Tensor &v_sf,
                   torch::Tensor &v_global_scale, float sm_scale) {
  check_cuda(q, at::kByte, "Q");
  TORCH_CHECK(q.dim() == 4, "Q must be a 4D tensor");
  const int64_t B = q.size(0), H = q.size(1), Nq = q.size(2), Dqk = q.size(3) * 2;
  TORCH_CHECK(Dqk % 16 == 0, "Dqk must be multiple of 16");
  TORCH_CHECK(Dqk <= 128, "Dqk must be less than 128");
  check_cuda(k, at::kByte, "K");
  TORCH_CHECK(k.dim() == 4, "K must be a 4D tensor");
  TORCH_CHECK(k.size(0) == B, "K must have the same batch size as Q");
  TORCH_CHECK(k.size(1) == H, "K must have the same head number as Q");
  const int64_t Nkv = k.size(2);
  TORCH_CHECK(k.size(3) == q.size(3), "K must have the same dim as Q");
  check_cuda(v, at::kByte, "V");
  TORCH_CHECK(v.dim() == 4, "V must be a 4D tensor");
  TORCH_CHECK(v.size(0) == B, "V must have the same batch size as Q");
  TORCH_CHECK(v.size(1) == H, "V must have the same head number as Q");
  const int64_t Dv = v.size(2);
  TORCH_CHECK(v.size(3) * 2 == align_up(Nkv, 64), "V must have the same sequence length as K");
  TORCH_CHECK(Dv <= 128, "Dv must be less than 128");
  struct Sf { const char *name; torch::Tensor *t; int64_t rows, red; };
  const Sf sfs[3] = {{"q_sf", &q_sf, Nq, Dqk}, {"k_sf", &k_sf, Nkv, Dqk}, {"v_sf", &v_sf, Dv, Nkv}};
  const bool tiled = q_sf.dim() == 7;
  for (const Sf &s : sfs) {
    check_cuda(*s.t, at::kFloat8_e4m3fn, s.name);
    if (tiled) {
      const std::vector<int64_t> want = {B, H, ceil_div(s.rows, 128), ceil_div(s.red, 64), 32, 4, 4};
      TORCH_CHECK(s.t->sizes().vec() == want, "Meet invalid ", s.name, " shape (tiled layout)");
    } else {   // the reference's layout and checks (mha_nvfp4.cu:915-1008)
      TORCH_CHECK(s.t->dim() == 5, s.name, " must be a 5D tensor");
      const std::vector<int64_t> want = {B, H, ceil_div(s.red, 64), align_up(s.rows, 16), 4};
      TORCH_CHECK(s.t->sizes().vec() == want, "Meet invalid ", s.name, " shape");
    }
  }
  for (torch::Tensor *g : {&q_global_scale, &k_global_scale, &v_global_scale}) {
    check_cuda(*g, at::kFloat, "global_scale");
    TORCH_CHECK(g->dim() == 0, "global_scale must be a scalar");
  }
  TORCH_CHECK(o.is_cuda(), "O must be a CUDA tensor");
  TORCH_CHECK(o.scalar_type() == at::kBFloat16, "O must be a bfloat16 tensor");
  TORCH_CHECK(o.dim() == 4 && o.size(0) == B && o.size(1) == H && o.size(2) == Nq && o.size(3) == Dv,
              "O must have shape [B, H, Nq, Dv]");
  const c10::cuda::CUDAGuard guard(o.device());
  const int64_t os[4] = {o.stride(0), o.stride(1), o.stride(2), o.stride(3)};
  const int rc = ac4k_mha_nvfp4_fwd(o.data_ptr(), os, q.data_ptr(), q_sf.data_ptr(), q_global_scale.data_ptr<float>(),
                                    k.data_ptr(), k_sf.data_ptr(), k_global_scale.data_ptr<float>(), v.data_ptr(),
                                    v_sf.data_ptr(), v_global_scale.data_ptr<float>(), B, H, Nq, Nkv, Dqk, Dv, sm_scale,
                                    tiled ? AC4K_SF_TILE128X4 : AC4K_SF_AC4K, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_mha_nvfp4_fwd: ", ac4k_last_error());
}

// ops.h:19-25; checks of mha_int8_x_fp8.cu:983-1060
void mha_int8_x_fp8_fwd(torch::Tensor &o, torch::Tensor &q, torch::Tensor &q_sf, int q_quantize_block_size, torch::Tensor &k,
                        torch::Tensor &k_sf, int k_quantize_block_size, torch::Tensor &v, torch::Tensor &v_sf, float sm_scale) {
  check_cuda(q, at::kChar, "Q");
  TORCH_CHECK(q.dim() == 4, "Q must be a 4D tensor");
  const int64_t B = q.size(0), H = q.size(1), Nq = q.size(2), Dqk = q.size(3);
  TORCH_CHECK(Dqk % 16 == 0, "Dqk must be multiple of 16");
  TORCH_CHECK(Dqk <= 128, "Dqk must be less than 128");
  check_cuda(q_sf, at::kFloat, "Q_SF");
  TORCH_CHECK(q_sf.dim() == 3 && q_sf.size(0) == B && q_sf.size(1) == H && q_sf.size(2) == ceil_div(Nq, q_quantize_block_size),
              "Meet invalid Q_SF shape");
  check_cuda(k, at::kChar, "K");
  TORCH_CHECK(k.dim() == 4, "K must be a 4D tensor");
  TORCH_CHECK(k.size(0) == B, "K must have the same batch size as Q");
  TORCH_CHECK(k.size(1) == H, "K must have the same head number as Q");
  const int64_t Nkv = k.size(2);
  TORCH_CHECK(k.size(3) == Dqk, "K must have the same dim as Q");
  check_cuda(k_sf, at::kFloat, "K_SF");
  TORCH_CHECK(k_sf.dim() == 3 && k_sf.size(0) == B && k_sf.size(1) == H && k_sf.size(2) == ceil_div(Nkv, k_quantize_block_size),
              "Meet invalid K_SF shape");
  check_cuda(v, at::kFloat8_e4m3fn, "V");
  TORCH_CHECK(v.dim() == 4, "V must be a 4D tensor");
  TORCH_CHECK(v.size(0) == B, "V must have the same batch size as Q");
  TORCH_CHECK(v.size(1) == H, "V must have the same head number as Q");
  const int64_t Dv = v.size(2);
  TORCH_CHECK(v.size(3) == align_up(Nkv, 16), "V must have the same sequence length as K");
  TORCH_CHECK(Dv <= 128, "Dv must be less than 128");
  check_cuda(v_sf, at::kFloat, "V_SF");
  TORCH_CHECK(v_sf.dim() == 3 && v_sf.size(0) == B && v_sf.size(1) == H && v_sf.size(2) == align_up(Dv, 16), "Meet invalid v_sf shape");
  TORCH_CHECK(o.is_cuda(), "O must be a CUDA tensor");
  TORCH_CHECK(o.scalar_type() == at::kBFloat16, "O must be a bfloat16 tensor");
  TORCH_CHECK(o.dim() == 4 && o.size(0) == B && o.size(1) == H && o.size(2) == Nq && o.size(3) == Dv, "O must have shape [B, H, Nq, Dv]");
  const c10::cuda::CUDAGuard guard(o.device());
  const int64_t os[4] = {o.stride(0), o.stride(1), o.stride(2), o.stride(3)};
  const int rc = ac4k_mha_int8_x_fp8_fwd(o.data_ptr(), os, q.data_ptr(), q_sf.data_ptr<float>(), q_quantize_block_size, k.data_ptr(),
                                         k_sf.data_ptr<float>(), k_quantize_block_size, v.data_ptr(), v_sf.data_ptr<float>(), B, H, Nq,
                                         Nkv, Dqk, Dv, sm_scale, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_mha_int8_x_fp8_fwd: ", ac4k_last_error());
}

// ops.h:50-54; checks of rope3d.cu:133-165
void rope3d(const torch::Tensor &x, const torch::Tensor &grid_sizes, const torch::Tensor &freqs, torch::Tensor &output) {
  check_cuda(x, at::kBFloat16, "x");
  check_cuda(grid_sizes, at::kInt, "grid_sizes");
  check_cuda(freqs, at::kComplexDouble, "freqs");
  check_cuda(output, at::kBFloat16, "output");
  TORCH_CHECK(x.dim() == 4, "x must be 4D tensor");
  TORCH_CHECK(grid_sizes.dim() == 2, "grid_sizes must be 2D tensor");
  TORCH_CHECK(freqs.dim() == 2, "freqs must be 2D tensor");
  TORCH_CHECK(output.dim() == 4, "output must be 4D tensor");
  const int64_t B = x.size(0), S = x.size(1), N = x.size(2), D = x.size(3);
  TORCH_CHECK(grid_sizes.size(0) == B, "grid_sizes batch size must match x");
  TORCH_CHECK(grid_sizes.size(1) == 3, "grid_sizes must have 3 dimensions (F, H, W)");
  TORCH_CHECK(output.sizes() == x.sizes(), "output shape must match x");
  TORCH_CHECK(D % 2 == 0 && freqs.size(1) == D / 2, "freqs must have D / 2 columns");
  const c10::cuda::CUDAGuard guard(x.device());
  const int rc = ac4k_rope3d(output.data_ptr(), x.data_ptr(), grid_sizes.data_ptr<int32_t>(), freqs.data_ptr(), B, S, N, D,
                             freqs.size(0), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ac4k_rope3d: ", ac4k_last_error());
}

}  // namespace ac4k

PYBIND11_MODULE(_cuda_ops, m) {
  m.doc() = "ac4k_kernel operators for B200 (sm_100a) over libac4k_b200.so";
  m.attr("__arch__") = ac4k_arch();
  m.attr("__arch_description__") = ac4k_arch_description();
  m.attr("__backend__") = ac4k_backend();
  m.attr("__version__") = ac4k_version();
  m.def("mha_nvfp4_fwd", &ac4k::mha_nvfp4_fwd, "Multi-Head Attention Forward (NVFP4)");
  m.def("mha_int8_x_fp8_fwd", &ac4k::mha_int8_x_fp8_fwd, "Multi-Head Attention Forward (QK=INT8, PV=FP8)");
  m.def("quantize_nvfp4", &ac4k::quantize_nvfp4, "Quantize bfloat16 tensor to NVFP4 format");
  m.def("quantize_fp8", &ac4k::quantize_fp8, "Quantize bfloat16 tensor to FP8 format");
  m.def("quantize_int8", &ac4k::quantize_int8, "Quantize bfloat16 tensor to INT8 format");
  m.def("linear_nvfp4", &ac4k::linear_nvfp4, "NVFP4 Linear (fully-connected layer): y = x @ weight.T + bias");
  m.def("rope3d", &ac4k::rope3d, "3D Rotary Position Embedding");
  m.def("global_scale_bf16", &ac4k::global_scale_bf16, "out[0] = max|x| / max_scale");
}

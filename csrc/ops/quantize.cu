// Per-tensor quantisation to 8-bit floats and the Python bindings of the fp8 GEMM.
//   q = saturate_to_fp8(x * fp8_max / amax),   dequantisation factor = amax / fp8_max
// The amax arrives as a device scalar (computed by a reduction on the same stream), so nothing waits on the host.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "ops.h"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

template <int FMT>
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = FMT == 0 ? __NV_E4M3 : __NV_E5M2;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return lo | (hi << 16);
}

// 8 bf16 in, 8 bytes out per thread iteration.
template <int FMT>
__global__ void quantize_bf16_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, const float* __restrict__ amax,
                                     float* __restrict__ scale_inv, long long nv) {
  const float fp8_max = FMT == 0 ? 448.f : 57344.f;
  const float a = fmaxf(amax[0], 1e-12f);
  const float scale = fp8_max / a;
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_inv[0] = a / fp8_max;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = x[i];
    const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
    q[i] = make_uint2(quant4<FMT>(f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale),
                      quant4<FMT>(f2.x * scale, f2.y * scale, f3.x * scale, f3.y * scale));
  }
}

// x: bf16 (any shape, contiguous, numel % 8 == 0); amax: fp32 device scalar. Returns (uint8 tensor like x, fp32 dequantisation factor).
std::vector<Tensor> quantize_fp8(const Tensor& x, const Tensor& amax, int64_t fmt) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.numel() % 8 == 0, "x: contiguous bf16, numel % 8 == 0");
  TORCH_CHECK(amax.is_cuda() && amax.scalar_type() == torch::kFloat32 && amax.numel() == 1, "amax: fp32 device scalar");
  TORCH_CHECK(fmt == 0 || fmt == 1, "fmt: 0 = e4m3, 1 = e5m2");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty(x.sizes(), x.options().dtype(torch::kUInt8));
  Tensor scale_inv = torch::empty({1}, amax.options());
  const long long nv = x.numel() / 8;
  if (nv == 0) return {q, scale_inv.fill_(1.0)};
  long long blocks = (nv + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (fmt == 0)
    quantize_bf16_kernel<0><<<(unsigned)blocks, 256, 0, cur_stream()>>>(reinterpret_cast<const uint4*>(x.data_ptr()),
                                                                       reinterpret_cast<uint2*>(q.data_ptr()), amax.data_ptr<float>(),
                                                                       scale_inv.data_ptr<float>(), nv);
  else
    quantize_bf16_kernel<1><<<(unsigned)blocks, 256, 0, cur_stream()>>>(reinterpret_cast<const uint4*>(x.data_ptr()),
                                                                       reinterpret_cast<uint2*>(q.data_ptr()), amax.data_ptr<float>(),
                                                                       scale_inv.data_ptr<float>(), nv);
  count_launch();
  check_cuda(cudaGetLastError(), "quantize_fp8 launch");
  return {q, scale_inv};
}

// out[M, N] (bf16 or fp32) = (a . b^T) * scale_a * scale_b * alpha; a, b: uint8 tensors holding 8-bit floats.
void gemm_fp8_py(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, int64_t a_fmt, int64_t b_fmt, bool accumulate,
                 double alpha, const c10::optional<Tensor>& scale_a, const c10::optional<Tensor>& scale_b, Tensor& status) {
  for (const Tensor* t : {&a, &b})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kUInt8 && t->dim() == 2 && t->stride(1) == 1, "fp8 operands: uint8 matrices, unit inner stride");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && (out.scalar_type() == torch::kBFloat16 || out.scalar_type() == torch::kFloat32),
              "out: bf16 or fp32 matrix");
  const int M = (int)(a_mn ? a.size(1) : a.size(0)), K = (int)(a_mn ? a.size(0) : a.size(1));
  const int N = (int)(b_mn ? b.size(1) : b.size(0)), Kb = (int)(b_mn ? b.size(0) : b.size(1));
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm_fp8: shape mismatch");
  auto scalar = [](const c10::optional<Tensor>& s) -> const float* {
    if (!s.has_value()) return nullptr;
    TORCH_CHECK(s->is_cuda() && s->scalar_type() == torch::kFloat32 && s->numel() == 1, "scale: fp32 device scalar");
    return s->data_ptr<float>();
  };
  const bool f32 = out.scalar_type() == torch::kFloat32;
  const int epi = f32 ? (accumulate ? 2 : 1) : (accumulate ? 3 : 0);
  const c10::cuda::CUDAGuard guard(a.device());
  gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), a_mn, b_mn, (int)a_fmt, (int)b_fmt, epi,
           (float)alpha, scalar(scale_a), scalar(scale_b), status.data_ptr<int>(), cur_stream());
}

}  // namespace

void register_fp8(py::module_& m) {
  m.def("quantize_fp8", &quantize_fp8);
  m.def("gemm_fp8", &gemm_fp8_py, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("a_fmt") = 0, py::arg("b_fmt") = 0, py::arg("accumulate") = false, py::arg("alpha") = 1.0, py::arg("scale_a") = py::none(),
        py::arg("scale_b") = py::none(), py::arg("status") = py::none());
}

}  // namespace b200

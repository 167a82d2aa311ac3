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

// ----------------------------------------------------------------------------------------------------------------
// OCP microscaling (MX) quantisation: 8-bit payload plus one UE8M0 scale per 32 elements along the contraction
// dimension. Shared exponent of a block = floor(log2(amax)) - emax(format) (8 for e4m3, 15 for e5m2), clamped to
// [-127, 127]; payload = round-to-nearest-even(x * 2^-exponent), saturating. Scale codes (exponent + 127) are written
// in the tile layout that the block-scaled GEMM copies into tensor memory (gemm/gemm_mxfp8.cu).
// ----------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ long long mx_scale_offset(long long op_row, long long kb, long long k_tiles) {
  return ((op_row >> 7) * k_tiles + (kb >> 2)) * 512 + (op_row & 31) * 16 + ((op_row >> 5) & 3) * 4 + (kb & 3);
}

__device__ __forceinline__ int mx_shared_exponent(float amax, int emax) {
  const float a = fmaxf(amax, 1.17549435e-38f);  // 2^-126
  int e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127 - emax;
  return max(-127, min(127, e));
}

__device__ __forceinline__ float mx_inverse_scale(int exponent) { return __uint_as_float((uint32_t)(127 - exponent) << 23); }

// Blocks along the contiguous dimension: one thread per block of 32 elements of x [R, C].
template <int FMT>
__global__ void quantize_mx_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ q, uint8_t* __restrict__ sf, long long R, int Cb) {
  const long long blocks = R * Cb;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < blocks; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / Cb;
    const int kb = (int)(i - r * Cb);
    uint4 v[4];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = x[i * 4 + j];
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(w[e]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    const int exponent = mx_shared_exponent(amax, FMT == 0 ? 8 : 15);
    const float inv = mx_inverse_scale(exponent);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f0 = unpack_bf16x2(v[j].x), f1 = unpack_bf16x2(v[j].y), f2 = unpack_bf16x2(v[j].z), f3 = unpack_bf16x2(v[j].w);
      out[2 * j] = quant4<FMT>(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
      out[2 * j + 1] = quant4<FMT>(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
    }
    q[i * 2] = make_uint4(out[0], out[1], out[2], out[3]);
    q[i * 2 + 1] = make_uint4(out[4], out[5], out[6], out[7]);
    sf[mx_scale_offset(r, kb, Cb >> 2)] = (uint8_t)(exponent + 127);
  }
}

// Blocks along the rows: one thread per 32 rows x 8 adjacent columns of x [R, C]; the operand row of the GEMM is the
// column index, its contraction index the row index.
template <int FMT>
__global__ void quantize_mx_cols_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, uint8_t* __restrict__ sf, int Rb, int Cv) {
  const long long items = (long long)Rb * Cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < items; i += (long long)gridDim.x * blockDim.x) {
    const int rb = (int)(i / Cv);
    const int cv = (int)(i - (long long)rb * Cv);
    float amax[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < 32; ++r) {
      const uint4 v = x[((long long)rb * 32 + r) * Cv + cv];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(w[e]);
        amax[2 * e] = fmaxf(amax[2 * e], fabsf(f.x));
        amax[2 * e + 1] = fmaxf(amax[2 * e + 1], fabsf(f.y));
      }
    }
    float inv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int exponent = mx_shared_exponent(amax[e], FMT == 0 ? 8 : 15);
      inv[e] = mx_inverse_scale(exponent);
      sf[mx_scale_offset((long long)cv * 8 + e, rb, Rb >> 2)] = (uint8_t)(exponent + 127);
    }
    for (int r = 0; r < 32; ++r) {
      const long long at = ((long long)rb * 32 + r) * Cv + cv;
      const uint4 v = x[at];
      const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      q[at] = make_uint2(quant4<FMT>(f0.x * inv[0], f0.y * inv[1], f1.x * inv[2], f1.y * inv[3]),
                         quant4<FMT>(f2.x * inv[4], f2.y * inv[5], f3.x * inv[6], f3.y * inv[7]));
    }
  }
}

// x: bf16 [R, C] contiguous. along_rows = false: blocks of 32 along C (C % 128 == 0), scales indexed (r, c / 32);
// along_rows = true: blocks of 32 along R (R % 128 == 0, C % 8 == 0), scales indexed (c, r / 32).
// Returns (payload uint8 [R, C], scale codes uint8 in the GEMM's tile layout).
std::vector<Tensor> quantize_mx(const Tensor& x, bool along_rows, int64_t fmt) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: contiguous bf16 matrix");
  TORCH_CHECK(fmt == 0 || fmt == 1, "fmt: 0 = e4m3, 1 = e5m2");
  const long long R = x.size(0), C = x.size(1);
  TORCH_CHECK(along_rows ? (R % 128 == 0 && C % 8 == 0) : (C % 128 == 0), "quantize_mx: the block dimension must be a multiple of 128");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor q = torch::empty({R, C}, x.options().dtype(torch::kUInt8));
  const long long op_rows = along_rows ? C : R, k = along_rows ? R : C;
  Tensor sf = torch::zeros({mx_scale_bytes(op_rows, k)}, x.options().dtype(torch::kUInt8));
  if (R == 0 || C == 0) return {q, sf};
  const long long items = along_rows ? (R / 32) * (C / 8) : R * (C / 32);
  long long blocks = (items + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  auto X = reinterpret_cast<const uint4*>(x.data_ptr());
  auto S = sf.data_ptr<uint8_t>();
  if (along_rows) {
    auto Q = reinterpret_cast<uint2*>(q.data_ptr());
    if (fmt == 0) quantize_mx_cols_kernel<0><<<(unsigned)blocks, 256, 0, cur_stream()>>>(X, Q, S, (int)(R / 32), (int)(C / 8));
    else quantize_mx_cols_kernel<1><<<(unsigned)blocks, 256, 0, cur_stream()>>>(X, Q, S, (int)(R / 32), (int)(C / 8));
  } else {
    auto Q = reinterpret_cast<uint4*>(q.data_ptr());
    if (fmt == 0) quantize_mx_rows_kernel<0><<<(unsigned)blocks, 256, 0, cur_stream()>>>(X, Q, S, R, (int)(C / 32));
    else quantize_mx_rows_kernel<1><<<(unsigned)blocks, 256, 0, cur_stream()>>>(X, Q, S, R, (int)(C / 32));
  }
  count_launch();
  check_cuda(cudaGetLastError(), "quantize_mx launch");
  return {q, sf};
}

// Scale codes in plain [rows, k / 32] order (for tests and tools): the inverse of the tile layout.
Tensor mx_scales_to_plain(const Tensor& sf, int64_t rows, int64_t k) {
  TORCH_CHECK(sf.is_cuda() && sf.scalar_type() == torch::kUInt8 && sf.is_contiguous() && sf.numel() == mx_scale_bytes(rows, k), "sf: tiled scale buffer");
  const int64_t kb = k / 32, k_tiles = k / 128, row_tiles = sf.numel() / (k_tiles * 512);
  Tensor t = sf.view({row_tiles, k_tiles, 32, 4, 4});            // [row tile, k tile, r % 32, (r / 32) % 4, kb % 4]
  t = t.permute({0, 3, 2, 1, 4}).reshape({row_tiles * 128, kb});  // row = tile * 128 + quarter * 32 + r % 32
  return t.slice(0, 0, rows).contiguous();
}

// out[M, N] (bf16 or fp32) (+)= alpha * (a . b^T) with MX block scales; a, b: uint8 payloads, sfa / sfb: tiled scale codes.
void gemm_mxfp8_py(const Tensor& a, const Tensor& sfa, const Tensor& b, const Tensor& sfb, Tensor& out, bool a_mn, bool b_mn, int64_t a_fmt,
                   int64_t b_fmt, bool accumulate, double alpha, Tensor& status) {
  for (const Tensor* t : {&a, &b})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kUInt8 && t->dim() == 2 && t->stride(1) == 1, "mxfp8 operands: uint8 matrices, unit inner stride");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && (out.scalar_type() == torch::kBFloat16 || out.scalar_type() == torch::kFloat32),
              "out: bf16 or fp32 matrix");
  const int M = (int)(a_mn ? a.size(1) : a.size(0)), K = (int)(a_mn ? a.size(0) : a.size(1));
  const int N = (int)(b_mn ? b.size(1) : b.size(0)), Kb = (int)(b_mn ? b.size(0) : b.size(1));
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm_mxfp8: shape mismatch");
  TORCH_CHECK(K % 128 == 0, "gemm_mxfp8: the contraction size must be a multiple of 128");
  TORCH_CHECK(sfa.is_cuda() && sfa.scalar_type() == torch::kUInt8 && sfa.is_contiguous() && sfa.numel() == mx_scale_bytes(M, K), "sfa: tiled scales of a");
  TORCH_CHECK(sfb.is_cuda() && sfb.scalar_type() == torch::kUInt8 && sfb.is_contiguous() && sfb.numel() == mx_scale_bytes(N, K), "sfb: tiled scales of b");
  const bool f32 = out.scalar_type() == torch::kFloat32;
  const int epi = f32 ? (accumulate ? 2 : 1) : (accumulate ? 3 : 0);
  const c10::cuda::CUDAGuard guard(a.device());
  gemm_mxfp8(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), a_mn,
             b_mn, (int)a_fmt, (int)b_fmt, epi, (float)alpha, status.data_ptr<int>(), cur_stream());
}

}  // namespace

void register_fp8(py::module_& m) {
  m.def("quantize_mx", &quantize_mx, py::arg("x"), py::arg("along_rows") = false, py::arg("fmt") = 0);
  m.def("mx_scales_to_plain", &mx_scales_to_plain);
  m.def("gemm_mxfp8", &gemm_mxfp8_py, py::arg("a"), py::arg("sfa"), py::arg("b"), py::arg("sfb"), py::arg("out"), py::arg("a_mn") = false,
        py::arg("b_mn") = false, py::arg("a_fmt") = 0, py::arg("b_fmt") = 0, py::arg("accumulate") = false, py::arg("alpha") = 1.0,
        py::arg("status") = py::none());
  m.def("quantize_fp8", &quantize_fp8);
  m.def("gemm_fp8", &gemm_fp8_py, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("a_fmt") = 0, py::arg("b_fmt") = 0, py::arg("accumulate") = false, py::arg("alpha") = 1.0, py::arg("scale_a") = py::none(),
        py::arg("scale_b") = py::none(), py::arg("status") = py::none());
}

}  // namespace b200

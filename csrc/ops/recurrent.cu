// Multi-head recurrent scans with block-diagonal state transitions (sm_100a): a tanh RNN and a GRU, forward and backward,
// over packed sequences.
//
//   RNN:  h_t = tanh(h_{t-1} W + x_t)
//   GRU:  f = sigmoid(h W_f + x_f),  r = sigmoid(h W_r + x_r),  z = tanh((r * h) W + x_z),  h_t = f * h + (1 - f) * z
//
// One CTA owns one (document, head) pair and walks its tokens in order; the d x d transition matrices of the head stay
// in shared memory as fp32 for the whole scan and the state never leaves the SM. With G matrices per head (1 or 3) the
// CTA has G * d threads: thread (m, e) owns output column e of matrix m, both for the matrix-vector products and, in the
// backward pass, for the weight-gradient column it accumulates in registers over the whole document (one atomic add per
// element at the end). The gradient that flows back through the state is clamped at every step when a limit is given.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "../common/launch.h"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float tanh_f(float x) {
  const float e = __expf(-2.f * fabsf(x));
  const float t = (1.f - e) / (1.f + e);
  return copysignf(t, x);
}

// sum_k v[k] * w[k * D] with v in shared memory (read as float4 broadcasts) and w a column of a [D, D] matrix
template <int D>
__device__ __forceinline__ float column_dot(const float* __restrict__ v, const float* __restrict__ w) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int k = 0; k < D; k += 4) {
    const float4 h = *reinterpret_cast<const float4*>(v + k);
    a0 = fmaf(h.x, w[(k + 0) * D], a0);
    a1 = fmaf(h.y, w[(k + 1) * D], a1);
    a2 = fmaf(h.z, w[(k + 2) * D], a2);
    a3 = fmaf(h.w, w[(k + 3) * D], a3);
  }
  return (a0 + a1) + (a2 + a3);
}

// sum_k v[k] * w[k] with v in shared memory and w (one matrix column, or row of the transposed matrix) in registers
template <int D>
__device__ __forceinline__ float register_dot(const float* __restrict__ v, const float (&w)[D]) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int k = 0; k < D; k += 4) {
    const float4 h = *reinterpret_cast<const float4*>(v + k);
    a0 = fmaf(h.x, w[k + 0], a0);
    a1 = fmaf(h.y, w[k + 1], a1);
    a2 = fmaf(h.z, w[k + 2], a2);
    a3 = fmaf(h.w, w[k + 3], a3);
  }
  return (a0 + a1) + (a2 + a3);
}

// ------------------------------------------------------------------------------------------------ forward
// x: [T, G, n, d] through (row_stride, gate_stride = n * d); weight: [G * n, d, d] fp32; h0: [docs, n, d] fp32 or null.
// out: [T, n, d]; gates (GRU only): [T, 3, n, d] = z, f, r of every step, kept for the backward pass.
template <int D, bool GRU, typename T>
__global__ void __launch_bounds__((GRU ? 3 : 1) * D)
    recurrent_fwd_kernel(const T* __restrict__ x, long long row_stride, const float* __restrict__ weight, const float* __restrict__ h0,
                         const int* __restrict__ cu, int n, T* __restrict__ out, T* __restrict__ gates) {
  constexpr int G = GRU ? 3 : 1;
  extern __shared__ __align__(16) float smem_f[];
  float* sW = smem_f;               // [G][D][D]
  float* sH = sW + G * D * D;       // [2][D] state, double-buffered
  float* sRH = sH + 2 * D;          // [D] r * h
  float* sF = sRH + D;              // [D] f
  const int doc = blockIdx.x, head = blockIdx.y;
  const int m = threadIdx.x / D, e = threadIdx.x - m * D;
  const int t0 = cu[doc], t1 = cu[doc + 1];
  for (int i = threadIdx.x; i < G * D * D; i += G * D) {
    const int mm = i / (D * D);
    sW[i] = weight[((size_t)(mm * n + head)) * D * D + (i - mm * D * D)];
  }
  if (m == 0) sH[e] = h0 != nullptr ? h0[((size_t)doc * n + head) * D + e] : 0.f;
  __syncthreads();
  // this thread's matrix column lives in registers for the whole scan (shared memory only stages the load)
  float w_col[D];
#pragma unroll
  for (int k = 0; k < D; ++k) w_col[k] = sW[m * D * D + k * D + e];
  const size_t gate_stride = (size_t)n * D;
  int cur = 0;
  for (int t = t0; t < t1; ++t) {
    const float* h = sH + cur * D;
    const float xv = ld_f(x + (size_t)t * row_stride + m * gate_stride + (size_t)head * D + e);
    if (!GRU) {
      const float hn = tanh_f(xv + register_dot<D>(h, w_col));
      st_f(out + ((size_t)t * n + head) * D + e, hn);
      sH[(cur ^ 1) * D + e] = hn;
      __syncthreads();
    } else {
      float gate = 0.f;
      if (m != 0) {
        gate = sigmoid_f(xv + register_dot<D>(h, w_col));
        if (m == 1) sF[e] = gate; else sRH[e] = gate * h[e];
        st_f(gates + (((size_t)t * 3 + m) * n + head) * D + e, gate);
      }
      __syncthreads();
      if (m == 0) {
        const float z = tanh_f(xv + register_dot<D>(sRH, w_col));
        const float f = sF[e];
        const float hn = f * h[e] + (1.f - f) * z;
        st_f(gates + (((size_t)t * 3) * n + head) * D + e, z);
        st_f(out + ((size_t)t * n + head) * D + e, hn);
        sH[(cur ^ 1) * D + e] = hn;
      }
      __syncthreads();
    }
    cur ^= 1;
  }
}

// ------------------------------------------------------------------------------------------------ backward
// dout / out: [T, n, d]; gates: [T, 3, n, d]; dx: [T, G, n, d] (contiguous); dweight: [G * n, d, d] fp32 (added to);
// dh0: [docs, n, d] fp32 or null. clip <= 0 disables the clamp of the state gradient.
template <int D, bool GRU, typename T>
__global__ void __launch_bounds__((GRU ? 3 : 1) * D)
    recurrent_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ out, const T* __restrict__ gates,
                         const float* __restrict__ weight, const float* __restrict__ h0, const int* __restrict__ cu, int n, float clip,
                         T* __restrict__ dx, float* __restrict__ dweight, float* __restrict__ dh0) {
  constexpr int G = GRU ? 3 : 1;
  extern __shared__ __align__(16) float smem_f[];
  float* sWT = smem_f;              // [G][D (e)][D (k)]: transposed, so that thread k reads row k of W without conflicts
  float* sDP = sWT + G * D * D;     // [G][D] gradients of the pre-activations (z, f, r)
  float* sHP = sDP + G * D;         // [D] previous state
  float* sRH = sHP + D;             // [D] r * previous state
  float* sPart = sRH + D;           // [3][D] partial state gradients: W dpz, W_f dpf, W_r dpr
  const int doc = blockIdx.x, head = blockIdx.y;
  const int m = threadIdx.x / D, e = threadIdx.x - m * D;
  const int t0 = cu[doc], t1 = cu[doc + 1];
  for (int i = threadIdx.x; i < G * D * D; i += G * D) {
    const int mm = i / (D * D), rest = i - mm * D * D;
    const int k = rest / D, c = rest - k * D;
    sWT[mm * D * D + c * D + k] = weight[((size_t)(mm * n + head)) * D * D + rest];
  }
  __syncthreads();
  const float* wt_col = sWT + m * D * D + e;  // element j of row e of W_m at wt_col[j * D]
  // up to d = 64 that row also fits in registers next to the weight-gradient column (2 d registers per thread)
  constexpr bool kRowInRegisters = D <= 64;
  float wt_reg[kRowInRegisters ? D : 1];
  if constexpr (kRowInRegisters) {
#pragma unroll
    for (int j = 0; j < D; ++j) wt_reg[j] = wt_col[j * D];
  }
  auto row_dot = [&](const float* vec) -> float {
    if constexpr (kRowInRegisters) return register_dot<D>(vec, wt_reg);
    else return column_dot<D>(vec, wt_col);
  };
  float dw[D];
#pragma unroll
  for (int k = 0; k < D; ++k) dw[k] = 0.f;
  float carry = 0.f;
  const size_t gs = (size_t)n * D;
  for (int t = t1 - 1; t >= t0; --t) {
    const size_t at = ((size_t)t * n + head) * D + e;
    const float g = ld_f(dout + at) + carry;
    const float hp = t > t0 ? ld_f(out + at - gs) : (h0 != nullptr ? h0[((size_t)doc * n + head) * D + e] : 0.f);
    if (!GRU) {
      const float ht = ld_f(out + at);
      const float dp = g * (1.f - ht * ht);
      st_f(dx + at, dp);
      sDP[e] = dp;
      sHP[e] = hp;
      __syncthreads();
      carry = row_dot(sDP);
      if (clip > 0.f) carry = fminf(fmaxf(carry, -clip), clip);
#pragma unroll
      for (int k = 0; k < D; k += 4) {
        const float4 h4 = *reinterpret_cast<const float4*>(sHP + k);
        dw[k] = fmaf(h4.x, dp, dw[k]);
        dw[k + 1] = fmaf(h4.y, dp, dw[k + 1]);
        dw[k + 2] = fmaf(h4.z, dp, dw[k + 2]);
        dw[k + 3] = fmaf(h4.w, dp, dw[k + 3]);
      }
      __syncthreads();
    } else {
      const size_t ag = (((size_t)t * 3) * n + head) * D + e;
      const float z = ld_f(gates + ag), f = ld_f(gates + ag + gs), r = ld_f(gates + ag + 2 * gs);
      const float dpz = g * (1.f - f) * (1.f - z * z);
      const float dpf = g * (hp - z) * f * (1.f - f);
      if (m == 0) {
        st_f(dx + ag, dpz);
        sDP[e] = dpz;
        sRH[e] = r * hp;
        sHP[e] = hp;
      } else if (m == 1) {
        st_f(dx + ag + gs, dpf);
        sDP[D + e] = dpf;
      }
      __syncthreads();
      if (m < 2) sPart[m * D + e] = row_dot(sDP + m * D);
      __syncthreads();
      const float drh = sPart[e];
      const float dpr = drh * hp * r * (1.f - r);
      if (m == 2) {
        st_f(dx + ag + 2 * gs, dpr);
        sDP[2 * D + e] = dpr;
      }
      __syncthreads();
      if (m == 2) sPart[2 * D + e] = row_dot(sDP + 2 * D);
      // weight-gradient column of this thread: dW_m[k, e] += a[k] * dp_m[e], a = r * h for the candidate matrix, h otherwise
      {
        const float dp = m == 0 ? dpz : (m == 1 ? dpf : dpr);
        const float* a = m == 0 ? sRH : sHP;
#pragma unroll
        for (int k = 0; k < D; k += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(a + k);
          dw[k] = fmaf(a4.x, dp, dw[k]);
          dw[k + 1] = fmaf(a4.y, dp, dw[k + 1]);
          dw[k + 2] = fmaf(a4.z, dp, dw[k + 2]);
          dw[k + 3] = fmaf(a4.w, dp, dw[k + 3]);
        }
      }
      __syncthreads();
      carry = g * f + drh * r + sPart[D + e] + sPart[2 * D + e];
      if (clip > 0.f) carry = fminf(fmaxf(carry, -clip), clip);
    }
  }
  if (dh0 != nullptr && m == 0) dh0[((size_t)doc * n + head) * D + e] = carry;
  float* dst = dweight + ((size_t)(m * n + head)) * D * D + e;
#pragma unroll
  for (int k = 0; k < D; ++k) atomicAdd(dst + (size_t)k * D, dw[k]);
}

template <int D, bool GRU, typename T>
void launch_fwd(const Tensor& x, const Tensor& weight, const float* h0, const Tensor& cu, int n, Tensor& out, T* gates) {
  constexpr int G = GRU ? 3 : 1;
  const size_t smem = (size_t)(G * D * D + 4 * D) * sizeof(float);
  auto kernel = recurrent_fwd_kernel<D, GRU, T>;
  check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "recurrent_fwd smem attr");
  dim3 grid((unsigned)(cu.numel() - 1), (unsigned)n);
  kernel<<<grid, G * D, smem, cur_stream()>>>(reinterpret_cast<const T*>(x.data_ptr()), x.stride(0), weight.data_ptr<float>(), h0,
                                              cu.data_ptr<int>(), n, reinterpret_cast<T*>(out.data_ptr()), gates);
  count_launch();
  check_cuda(cudaGetLastError(), "recurrent_fwd launch");
}

template <int D, bool GRU, typename T>
void launch_bwd(const Tensor& dout, const Tensor& out, const T* gates, const Tensor& weight, const float* h0, const Tensor& cu, int n,
                float clip, Tensor& dx, Tensor& dweight, float* dh0) {
  constexpr int G = GRU ? 3 : 1;
  const size_t smem = (size_t)(G * D * D + G * D + 2 * D + 3 * D) * sizeof(float);
  auto kernel = recurrent_bwd_kernel<D, GRU, T>;
  check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "recurrent_bwd smem attr");
  dim3 grid((unsigned)(cu.numel() - 1), (unsigned)n);
  kernel<<<grid, G * D, smem, cur_stream()>>>(reinterpret_cast<const T*>(dout.data_ptr()), reinterpret_cast<const T*>(out.data_ptr()), gates,
                                              weight.data_ptr<float>(), h0, cu.data_ptr<int>(), n, clip,
                                              reinterpret_cast<T*>(dx.data_ptr()), dweight.data_ptr<float>(), dh0);
  count_launch();
  check_cuda(cudaGetLastError(), "recurrent_bwd launch");
}

#define B200_RECURRENT_DISPATCH(D_, GRU_, IS_BF16_, CALL)                         \
  do {                                                                            \
    if (IS_BF16_) {                                                               \
      using scalar_t = __nv_bfloat16;                                             \
      if (GRU_) { constexpr bool kGru = true; CALL(D_, kGru, scalar_t); }         \
      else { constexpr bool kGru = false; CALL(D_, kGru, scalar_t); }             \
    } else {                                                                      \
      using scalar_t = float;                                                     \
      if (GRU_) { constexpr bool kGru = true; CALL(D_, kGru, scalar_t); }         \
      else { constexpr bool kGru = false; CALL(D_, kGru, scalar_t); }             \
    }                                                                             \
  } while (0)

void check_common(const Tensor& x, const Tensor& weight, const Tensor& cu, int64_t n, int64_t d, bool gru) {
  const int64_t G = gru ? 3 : 1;
  TORCH_CHECK(x.is_cuda() && (x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat32), "x: bf16 or fp32 on the GPU");
  TORCH_CHECK(x.dim() == 2 && x.size(1) == G * n * d && x.stride(1) == 1, "x: [tokens, gates * heads * d] with unit inner stride");
  TORCH_CHECK(weight.scalar_type() == torch::kFloat32 && weight.is_contiguous() && weight.dim() == 3 && weight.size(0) == G * n &&
                  weight.size(1) == d && weight.size(2) == d, "weight: fp32 [gates * heads, d, d]");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && cu.is_contiguous() && cu.numel() >= 2, "cu_seqlens: int32");
  TORCH_CHECK(d == 16 || d == 32 || d == 64 || d == 128, "state width per head must be 16, 32, 64 or 128");
}

// -> (states [T, n, d], gates [T, 3, n, d] or an empty tensor)
std::vector<Tensor> recurrent_scan_fwd(const Tensor& x, const Tensor& weight, const c10::optional<Tensor>& h0, const Tensor& cu, int64_t n,
                                       int64_t d, bool gru) {
  check_common(x, weight, cu, n, d, gru);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0);
  Tensor out = torch::empty({T, n, d}, x.options());
  Tensor gates = gru ? torch::empty({T, 3, n, d}, x.options()) : torch::empty({0}, x.options());
  const float* h0p = nullptr;
  if (h0.has_value()) {
    TORCH_CHECK(h0->scalar_type() == torch::kFloat32 && h0->is_contiguous() && h0->numel() == (cu.numel() - 1) * n * d, "h0: fp32 [docs, n, d]");
    h0p = h0->data_ptr<float>();
  }
  if (T == 0) return {out, gates};
  const bool bf16 = x.scalar_type() == torch::kBFloat16;
#define B200_CALL_FWD(D_, G_, T_) launch_fwd<D_, G_, T_>(x, weight, h0p, cu, (int)n, out, gru ? reinterpret_cast<T_*>(gates.data_ptr()) : nullptr)
  switch (d) {
    case 16: B200_RECURRENT_DISPATCH(16, gru, bf16, B200_CALL_FWD); break;
    case 32: B200_RECURRENT_DISPATCH(32, gru, bf16, B200_CALL_FWD); break;
    case 64: B200_RECURRENT_DISPATCH(64, gru, bf16, B200_CALL_FWD); break;
    default: B200_RECURRENT_DISPATCH(128, gru, bf16, B200_CALL_FWD); break;
  }
#undef B200_CALL_FWD
  return {out, gates};
}

// -> (dx [T, G * n * d], dweight fp32 [G * n, d, d], dh0 fp32 [docs, n, d])
std::vector<Tensor> recurrent_scan_bwd(const Tensor& dout, const Tensor& out, const Tensor& gates, const Tensor& weight,
                                       const c10::optional<Tensor>& h0, const Tensor& cu, int64_t n, int64_t d, bool gru, double clip) {
  TORCH_CHECK(dout.is_contiguous() && out.is_contiguous() && dout.sizes() == out.sizes() && dout.scalar_type() == out.scalar_type(), "dout / out: contiguous [T, n, d]");
  TORCH_CHECK(out.dim() == 3 && out.size(1) == n && out.size(2) == d, "out: [T, n, d]");
  const int64_t G = gru ? 3 : 1;
  const int64_t T = out.size(0);
  TORCH_CHECK(weight.scalar_type() == torch::kFloat32 && weight.is_contiguous() && weight.size(0) == G * n, "weight: fp32 [gates * heads, d, d]");
  TORCH_CHECK(d == 16 || d == 32 || d == 64 || d == 128, "state width per head must be 16, 32, 64 or 128");
  if (gru) TORCH_CHECK(gates.is_contiguous() && gates.numel() == T * 3 * n * d && gates.scalar_type() == out.scalar_type(), "gates: [T, 3, n, d]");
  const c10::cuda::CUDAGuard guard(out.device());
  Tensor dx = torch::empty({T, G * n * d}, out.options());
  Tensor dweight = torch::zeros_like(weight);
  const int64_t docs = cu.numel() - 1;
  Tensor dh0 = torch::zeros({docs, n, d}, weight.options());
  const float* h0p = h0.has_value() ? h0->data_ptr<float>() : nullptr;
  if (T == 0) return {dx, dweight, dh0};
  const bool bf16 = out.scalar_type() == torch::kBFloat16;
#define B200_CALL_BWD(D_, G_, T_) \
  launch_bwd<D_, G_, T_>(dout, out, gru ? reinterpret_cast<const T_*>(gates.data_ptr()) : nullptr, weight, h0p, cu, (int)n, (float)clip, dx, dweight, dh0.data_ptr<float>())
  switch (d) {
    case 16: B200_RECURRENT_DISPATCH(16, gru, bf16, B200_CALL_BWD); break;
    case 32: B200_RECURRENT_DISPATCH(32, gru, bf16, B200_CALL_BWD); break;
    case 64: B200_RECURRENT_DISPATCH(64, gru, bf16, B200_CALL_BWD); break;
    default: B200_RECURRENT_DISPATCH(128, gru, bf16, B200_CALL_BWD); break;
  }
#undef B200_CALL_BWD
  return {dx, dweight, dh0};
}

}  // namespace

void register_recurrent(py::module_& m) {
  m.def("recurrent_scan_fwd", &recurrent_scan_fwd);
  m.def("recurrent_scan_bwd", &recurrent_scan_bwd);
}

}  // namespace b200

// Token-layout kernels: padded <-> packed copies, depthwise causal convolution over packed sequences, and the MoE router
// (top-k + softmax over the selected logits + expert histogram). All memory-bound; one warp per token row.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// Sequence that holds packed token t: the last b with cu[b] <= t (cu has batch + 1 entries).
__device__ __forceinline__ int sequence_of(const int* __restrict__ cu, int batch, int t) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// ---------------------------------------------------------------------------------------------- pack / unpack
// PACK: packed[t] = padded[b, s];  UNPACK: padded[b, s] = packed[t] (the rest of `padded` is zeroed by the caller).
template <bool PACK>
__global__ void pack_kernel(uint4* __restrict__ packed, uint4* __restrict__ padded, const int* __restrict__ cu, int batch, int seq,
                            int row_v, int total, int left_padded) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= total) return;
  const int b = sequence_of(cu, batch, warp);
  const int len = cu[b + 1] - cu[b];
  const int pos = warp - cu[b];
  const int s = left_padded ? seq - len + pos : pos;
  uint4* p = packed + (size_t)warp * row_v;
  uint4* q = padded + ((size_t)b * seq + s) * row_v;
  for (int i = lane; i < row_v; i += 32) {
    if (PACK) p[i] = q[i]; else q[i] = p[i];
  }
}

// ---------------------------------------------------------------------------------------------- depthwise causal conv
// y[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (K - 1) + j, c]) with x = 0 before the start of t's sequence.
template <typename T>
__global__ void conv_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, T* __restrict__ y,
                                const int* __restrict__ cu, int batch, int tokens, int channels, int K, int silu) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)tokens * channels) return;
  const int t = (int)(idx / channels), c = (int)(idx - (long long)t * channels);
  const int start = cu[sequence_of(cu, batch, t)];
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = t - (K - 1) + j;
    if (src >= start) acc += w[c * K + j] * to_f(x[(long long)src * channels + c]);
  }
  if (silu) acc = acc / (1.f + __expf(-acc));
  y[idx] = from_f<T>(acc);
}

// dx[t, c] = sum_j w[c, j] * g[t + (K - 1) - j, c] inside t's sequence, g = dy * act'(pre-activation).
// dw[c, j] += sum_t g[t, c] * x[t - (K - 1) + j, c]; dbias[c] += sum_t g[t, c]   (fp32 atomics, one partial per block row range)
template <typename T>
__global__ void conv_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw, float* __restrict__ dbias,
                                const int* __restrict__ cu, int batch, int tokens, int channels, int K, int silu, int rows_per_block) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int t0 = blockIdx.y * rows_per_block;
  const int t1 = min(t0 + rows_per_block, tokens);
  float wreg[8], dwacc[8];
  for (int j = 0; j < K; ++j) wreg[j] = w[c * K + j], dwacc[j] = 0.f;
  float dbacc = 0.f;
  // gradient through the activation at token u (needs the pre-activation, recomputed from x)
  auto grad_at = [&](int u, int start) -> float {
    float g = to_f(dy[(long long)u * channels + c]);
    if (silu) {
      float pre = bias ? bias[c] : 0.f;
      for (int j = 0; j < K; ++j) {
        const int src = u - (K - 1) + j;
        if (src >= start) pre += wreg[j] * to_f(x[(long long)src * channels + c]);
      }
      const float s = 1.f / (1.f + __expf(-pre));
      g *= s * (1.f + pre * (1.f - s));
    }
    return g;
  };
  for (int t = t0; t < t1; ++t) {
    const int b = sequence_of(cu, batch, t);
    const int start = cu[b], end = cu[b + 1];
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int u = t + (K - 1) - j;
      if (u < end) acc += wreg[j] * grad_at(u, start);
    }
    dx[(long long)t * channels + c] = from_f<T>(acc);
    const float g = grad_at(t, start);
    dbacc += g;
    for (int j = 0; j < K; ++j) {
      const int src = t - (K - 1) + j;
      if (src >= start) dwacc[j] += g * to_f(x[(long long)src * channels + c]);
    }
  }
  for (int j = 0; j < K; ++j) atomicAdd(&dw[c * K + j], dwacc[j]);
  if (dbias) atomicAdd(&dbias[c], dbacc);
}

// ---------------------------------------------------------------------------------------------- router
// One warp per token: k rounds of warp arg-max over up to 256 logits (lowest index wins ties), softmax over the k
// selected logits in fp32, and a histogram of the selected experts.
template <typename T>
__global__ void topk_route_kernel(const T* __restrict__ logits, float* __restrict__ weights, int* __restrict__ experts,
                                  int* __restrict__ counts, int tokens, int E, int k) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? to_f(logits[(long long)warp * E + e]) : -INFINITY;
  }
  float picked[8];
  int picked_e[8];
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) best = v[i], best_e = e;
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) best = ob, best_e = oe;
    }
    picked[r] = best;
    picked_e[r] = best_e;
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i == (best_e >> 5)) v[i] = -INFINITY;
    }
  }
  if (lane == 0) {
    float denom = 0.f;
    for (int r = 0; r < k; ++r) denom += __expf(picked[r] - picked[0]);
    for (int r = 0; r < k; ++r) {
      weights[(long long)warp * k + r] = __expf(picked[r] - picked[0]) / denom;
      experts[(long long)warp * k + r] = picked_e[r];
      if (counts) atomicAdd(&counts[picked_e[r]], 1);
    }
  }
}

int row_vectors(const Tensor& t, int lead_dims) {
  int64_t row = 1;
  for (int d = lead_dims; d < t.dim(); ++d) row *= t.size(d);
  const int64_t bytes = row * t.element_size();
  TORCH_CHECK(bytes % 16 == 0, "rows must be a multiple of 16 bytes");
  return (int)(bytes / 16);
}

Tensor pack_sequence(const Tensor& padded, const Tensor& cu_seqlens, int64_t total_tokens, bool left_padded) {
  TORCH_CHECK(padded.is_cuda() && padded.is_contiguous() && padded.dim() >= 2, "padded: contiguous CUDA [batch, seq, ...]");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == torch::kInt32 && cu_seqlens.numel() == padded.size(0) + 1, "cu_seqlens: int32 [batch + 1]");
  const c10::cuda::CUDAGuard guard(padded.device());
  std::vector<int64_t> shape{total_tokens};
  for (int d = 2; d < padded.dim(); ++d) shape.push_back(padded.size(d));
  Tensor out = torch::empty(shape, padded.options());
  if (total_tokens == 0) return out;
  const int row_v = row_vectors(padded, 2);
  const long long threads = total_tokens * 32;
  pack_kernel<true><<<(unsigned)((threads + 255) / 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<uint4*>(out.data_ptr()), reinterpret_cast<uint4*>(padded.data_ptr()), cu_seqlens.data_ptr<int>(),
      (int)padded.size(0), (int)padded.size(1), row_v, (int)total_tokens, left_padded ? 1 : 0);
  count_launch();
  check_cuda(cudaGetLastError(), "pack_sequence launch");
  return out;
}

Tensor unpack_sequence(const Tensor& packed, const Tensor& cu_seqlens, int64_t batch, int64_t seq, bool left_padded) {
  TORCH_CHECK(packed.is_cuda() && packed.is_contiguous() && packed.dim() >= 1, "packed: contiguous CUDA [tokens, ...]");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == torch::kInt32 && cu_seqlens.numel() == batch + 1, "cu_seqlens: int32 [batch + 1]");
  const c10::cuda::CUDAGuard guard(packed.device());
  std::vector<int64_t> shape{batch, seq};
  for (int d = 1; d < packed.dim(); ++d) shape.push_back(packed.size(d));
  Tensor out = torch::zeros(shape, packed.options());
  const int64_t total = packed.size(0);
  if (total == 0) return out;
  const int row_v = row_vectors(packed, 1);
  const long long threads = total * 32;
  pack_kernel<false><<<(unsigned)((threads + 255) / 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<uint4*>(packed.data_ptr()), reinterpret_cast<uint4*>(out.data_ptr()), cu_seqlens.data_ptr<int>(), (int)batch,
      (int)seq, row_v, (int)total, left_padded ? 1 : 0);
  count_launch();
  check_cuda(cudaGetLastError(), "unpack_sequence launch");
  return out;
}

void check_conv(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, const Tensor& cu) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2, "x: contiguous CUDA [tokens, channels]");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat32, "x: bf16 or fp32");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kFloat32 && w.is_contiguous() && w.dim() == 2 && w.size(0) == x.size(1) && w.size(1) <= 8,
              "w: fp32 [channels, K <= 8]");
  if (bias.has_value()) TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == torch::kFloat32 && bias->numel() == x.size(1), "bias: fp32 [channels]");
  TORCH_CHECK(cu.is_cuda() && cu.scalar_type() == torch::kInt32 && cu.numel() >= 2, "cu_seqlens: int32 [batch + 1]");
}

Tensor causal_conv1d_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, const Tensor& cu_seqlens, bool silu) {
  check_conv(x, w, bias, cu_seqlens);
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  const long long total = x.numel();
  if (total == 0) return y;
  const float* b = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const int batch = (int)cu_seqlens.numel() - 1, T = (int)x.size(0), C = (int)x.size(1), K = (int)w.size(1);
  if (x.scalar_type() == torch::kBFloat16)
    conv_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, cur_stream()>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), w.data_ptr<float>(), b,
                                                                    reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), cu_seqlens.data_ptr<int>(), batch, T, C, K, silu);
  else
    conv_fwd_kernel<float><<<blocks, 256, 0, cur_stream()>>>(x.data_ptr<float>(), w.data_ptr<float>(), b, y.data_ptr<float>(),
                                                            cu_seqlens.data_ptr<int>(), batch, T, C, K, silu);
  count_launch();
  check_cuda(cudaGetLastError(), "causal_conv1d_fwd launch");
  return y;
}

std::vector<Tensor> causal_conv1d_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias,
                                      const Tensor& cu_seqlens, bool silu) {
  check_conv(x, w, bias, cu_seqlens);
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type(), "dy: like x");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dw = torch::zeros_like(w);
  Tensor db = torch::zeros({x.size(1)}, w.options());
  if (x.numel() == 0) return {dx, dw, db};
  const float* b = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  const int batch = (int)cu_seqlens.numel() - 1, T = (int)x.size(0), C = (int)x.size(1), K = (int)w.size(1);
  const int rows_per_block = 64;
  dim3 grid((C + 127) / 128, (T + rows_per_block - 1) / rows_per_block);
  if (x.scalar_type() == torch::kBFloat16)
    conv_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, cur_stream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), w.data_ptr<float>(), b, reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()),
        reinterpret_cast<__nv_bfloat16*>(dx.data_ptr()), dw.data_ptr<float>(), db.data_ptr<float>(), cu_seqlens.data_ptr<int>(), batch, T, C, K, silu,
        rows_per_block);
  else
    conv_bwd_kernel<float><<<grid, 128, 0, cur_stream()>>>(x.data_ptr<float>(), w.data_ptr<float>(), b, dy.data_ptr<float>(), dx.data_ptr<float>(),
                                                          dw.data_ptr<float>(), db.data_ptr<float>(), cu_seqlens.data_ptr<int>(), batch, T, C, K, silu,
                                                          rows_per_block);
  count_launch();
  check_cuda(cudaGetLastError(), "causal_conv1d_bwd launch");
  return {dx, dw, db};
}

std::vector<Tensor> topk_route(const Tensor& logits, int64_t k, bool want_counts) {
  TORCH_CHECK(logits.is_cuda() && logits.is_contiguous() && logits.dim() == 2, "logits: contiguous CUDA [tokens, experts]");
  TORCH_CHECK(logits.scalar_type() == torch::kBFloat16 || logits.scalar_type() == torch::kFloat32, "logits: bf16 or fp32");
  const int64_t T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 256 && k >= 1 && k <= 8 && k <= E, "router kernel: at most 256 experts and top-8");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor weights = torch::empty({T, k}, logits.options().dtype(torch::kFloat32));
  Tensor experts = torch::empty({T, k}, logits.options().dtype(torch::kInt32));
  Tensor counts = torch::zeros({want_counts ? E : 0}, logits.options().dtype(torch::kInt32));
  if (T == 0) return {weights, experts, counts};
  const long long threads = T * 32;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  int* cptr = want_counts ? counts.data_ptr<int>() : nullptr;
  if (logits.scalar_type() == torch::kBFloat16)
    topk_route_kernel<__nv_bfloat16><<<blocks, 256, 0, cur_stream()>>>(reinterpret_cast<const __nv_bfloat16*>(logits.data_ptr()),
                                                                      weights.data_ptr<float>(), experts.data_ptr<int>(), cptr, (int)T, (int)E, (int)k);
  else
    topk_route_kernel<float><<<blocks, 256, 0, cur_stream()>>>(logits.data_ptr<float>(), weights.data_ptr<float>(), experts.data_ptr<int>(), cptr,
                                                              (int)T, (int)E, (int)k);
  count_launch();
  check_cuda(cudaGetLastError(), "topk_route launch");
  return {weights, experts, counts};
}

}  // namespace

void register_sequence(py::module_& m) {
  m.def("pack_sequence", &pack_sequence);
  m.def("unpack_sequence", &unpack_sequence);
  m.def("causal_conv1d_fwd", &causal_conv1d_fwd);
  m.def("causal_conv1d_bwd", &causal_conv1d_bwd);
  m.def("topk_route", &topk_route);
}

}  // namespace b200

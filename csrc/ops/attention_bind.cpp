// Python bindings of the packed-sequence attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.h"

namespace b200 {

namespace {

using torch::Tensor;

inline int* status_of(const c10::optional<Tensor>& s) { return s.has_value() ? s->data_ptr<int>() : nullptr; }

// qkv: [T, groups*(qpg+2)*d] bf16 (unit inner stride). Returns (out [T, groups*qpg*d] bf16, lse [groups*qpg, T] fp32).
std::vector<Tensor> attn_fwd(const Tensor& qkv, const Tensor& cu_seqlens, int64_t max_seqlen, int64_t groups, int64_t qpg,
                             int64_t d, double scale, bool causal, const c10::optional<Tensor>& status) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1, "qkv: [T, C] bf16");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == torch::kInt32 && cu_seqlens.is_contiguous(), "cu_seqlens: int32");
  TORCH_CHECK(qkv.size(1) >= groups * (qpg + 2) * d, "qkv row is too narrow");
  (void)max_seqlen;
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t T = qkv.size(0);
  Tensor out = torch::empty({T, groups * qpg * d}, qkv.options());
  Tensor lse = torch::empty({groups * qpg, T}, qkv.options().dtype(torch::kFloat32));
  attn_varlen_fwd(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), lse.data_ptr<float>(), cu_seqlens.data_ptr<int>(),
                  (int)cu_seqlens.numel() - 1, (int)T, (int)groups, (int)qpg, (int)d, (float)scale, causal, status_of(status),
                  at::cuda::getCurrentCUDAStream().stream());
  return {out, lse};
}

// Returns dqkv with the layout of qkv.
Tensor attn_bwd(const Tensor& dout, const Tensor& qkv, const Tensor& out, const Tensor& lse, const Tensor& cu_seqlens,
                int64_t max_seqlen, int64_t groups, int64_t qpg, int64_t d, double scale, bool causal,
                const c10::optional<Tensor>& status) {
  TORCH_CHECK(dout.is_cuda() && dout.scalar_type() == torch::kBFloat16 && dout.is_contiguous(), "dout: contiguous bf16");
  TORCH_CHECK(out.is_contiguous() && out.sizes() == dout.sizes(), "out/dout mismatch");
  TORCH_CHECK(qkv.stride(1) == 1, "qkv: unit inner stride");
  (void)max_seqlen;
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t T = qkv.size(0);
  const int64_t hq = groups * qpg;
  Tensor dqkv = torch::empty({T, groups * (qpg + 2) * d}, qkv.options());
  Tensor delta = torch::empty({hq, T}, qkv.options().dtype(torch::kFloat32));
  Tensor dq_accum = torch::empty({T, hq * d}, qkv.options().dtype(torch::kFloat32));
  attn_varlen_bwd(dout.data_ptr(), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), lse.data_ptr<float>(),
                  delta.data_ptr<float>(), dq_accum.data_ptr<float>(), dqkv.data_ptr(), dqkv.stride(0),
                  cu_seqlens.data_ptr<int>(), (int)cu_seqlens.numel() - 1, (int)T, (int)groups, (int)qpg, (int)d,
                  (float)scale, causal, status_of(status), at::cuda::getCurrentCUDAStream().stream());
  return dqkv;
}

// Stick-breaking attention: returns (out [T, groups*qpg*d] bf16 without the head-bias term, rem [groups*qpg, T] fp32).
std::vector<Tensor> sb_attn_fwd(const Tensor& qkv, const Tensor& cu_seqlens, int64_t groups, int64_t qpg, int64_t d, double scale,
                                const c10::optional<Tensor>& status) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1, "qkv: [T, C] bf16");
  TORCH_CHECK(cu_seqlens.is_cuda() && cu_seqlens.scalar_type() == torch::kInt32 && cu_seqlens.is_contiguous(), "cu_seqlens: int32");
  TORCH_CHECK(qkv.size(1) >= groups * (qpg + 2) * d, "qkv row is too narrow");
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t T = qkv.size(0);
  Tensor out = torch::empty({T, groups * qpg * d}, qkv.options());
  Tensor rem = torch::empty({groups * qpg, T}, qkv.options().dtype(torch::kFloat32));
  sb_attn_varlen_fwd(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), rem.data_ptr<float>(), cu_seqlens.data_ptr<int>(),
                     (int)cu_seqlens.numel() - 1, (int)T, (int)groups, (int)qpg, (int)d, (float)scale, status_of(status),
                     at::cuda::getCurrentCUDAStream().stream());
  return {out, rem};
}

// Gradient of the fused qkv buffer from (d out, d rem); out / rem are the forward results.
Tensor sb_attn_bwd(const Tensor& dout, const Tensor& drem, const Tensor& qkv, const Tensor& out, const Tensor& rem, const Tensor& cu_seqlens,
                   int64_t groups, int64_t qpg, int64_t d, double scale, const c10::optional<Tensor>& status) {
  TORCH_CHECK(dout.is_cuda() && dout.scalar_type() == torch::kBFloat16 && dout.is_contiguous(), "dout: contiguous bf16");
  TORCH_CHECK(out.is_contiguous() && out.sizes() == dout.sizes(), "out/dout mismatch");
  TORCH_CHECK(qkv.scalar_type() == torch::kBFloat16 && qkv.stride(1) == 1, "qkv: bf16 with unit inner stride");
  TORCH_CHECK(rem.scalar_type() == torch::kFloat32 && drem.scalar_type() == torch::kFloat32 && rem.is_contiguous() && drem.is_contiguous() &&
                  rem.sizes() == drem.sizes(), "rem / drem: contiguous fp32 [heads, T]");
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t T = qkv.size(0);
  const int64_t hq = groups * qpg;
  TORCH_CHECK(rem.numel() == hq * T, "rem: [heads, T]");
  Tensor dqkv = torch::empty({T, groups * (qpg + 2) * d}, qkv.options());
  auto f32 = qkv.options().dtype(torch::kFloat32);
  Tensor gtot = torch::empty({hq, T}, f32);
  Tensor dk_accum = torch::empty({T, groups * d}, f32);
  Tensor dv_accum = torch::empty({T, groups * d}, f32);
  sb_attn_varlen_bwd(dout.data_ptr(), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), rem.data_ptr<float>(),
                     drem.data_ptr<float>(), gtot.data_ptr<float>(), dk_accum.data_ptr<float>(), dv_accum.data_ptr<float>(), dqkv.data_ptr(),
                     dqkv.stride(0), cu_seqlens.data_ptr<int>(), (int)cu_seqlens.numel() - 1, (int)T, (int)groups, (int)qpg, (int)d,
                     (float)scale, status_of(status), at::cuda::getCurrentCUDAStream().stream());
  return dqkv;
}

}  // namespace

// trace: int64 [16] on the device, or None to switch the counters off.
void attn_bwd_trace(const c10::optional<Tensor>& trace) {
  if (trace.has_value()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == torch::kInt64 && trace->numel() >= 16 && trace->is_contiguous(), "trace: int64 [16] on the device");
    attn_bwd_set_trace(reinterpret_cast<long long*>(trace->data_ptr<int64_t>()));
  } else {
    attn_bwd_set_trace(nullptr);
  }
}

void register_attention(pybind11::module_& m) {
  m.def("attn_bwd_trace", &attn_bwd_trace, pybind11::arg("trace") = pybind11::none());
  m.def("sb_attn_fwd", &sb_attn_fwd);
  m.def("sb_attn_bwd", &sb_attn_bwd);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
}

}  // namespace b200

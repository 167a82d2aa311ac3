// Python bindings of the peer-memory collectives. Peer buffers are not torch tensors in this process (they are
// mappings of other ranks' allocations), so they arrive as integer device addresses.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cmath>
#include <vector>

#include "peer.h"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

PeerPtrs table(const std::vector<int64_t>& ptrs, const char* what) {
  TORCH_CHECK(!ptrs.empty() && (int)ptrs.size() <= kMaxPeers, what, ": between 1 and ", kMaxPeers, " ranks");
  PeerPtrs t{};
  t.n = (int)ptrs.size();
  for (int i = 0; i < t.n; ++i) {
    TORCH_CHECK(ptrs[i] != 0 && ptrs[i] % 16 == 0, what, ": null or misaligned peer pointer");
    t.p[i] = reinterpret_cast<void*>(ptrs[i]);
  }
  return t;
}

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

void py_peer_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch, double timeout_seconds, Tensor& status) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32 && status.numel() >= 1, "status: int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(status.device());
  peer_barrier(table(flag_ptrs, "peer_barrier"), (int)rank, (uint32_t)epoch, timeout_seconds, status.data_ptr<int>(), stream_of(status));
}

void py_peer_reduce_scatter_f32(const std::vector<int64_t>& src_ptrs, int64_t multicast_ptr, Tensor& out, int64_t elem_offset,
                                double scale) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.is_contiguous(), "out: contiguous fp32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(out.device());
  peer_reduce_scatter_f32(table(src_ptrs, "peer_reduce_scatter"), reinterpret_cast<const void*>(multicast_ptr), out.data_ptr<float>(),
                          elem_offset, out.numel(), (float)scale, stream_of(out));
}

void py_peer_all_gather(const std::vector<int64_t>& ptrs, int64_t rank, int64_t shard_bytes, const Tensor& local) {
  TORCH_CHECK(local.is_cuda(), "local: the CUDA tensor of this rank's copy");
  TORCH_CHECK(rank >= 0 && rank < (int64_t)ptrs.size() && reinterpret_cast<int64_t>(local.data_ptr()) == ptrs[rank],
              "peer_all_gather: pointer table does not hold the local buffer at this rank");
  const c10::cuda::CUDAGuard guard(local.device());
  peer_all_gather(table(ptrs, "peer_all_gather"), (int)rank, shard_bytes, stream_of(local));
}

void py_adamw_step_bcast(Tensor& p, Tensor& m, Tensor& v, Tensor& g, const std::vector<int64_t>& dst_ptrs, int64_t multicast_ptr,
                         int64_t dst_elem_offset, double lr, double beta1, double beta2, double eps, double weight_decay, int64_t step,
                         const c10::optional<Tensor>& grad_scale, double grad_mul, bool zero_grad) {
  for (const Tensor* t : {&p, &m, &v, &g})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous() && t->numel() == p.numel(),
                "adamw_step_bcast: contiguous fp32 CUDA tensors of one size");
  const float* gs = nullptr;
  if (grad_scale.has_value()) {
    TORCH_CHECK(grad_scale->is_cuda() && grad_scale->scalar_type() == torch::kFloat32, "grad_scale: fp32 CUDA scalar");
    gs = grad_scale->data_ptr<float>();
  }
  const double bc1 = 1.0 - std::pow(beta1, (double)step);
  const double bc2 = 1.0 - std::pow(beta2, (double)step);
  const c10::cuda::CUDAGuard guard(p.device());
  adamw_step_bcast(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), table(dst_ptrs, "adamw_step_bcast"),
                   reinterpret_cast<void*>(multicast_ptr), dst_elem_offset, p.numel(), (float)lr, (float)beta1, (float)beta2, (float)eps,
                   (float)weight_decay, (float)bc1, (float)bc2, gs, (float)grad_mul, zero_grad, stream_of(p));
}

bool is_bf16_2d(const Tensor& t) { return t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.stride(1) == 1; }

// out[M, N] = gather(x)[M, K] . w^T (w: [N, K], or [K, N] when w_mn). staging: [M, K] contiguous with this rank's rows in place.
void py_ag_gemm(const std::vector<int64_t>& x_ptrs, Tensor& staging, Tensor& ready, int64_t epoch, const Tensor& w, Tensor& out, bool w_mn,
                int64_t rank, int64_t copy_ctas, Tensor& status) {
  TORCH_CHECK(is_bf16_2d(staging) && staging.is_contiguous(), "staging: contiguous bf16 [M, K]");
  TORCH_CHECK(is_bf16_2d(w) && is_bf16_2d(out), "w and out: bf16 matrices with unit inner stride");
  const int M = (int)staging.size(0), K = (int)staging.size(1);
  const int N = (int)(w_mn ? w.size(1) : w.size(0));
  TORCH_CHECK((w_mn ? w.size(0) : w.size(1)) == K && out.size(0) == M && out.size(1) == N, "ag_gemm: shape mismatch");
  TORCH_CHECK(ready.is_cuda() && ready.scalar_type() == torch::kInt32 && ready.numel() >= M / 128, "ready: int32 flags, one per 128 rows");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32, "status: int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(staging.device());
  ag_gemm_bf16(table(x_ptrs, "ag_gemm"), staging.data_ptr(), ready.data_ptr<int>(), (int)epoch, w.data_ptr(), out.data_ptr(), M, N, K,
               w.stride(0), out.stride(0), w_mn, (int)rank, (int)copy_ctas, status.data_ptr<int>(), stream_of(staging));
}

// For every rank r: slots_r[this rank][M / world, N] (bf16, contiguous) = (x[M, K] . w^T)[rows of r].
void py_gemm_rs(const Tensor& x, const Tensor& w, const std::vector<int64_t>& out_ptrs, bool w_mn, int64_t rank, Tensor& status) {
  TORCH_CHECK(is_bf16_2d(x) && is_bf16_2d(w), "x and w: bf16 matrices with unit inner stride");
  const int M = (int)x.size(0), K = (int)x.size(1);
  const int N = (int)(w_mn ? w.size(1) : w.size(0));
  TORCH_CHECK((w_mn ? w.size(0) : w.size(1)) == K, "gemm_rs: shape mismatch");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt32, "status: int32 CUDA tensor");
  const c10::cuda::CUDAGuard guard(x.device());
  gemm_rs_bf16(x.data_ptr(), w.data_ptr(), table(out_ptrs, "gemm_rs"), M, N, K, x.stride(0), w.stride(0), N, w_mn, (int)rank,
               status.data_ptr<int>(), stream_of(x));
}

}  // namespace

// out[rows, N] = sum over the `world` slots of slots[world, rows, N] (bf16, fp32 accumulation).
Tensor py_sum_slots(const Tensor& slots, int64_t world) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == torch::kBFloat16 && slots.is_contiguous() && slots.dim() == 3 && slots.size(0) == world,
              "slots: contiguous bf16 [world, rows, N]");
  const c10::cuda::CUDAGuard guard(slots.device());
  Tensor out = torch::empty({slots.size(1), slots.size(2)}, slots.options());
  sum_slots_bf16(slots.data_ptr(), out.data_ptr(), out.numel(), (int)world, stream_of(slots));
  return out;
}

void register_comm(py::module_& m) {
  m.def("sum_slots", &py_sum_slots);
  m.def("ag_gemm", &py_ag_gemm);
  m.def("gemm_rs", &py_gemm_rs);
  m.def("peer_barrier", &py_peer_barrier);
  m.def("peer_reduce_scatter_f32", &py_peer_reduce_scatter_f32);
  m.def("peer_all_gather", &py_peer_all_gather);
  m.def("adamw_step_bcast", &py_adamw_step_bcast);
}

}  // namespace b200

// Python bindings: thin adapters from torch tensors to the raw-pointer launch
// interface in ops/ops.h. Shape/dtype validation happens here; kernels run on
// the current CUDA stream of the calling thread.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <atomic>

#include "common/launch.h"
#include "ops/ops.h"

namespace b200 {
std::atomic<long long>& launch_counter() {
  static std::atomic<long long> c{0};
  return c;
}
// data/helpers.cpp
void register_data_helpers(pybind11::module_& m);
// ops/attention_*.cu, gemm/grouped_gemm.cu, comm/*.cu register themselves here
void register_attention(pybind11::module_& m);
void register_moe(pybind11::module_& m);
void register_comm(pybind11::module_& m);
void register_sequence(pybind11::module_& m);
void register_fp8(pybind11::module_& m);
void register_recurrent(pybind11::module_& m);
void register_moe_layout(pybind11::module_& m);
void register_ssd(pybind11::module_& m);
}  // namespace b200

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
}
inline void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, " must be fp32");
}
inline int* status_ptr(const c10::optional<Tensor>& s) {
  if (!s.has_value()) return nullptr;
  TORCH_CHECK(s->is_cuda() && s->scalar_type() == torch::kInt32, "status must be a CUDA int32 tensor");
  return s->data_ptr<int>();
}

// out[M,N] (+)= alpha * op(a) op(b)^T; see gemm_bf16.cu for operand conventions.
//  a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K] (b_mn=false) or [K,N] (b_mn=true). Inner dim contiguous.
// variant: 0 = choose (CTA-pair kernel for M >= 256), 1 = single-CTA kernel, 2 = CTA-pair kernel
int g_default_gemm_variant = 0;
void set_gemm_variant(int64_t v) { g_default_gemm_variant = (int)v; }

void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, bool accumulate, double alpha,
          const c10::optional<Tensor>& status, int64_t max_ctas, int64_t variant) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm operands must have a unit inner stride");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: contraction sizes differ (", K, " vs ", Kb, ")");
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm: output shape mismatch");
  TORCH_CHECK(out.is_cuda(), "out must be a CUDA tensor");
  int epi;
  if (out.scalar_type() == torch::kBFloat16) epi = accumulate ? 3 : 0;
  else if (out.scalar_type() == torch::kFloat32) epi = accumulate ? 2 : 1;
  else TORCH_CHECK(false, "gemm: output must be bf16 or fp32");
  const c10::cuda::CUDAGuard guard(a.device());
  if (variant == 0) variant = g_default_gemm_variant;
  const bool pair = variant == 2 || (variant == 0 && M >= 256);
  if (pair)
    b200::gemm_bf16_2sm(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                        out.stride(0), a_mn, b_mn, epi, (float)alpha, status_ptr(status), (int)max_ctas, cur_stream());
  else
    b200::gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                    out.stride(0), a_mn, b_mn, epi, (float)alpha, status_ptr(status), (int)max_ctas, cur_stream());
}

// Knobs of the CTA-pair GEMM for micro-benchmarks: raster group, k skew, register-store epilogue, trace buffer
// (int64 tensor with 8 words per CTA; pass None to switch tracing off).
void gemm_tuning(int64_t group, int64_t k_skew, bool direct_store, const c10::optional<Tensor>& trace, int64_t split_k) {
  auto& t = b200::pair_gemm_tuning();
  t.split_k = (int)split_k;
  t.group = (int)group;
  t.k_skew = (int)k_skew;
  t.direct_store = direct_store ? 1 : 0;
  t.trace = nullptr;
  if (trace.has_value()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == torch::kInt64 && trace->numel() >= 8 * 148, "trace must be a CUDA int64 tensor of >= 8 * 148 words");
    t.trace = reinterpret_cast<long long*>(trace->data_ptr<int64_t>());
  }
}

// fc = x w^T ([T, 2I], both halves kept for backward) and act = fc[:, :I] * silu(fc[:, I:]) in one launch.
void gemm_swiglu(const Tensor& x, const Tensor& w, Tensor& fc, Tensor& act, const c10::optional<Tensor>& status) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  check_bf16(fc, "fc");
  check_bf16(act, "act");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && fc.dim() == 2 && act.dim() == 2, "gemm_swiglu operands must be 2-D");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && fc.stride(1) == 1 && act.stride(1) == 1, "gemm_swiglu operands must have a unit inner stride");
  const int64_t M = x.size(0), K = x.size(1), I = w.size(0) / 2;
  TORCH_CHECK(w.size(1) == K && w.size(0) == 2 * I, "gemm_swiglu: weight must be [2I, K]");
  TORCH_CHECK(fc.size(0) == M && fc.size(1) == 2 * I && act.size(0) == M && act.size(1) == I, "gemm_swiglu: output shape mismatch");
  const c10::cuda::CUDAGuard guard(x.device());
  b200::gemm_bf16_swiglu(x.data_ptr(), w.data_ptr(), fc.data_ptr(), act.data_ptr(), (int)M, (int)I, (int)K, x.stride(0), w.stride(0),
                         fc.stride(0), act.stride(0), status_ptr(status), cur_stream());
}

// dfc = [d(up) | d(gate)] and act = up * silu(gate) from dy, the down-projection weight w [H, I] and the saved projection fc.
void gemm_swiglu_bwd(const Tensor& dy, const Tensor& w, const Tensor& fc, Tensor& dfc, Tensor& act, const c10::optional<Tensor>& status) {
  check_bf16(dy, "dy");
  check_bf16(w, "w");
  check_bf16(fc, "fc");
  check_bf16(dfc, "dfc");
  check_bf16(act, "act");
  const Tensor* operands[] = {&dy, &w, &fc, &dfc, &act};  // dfc / act are non-const references: no common initializer_list type
  for (const Tensor* t : operands) TORCH_CHECK(t->dim() == 2 && t->stride(1) == 1, "gemm_swiglu_bwd operands must be matrices with a unit inner stride");
  const int64_t M = dy.size(0), K = dy.size(1), I = w.size(1);
  TORCH_CHECK(w.size(0) == K && fc.size(0) == M && fc.size(1) == 2 * I && dfc.size(0) == M && dfc.size(1) == 2 * I && act.size(0) == M && act.size(1) == I,
              "gemm_swiglu_bwd: shape mismatch");
  const c10::cuda::CUDAGuard guard(dy.device());
  b200::gemm_bf16_swiglu_bwd(dy.data_ptr(), w.data_ptr(), fc.data_ptr(), dfc.data_ptr(), act.data_ptr(), (int)M, (int)I, (int)K, dy.stride(0),
                             w.stride(0), fc.stride(0), dfc.stride(0), act.stride(0), status_ptr(status), cur_stream());
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& residual, const Tensor& w, double eps,
                                bool want_sum) {
  check_bf16(x, "x");
  check_bf16(w, "weight");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "rmsnorm inputs must be contiguous");
  const int64_t H = x.size(-1);
  const int64_t T = x.numel() / H;
  TORCH_CHECK(w.numel() == H, "rmsnorm weight size mismatch");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({T}, x.options().dtype(torch::kFloat32));
  Tensor h;
  const void* rp = nullptr;
  void* hp = nullptr;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == x.numel(), "residual shape mismatch");
    rp = residual->data_ptr();
    if (want_sum) {
      h = torch::empty_like(x);
      hp = h.data_ptr();
    }
  }
  b200::rmsnorm_fwd(x.data_ptr(), rp, w.data_ptr(), y.data_ptr(), hp, rstd.data_ptr<float>(), (int)T, (int)H,
                    (float)eps, cur_stream());
  if (hp) return {y, rstd, h};
  return {y, rstd};
}

// Returns dh (bf16). dw (fp32 [H]) is accumulated into when accumulate_dw, else overwritten.
Tensor rmsnorm_bwd(const Tensor& dy, const Tensor& h, const Tensor& w, const Tensor& rstd,
                   const c10::optional<Tensor>& dres, Tensor& dw, bool accumulate_dw) {
  check_bf16(dy, "dy");
  check_bf16(h, "h");
  check_bf16(w, "weight");
  check_f32(rstd, "rstd");
  check_f32(dw, "dw");
  TORCH_CHECK(dy.is_contiguous() && h.is_contiguous(), "rmsnorm_bwd inputs must be contiguous");
  const int64_t H = h.size(-1);
  const int64_t T = h.numel() / H;
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dh = torch::empty_like(h);
  Tensor partial = torch::empty({b200::rmsnorm_bwd_partial_rows((int)T), H}, h.options().dtype(torch::kFloat32));
  const void* drp = nullptr;
  if (dres.has_value()) {
    check_bf16(*dres, "dres");
    TORCH_CHECK(dres->is_contiguous(), "dres must be contiguous");
    drp = dres->data_ptr();
  }
  b200::rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), drp, dh.data_ptr(),
                    partial.data_ptr<float>(), dw.data_ptr<float>(), accumulate_dw, (int)T, (int)H, cur_stream());
  return dh;
}

const int* tile_owner_ptr(const c10::optional<Tensor>& t, int64_t rows) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt32 && t->is_contiguous() && t->numel() * 128 >= rows, "tile_owner: int32, one entry per 128 rows");
  return t->data_ptr<int>();
}

Tensor swiglu_fwd(const Tensor& x, const c10::optional<Tensor>& tile_owner, int64_t owners) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous(), "swiglu input must be contiguous");
  const int64_t I = x.size(-1) / 2;
  const int64_t T = x.numel() / (2 * I);
  auto sizes = x.sizes().vec();
  sizes.back() = I;
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty(sizes, x.options());
  b200::swiglu_fwd(x.data_ptr(), y.data_ptr(), T, (int)I, cur_stream(), tile_owner_ptr(tile_owner, T), (int)owners);
  return y;
}

std::vector<Tensor> swiglu_bwd(const Tensor& dy, const Tensor& x, bool recompute_y, const c10::optional<Tensor>& tile_owner, int64_t owners) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous(), "swiglu_bwd inputs must be contiguous");
  const int64_t I = x.size(-1) / 2;
  const int64_t T = x.numel() / (2 * I);
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor y;
  void* yp = nullptr;
  if (recompute_y) {
    y = torch::empty_like(dy);
    yp = y.data_ptr();
  }
  b200::swiglu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), yp, T, (int)I, cur_stream(), tile_owner_ptr(tile_owner, T), (int)owners);
  if (recompute_y) return {dx, y};
  return {dx};
}

void rope_(Tensor& qkv, const Tensor& cos_t, const Tensor& sin_t, const c10::optional<Tensor>& position_ids,
           int64_t num_kv_groups, int64_t q_per_group, int64_t head_dim, int64_t rope_dim, bool inverse) {
  check_bf16(qkv, "qkv");
  check_f32(cos_t, "cos");
  check_f32(sin_t, "sin");
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1, "qkv must be [T, C] with unit inner stride");
  TORCH_CHECK(qkv.size(1) >= num_kv_groups * (q_per_group + 2) * head_dim, "qkv row is too narrow");
  TORCH_CHECK(cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(-1) == rope_dim / 2, "bad rope tables");
  const int* pos = nullptr;
  if (position_ids.has_value()) {
    TORCH_CHECK(position_ids->scalar_type() == torch::kInt32 && position_ids->is_contiguous(),
                "position_ids must be contiguous int32");
    pos = position_ids->data_ptr<int>();
  }
  const c10::cuda::CUDAGuard guard(qkv.device());
  b200::rope_inplace(qkv.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), pos, (int)qkv.size(0),
                     qkv.stride(0), (int)num_kv_groups, (int)q_per_group, (int)head_dim, (int)rope_dim, inverse,
                     cur_stream());
}

Tensor embedding_fwd(const Tensor& weight, const Tensor& ids, double scale) {
  check_bf16(weight, "weight");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids must be int64 CUDA");
  TORCH_CHECK(weight.is_contiguous(), "weight must be contiguous");
  const c10::cuda::CUDAGuard guard(weight.device());
  auto sizes = ids.sizes().vec();
  sizes.push_back(weight.size(1));
  Tensor out = torch::empty(sizes, weight.options());
  b200::embedding_fwd(weight.data_ptr(), ids.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()) : nullptr,
                      out.data_ptr(), (int)ids.numel(), (int)weight.size(1), (float)scale, cur_stream());
  return out;
}

void embedding_bwd(const Tensor& dy, const Tensor& ids, Tensor& dweight, double scale) {
  check_bf16(dy, "dy");
  check_f32(dweight, "dweight");
  TORCH_CHECK(dy.is_contiguous() && dweight.is_contiguous() && ids.is_contiguous(), "embedding_bwd needs contiguous inputs");
  const c10::cuda::CUDAGuard guard(dy.device());
  b200::embedding_bwd(dy.data_ptr(), reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dweight.data_ptr<float>(),
                      (int)ids.numel(), (int)dweight.size(1), (float)scale, cur_stream());
}

void cast_f32_to_bf16(const Tensor& src, Tensor& dst) {
  check_f32(src, "src");
  check_bf16(dst, "dst");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel(), "cast: shape mismatch");
  const c10::cuda::CUDAGuard guard(src.device());
  b200::cast_f32_to_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), cur_stream());
}

void cast_bf16_to_f32(const Tensor& src, Tensor& dst, bool accumulate, double scale) {
  check_bf16(src, "src");
  check_f32(dst, "dst");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel(), "cast: shape mismatch");
  const c10::cuda::CUDAGuard guard(src.device());
  b200::cast_bf16_to_f32(src.data_ptr(), dst.data_ptr<float>(), src.numel(), accumulate, (float)scale, cur_stream());
}

Tensor add_bf16(const Tensor& a, const Tensor& b) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.numel() == b.numel(), "add: shape mismatch");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = torch::empty_like(a);
  b200::add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream());
  return out;
}

// out[0] (+)= sum(x^2) with a fixed reduction order.
void sumsq(const Tensor& x, Tensor& out, bool accumulate) {
  check_f32(x, "x");
  check_f32(out, "out");
  TORCH_CHECK(x.is_contiguous(), "sumsq input must be contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor partials = torch::empty({b200::sumsq_partial_count(x.numel())}, x.options());
  b200::sumsq_f32(x.data_ptr<float>(), x.numel(), partials.data_ptr<float>(), out.data_ptr<float>(), accumulate,
                  cur_stream());
}

void clip_coef(const Tensor& total_sq, double max_norm, Tensor& coef, Tensor& norm) {
  check_f32(total_sq, "total_sq");
  check_f32(coef, "coef");
  check_f32(norm, "norm");
  const c10::cuda::CUDAGuard guard(total_sq.device());
  b200::clip_coef(total_sq.data_ptr<float>(), (float)max_norm, coef.data_ptr<float>(), norm.data_ptr<float>(), cur_stream());
}

void adamw_step(Tensor& p, Tensor& m, Tensor& v, Tensor& g, const c10::optional<Tensor>& p_bf16, double lr, double beta1,
                double beta2, double eps, double weight_decay, int64_t step, const c10::optional<Tensor>& grad_scale,
                double grad_mul, bool zero_grad) {
  check_f32(p, "p");
  check_f32(m, "m");
  check_f32(v, "v");
  check_f32(g, "g");
  TORCH_CHECK(p.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous(), "adamw: contiguous");
  TORCH_CHECK(p.numel() == m.numel() && p.numel() == v.numel() && p.numel() == g.numel(), "adamw: size mismatch");
  void* pb = nullptr;
  if (p_bf16.has_value()) {
    check_bf16(*p_bf16, "p_bf16");
    TORCH_CHECK(p_bf16->is_contiguous() && p_bf16->numel() == p.numel(), "adamw: bf16 copy size mismatch");
    pb = p_bf16->data_ptr();
  }
  const float* gs = nullptr;
  if (grad_scale.has_value()) {
    check_f32(*grad_scale, "grad_scale");
    gs = grad_scale->data_ptr<float>();
  }
  const double bc1 = 1.0 - std::pow(beta1, (double)step);
  const double bc2 = 1.0 - std::pow(beta2, (double)step);
  const c10::cuda::CUDAGuard guard(p.device());
  b200::adamw_step(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), pb, p.numel(),
                   (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, (float)bc1, (float)bc2, gs,
                   (float)grad_mul, zero_grad, cur_stream());
}

// In place: logits <- gradient. Returns per-row loss (fp32 [T]).
Tensor cross_entropy_(Tensor& logits, const Tensor& labels, double logit_scale, double grad_scale, int64_t ignore_index,
                      bool write_grad) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [T, V] with unit inner stride");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == torch::kInt64 && labels.is_contiguous(), "labels: int64 CUDA");
  TORCH_CHECK(labels.numel() == logits.size(0), "labels/logits row mismatch");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat32));
  b200::cross_entropy_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                              loss.data_ptr<float>(), nullptr, (int)logits.size(0), (int)logits.size(1), logits.stride(0),
                              (float)logit_scale, (float)grad_scale, ignore_index, write_grad, cur_stream());
  return loss;
}

// Vocabulary-parallel cross entropy, this rank's part: stats[T, 3] = (row max, sum of exp relative to it, target logit or 0).
Tensor ce_shard_stats(const Tensor& logits, const Tensor& labels, int64_t vocab_start, int64_t ignore_index) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [T, V] with unit inner stride");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == torch::kInt64 && labels.is_contiguous() && labels.numel() == logits.size(0), "labels: int64 [T]");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor stats = torch::empty({logits.size(0), 3}, logits.options().dtype(torch::kFloat32));
  b200::cross_entropy_shard_stats(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), stats.data_ptr<float>(),
                                  (int)logits.size(0), (int)logits.size(1), logits.stride(0), vocab_start, ignore_index, cur_stream());
  return stats;
}

// grad[T, V] (bf16) = row_scale * (exp(logits - lse) - onehot(label - vocab_start)); zero rows for ignored labels.
Tensor ce_shard_grad(const Tensor& logits, const Tensor& labels, const Tensor& lse, const Tensor& row_scale, int64_t vocab_start,
                     int64_t ignore_index) {
  check_bf16(logits, "logits");
  check_f32(lse, "lse");
  check_f32(row_scale, "row_scale");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [T, V] with unit inner stride");
  TORCH_CHECK(lse.is_contiguous() && row_scale.is_contiguous() && lse.numel() == logits.size(0) && row_scale.numel() == logits.size(0), "lse / row_scale: fp32 [T]");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == torch::kInt64 && labels.is_contiguous() && labels.numel() == logits.size(0), "labels: int64 [T]");
  const c10::cuda::CUDAGuard guard(logits.device());
  Tensor grad = torch::empty({logits.size(0), logits.size(1)}, logits.options());
  b200::cross_entropy_shard_grad(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), lse.data_ptr<float>(),
                                 row_scale.data_ptr<float>(), grad.data_ptr(), (int)logits.size(0), (int)logits.size(1), logits.stride(0),
                                 vocab_start, ignore_index, cur_stream());
  return grad;
}

long long launch_count() { return b200::launch_counter().load(); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a kernels of the engine";
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_mn") = false,
        py::arg("b_mn") = false, py::arg("accumulate") = false, py::arg("alpha") = 1.0, py::arg("status") = py::none(),
        py::arg("max_ctas") = 0, py::arg("variant") = 0);
  m.def("set_gemm_variant", &set_gemm_variant);
  m.def("gemm_tuning", &gemm_tuning, py::arg("group") = 0, py::arg("k_skew") = 0, py::arg("direct_store") = false, py::arg("trace") = py::none(), py::arg("split_k") = 0);
  m.def("gemm_swiglu_bwd", &gemm_swiglu_bwd, "down-projection data gradient with the SwiGLU backward in its epilogue", py::arg("dy"), py::arg("w"),
        py::arg("fc"), py::arg("dfc"), py::arg("act"), py::arg("status") = py::none());
  m.def("gemm_swiglu", &gemm_swiglu, "c_fc GEMM with the SwiGLU activation in its epilogue", py::arg("x"), py::arg("w"), py::arg("fc"), py::arg("act"), py::arg("status") = py::none());
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("eps"),
        py::arg("want_sum") = true);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd, py::arg("x"), py::arg("tile_owner") = py::none(), py::arg("owners") = 0);
  m.def("swiglu_bwd", &swiglu_bwd, py::arg("dy"), py::arg("x"), py::arg("recompute_y"), py::arg("tile_owner") = py::none(), py::arg("owners") = 0);
  m.def("rope_", &rope_);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cast_f32_to_bf16", &cast_f32_to_bf16);
  m.def("cast_bf16_to_f32", &cast_bf16_to_f32);
  m.def("add_bf16", &add_bf16);
  m.def("sumsq", &sumsq);
  m.def("clip_coef", &clip_coef);
  m.def("adamw_step", &adamw_step);
  m.def("cross_entropy_", &cross_entropy_);
  m.def("ce_shard_stats", &ce_shard_stats);
  m.def("ce_shard_grad", &ce_shard_grad);
  m.def("launch_count", &launch_count);
  b200::register_attention(m);
  b200::register_moe(m);
  b200::register_comm(m);
  b200::register_sequence(m);
  b200::register_fp8(m);
  b200::register_recurrent(m);
  b200::register_moe_layout(m);
  b200::register_ssd(m);
  b200::register_data_helpers(m);
}

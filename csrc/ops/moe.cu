// Row movement kernels of the mixture-of-experts path. Rows live either in this GPU's memory or, under expert
// parallelism, in a peer's buffer that is mapped into this process (plain 16-byte peer loads, one warp per row; no
// multicast of any kind). Source buffers are given as a small table of per-rank base pointers.
//
//   gather : out[r] = scale * src[rank(e)][token(e)]  for e = src_entry[r] >= 0, zero rows otherwise
//   combine: out[t] = sum_s w[t, s] * rows[rank(g)][row(g)]  with g = dest_row[t * k + s]
//   rowdot : out[e] = <a[row(e)], b[row(e)]>   (router-weight gradient)
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "ops.h"

namespace b200 {

void grouped_rows_gemm(const void* A, long long lda, const void* W, void* C, long long ldc, const int* tile_expert,
                       int max_m_tiles, int num_experts, int N, int K, bool w_mn, int* status, cudaStream_t stream);
void grouped_rows_dispatch_gemm(const void* const* src_ptrs, int num_ranks, const int* src_entry, int entries_per_rank, int k, void* a_rows,
                                int* ready, int copy_ctas, const void* W, void* C, long long ldc, const int* tile_expert, int max_m_tiles,
                                int num_experts, int N, int K, bool w_mn, int* status, cudaStream_t stream);
void grouped_wgrad_gemm(const void* dY, const void* X, float* dW, const int* padded_offsets, long long total_rows,
                        int num_experts, int Nw, int Kw, bool accumulate, int* status, cudaStream_t stream);

namespace {

constexpr int MAX_RANKS = 16;

struct PtrTable {
  const void* p[MAX_RANKS];
};

// entry e (global numbering over ranks) -> (rank, token): rank = e / entries_per_rank, token = (e % entries_per_rank) / k
__global__ void moe_gather_kernel(PtrTable src, PtrTable scale, const int* __restrict__ src_entry, uint4* __restrict__ out,
                                  int rows, int Hv, int entries_per_rank, int k, const int* __restrict__ tile_owner, int owners) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  if (tile_owner != nullptr && tile_owner[warp >> 7] >= owners) return;  // tile beyond the used rows: nothing reads it
  const int e = src_entry[warp];
  uint4* dst = out + (size_t)warp * Hv;
  if (e < 0) {
    for (int i = lane; i < Hv; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int rank = e / entries_per_rank;
  const int local = e - rank * entries_per_rank;
  const int token = local / k;
  const uint4* s = reinterpret_cast<const uint4*>(src.p[rank]) + (size_t)token * Hv;
  const float* sc = reinterpret_cast<const float*>(scale.p[rank]);
  if (sc == nullptr) {
    for (int i = lane; i < Hv; i += 32) dst[i] = s[i];
  } else {
    const float w = sc[local];
    for (int i = lane; i < Hv; i += 32) {
      const uint4 v = s[i];
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      dst[i] = make_uint4(pack_bf16x2(a.x * w, a.y * w), pack_bf16x2(b.x * w, b.y * w), pack_bf16x2(c.x * w, c.y * w),
                          pack_bf16x2(d.x * w, d.y * w));
    }
  }
}

// dest_row[g]: global row id = rank * rows_per_rank + local row (or -1: entry dropped)
template <int MAXV>
__global__ void moe_combine_kernel(PtrTable rows, const int* __restrict__ dest_row, const float* __restrict__ weights,
                                   uint4* __restrict__ out, int T, int Hv, int k, long long rows_per_rank) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  float acc[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  for (int s = 0; s < k; ++s) {
    const int g = dest_row[warp * k + s];
    if (g < 0) continue;
    const int rank = (int)(g / rows_per_rank);
    const long long local = g - (long long)rank * rows_per_rank;
    const float w = weights ? weights[warp * k + s] : 1.f;
    const uint4* src = reinterpret_cast<const uint4*>(rows.p[rank]) + (size_t)local * Hv;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = lane + j * 32;
      if (i < Hv) {
        const uint4 v = src[i];
        const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
        acc[j][0] += w * a.x; acc[j][1] += w * a.y; acc[j][2] += w * b.x; acc[j][3] += w * b.y;
        acc[j][4] += w * c.x; acc[j][5] += w * c.y; acc[j][6] += w * d.x; acc[j][7] += w * d.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = lane + j * 32;
    if (i < Hv)
      out[(size_t)warp * Hv + i] = make_uint4(pack_bf16x2(acc[j][0], acc[j][1]), pack_bf16x2(acc[j][2], acc[j][3]),
                                              pack_bf16x2(acc[j][4], acc[j][5]), pack_bf16x2(acc[j][6], acc[j][7]));
  }
}

// out[e] = <a[row], b[row]> with row = dest_row[e] (local rows only), 0 for dropped entries
__global__ void moe_rowdot_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, const int* __restrict__ dest_row,
                                  float* __restrict__ out, int entries, int Hv) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= entries) return;
  const int row = dest_row[warp];
  float s = 0.f;
  if (row >= 0) {
    const uint4* x = a + (size_t)row * Hv;
    const uint4* y = b + (size_t)row * Hv;
    for (int i = lane; i < Hv; i += 32) {
      const uint4 u = x[i], v = y[i];
      const float2 u0 = unpack_bf16x2(u.x), u1 = unpack_bf16x2(u.y), u2 = unpack_bf16x2(u.z), u3 = unpack_bf16x2(u.w);
      const float2 v0 = unpack_bf16x2(v.x), v1 = unpack_bf16x2(v.y), v2 = unpack_bf16x2(v.z), v3 = unpack_bf16x2(v.w);
      s += u0.x * v0.x + u0.y * v0.y + u1.x * v1.x + u1.y * v1.y + u2.x * v2.x + u2.y * v2.y + u3.x * v3.x + u3.y * v3.y;
    }
  }
  s = warp_sum(s);
  if (lane == 0) out[warp] = s;
}

// rows[r] *= w[r] (bf16 rows, fp32 per-row factors)
__global__ void scale_rows_kernel(uint4* __restrict__ x, const float* __restrict__ w, long long rows, int Hv,
                                  const int* __restrict__ tile_owner, int owners) {
  const long long total = rows * Hv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    if (tile_owner != nullptr && tile_owner[(idx / Hv) >> 7] >= owners) continue;
    const float f = w[idx / Hv];
    const uint4 v = x[idx];
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    x[idx] = make_uint4(pack_bf16x2(a.x * f, a.y * f), pack_bf16x2(b.x * f, b.y * f), pack_bf16x2(c.x * f, c.y * f),
                        pack_bf16x2(d.x * f, d.y * f));
  }
}

// Backward of the weighted expert activation, one warp per expert row r with routing weight w = row_weight[r]:
//   act_w[r] = w * up * silu(gate)                      (the operand of the second GEMM's weight gradient)
//   dfc[r]   = [w * dact * silu(gate) | w * dact * up * dsilu(gate)]
//   dot[r]   = <dact[r], up * silu(gate)>               (gradient of the routing weight)
// from fc[r] = [up | gate] and dact[r], each read once. Rows of unused tiles are skipped.
__global__ void moe_swiglu_bwd_kernel(const uint4* __restrict__ fc, const uint4* __restrict__ dact, const float* __restrict__ row_weight,
                                      uint4* __restrict__ act_w, uint4* __restrict__ dfc, float* __restrict__ dot, long long rows,
                                      int Iv, const int* __restrict__ tile_owner, int owners) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  if (tile_owner != nullptr && tile_owner[row >> 7] >= owners) return;
  const float w = row_weight[row];
  const uint4* up = fc + row * 2 * Iv;
  const uint4* gate = up + Iv;
  const uint4* dy = dact + row * Iv;
  float s = 0.f;
  for (int i = lane; i < Iv; i += 32) {
    const uint4 u = up[i], g = gate[i], d = dy[i];
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w}, gg[4] = {g.x, g.y, g.z, g.w}, dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t du[4], dg[4], yy[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(uu[e]), b = unpack_bf16x2(gg[e]), q = unpack_bf16x2(dd[e]);
      const float s0 = sigmoid_fast(b.x), s1 = sigmoid_fast(b.y);
      const float silu0 = b.x * s0, silu1 = b.y * s1;
      const float ds0 = s0 * (1.f + b.x * (1.f - s0)), ds1 = s1 * (1.f + b.y * (1.f - s1));
      const float y0 = a.x * silu0, y1 = a.y * silu1;
      s += q.x * y0 + q.y * y1;
      const float q0 = q.x * w, q1 = q.y * w;
      du[e] = pack_bf16x2(q0 * silu0, q1 * silu1);
      dg[e] = pack_bf16x2(q0 * a.x * ds0, q1 * a.y * ds1);
      yy[e] = pack_bf16x2(y0 * w, y1 * w);
    }
    act_w[row * Iv + i] = make_uint4(yy[0], yy[1], yy[2], yy[3]);
    dfc[row * 2 * Iv + i] = make_uint4(du[0], du[1], du[2], du[3]);
    dfc[row * 2 * Iv + Iv + i] = make_uint4(dg[0], dg[1], dg[2], dg[3]);
  }
  s = warp_sum(s);
  if (lane == 0) dot[row] = s;
}

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline int* status_of(const c10::optional<Tensor>& s) { return s.has_value() ? s->data_ptr<int>() : nullptr; }

PtrTable table_from(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && ptrs.size() <= MAX_RANKS, "between 1 and 16 source buffers are supported");
  PtrTable t = {};
  for (size_t i = 0; i < ptrs.size(); ++i) t.p[i] = reinterpret_cast<const void*>(ptrs[i]);
  return t;
}

// src_ptrs / scale_ptrs: device addresses of the per-rank [T, H] bf16 buffers and [T * k] fp32 scales (0 = none).
Tensor moe_gather(const std::vector<int64_t>& src_ptrs, const std::vector<int64_t>& scale_ptrs, const Tensor& src_entry,
                  int64_t H, int64_t entries_per_rank, int64_t k, const Tensor& like, const c10::optional<Tensor>& tile_owner,
                  int64_t owners) {
  TORCH_CHECK(src_entry.is_cuda() && src_entry.scalar_type() == torch::kInt32 && src_entry.is_contiguous(), "src_entry: int32");
  TORCH_CHECK(H % 8 == 0, "hidden size must be a multiple of 8");
  const c10::cuda::CUDAGuard guard(src_entry.device());
  const int64_t rows = src_entry.numel();
  Tensor out = torch::empty({rows, H}, like.options().dtype(torch::kBFloat16));
  PtrTable scale = {};
  if (!scale_ptrs.empty()) scale = table_from(scale_ptrs);
  const int threads = 256;
  const long long blocks = (rows * 32 + threads - 1) / threads;
  moe_gather_kernel<<<(unsigned)blocks, threads, 0, cur_stream()>>>(table_from(src_ptrs), scale, src_entry.data_ptr<int>(),
                                                                    reinterpret_cast<uint4*>(out.data_ptr()), (int)rows,
                                                                    (int)(H / 8), (int)entries_per_rank, (int)k,
                                                                    tile_owner.has_value() ? tile_owner->data_ptr<int>() : nullptr, (int)owners);
  count_launch();
  check_cuda(cudaGetLastError(), "moe_gather launch");
  return out;
}

Tensor moe_combine(const std::vector<int64_t>& row_ptrs, const Tensor& dest_row, const c10::optional<Tensor>& weights,
                   int64_t T, int64_t H, int64_t k, int64_t rows_per_rank, const Tensor& like) {
  TORCH_CHECK(dest_row.scalar_type() == torch::kInt32 && dest_row.is_contiguous() && dest_row.numel() == T * k, "dest_row: int32 [T*k]");
  TORCH_CHECK(H % 8 == 0 && H <= 8 * 32 * 32, "hidden size must be a multiple of 8 and at most 8192");
  const float* w = nullptr;
  if (weights.has_value()) {
    TORCH_CHECK(weights->scalar_type() == torch::kFloat32 && weights->is_contiguous() && weights->numel() == T * k, "weights: fp32 [T*k]");
    w = weights->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(dest_row.device());
  Tensor out = torch::empty({T, H}, like.options().dtype(torch::kBFloat16));
  const int Hv = (int)(H / 8);
  const int threads = 256;
  const long long blocks = (T * 32 + threads - 1) / threads;
  const PtrTable rows = table_from(row_ptrs);
  auto o = reinterpret_cast<uint4*>(out.data_ptr());
#define COMBINE(V) moe_combine_kernel<V><<<(unsigned)blocks, threads, 0, cur_stream()>>>(rows, dest_row.data_ptr<int>(), w, o, (int)T, Hv, (int)k, rows_per_rank)
  if (Hv <= 64) COMBINE(2);
  else if (Hv <= 128) COMBINE(4);
  else if (Hv <= 256) COMBINE(8);
  else if (Hv <= 512) COMBINE(16);
  else COMBINE(32);
#undef COMBINE
  count_launch();
  check_cuda(cudaGetLastError(), "moe_combine launch");
  return out;
}

Tensor moe_rowdot(const Tensor& a, const Tensor& b, const Tensor& dest_row) {
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16 && a.is_contiguous() && b.is_contiguous(), "bf16 rows");
  TORCH_CHECK(a.sizes() == b.sizes() && a.size(1) % 8 == 0, "row shapes");
  const c10::cuda::CUDAGuard guard(a.device());
  const int64_t n = dest_row.numel();
  Tensor out = torch::empty({n}, a.options().dtype(torch::kFloat32));
  const int threads = 256;
  const long long blocks = (n * 32 + threads - 1) / threads;
  moe_rowdot_kernel<<<(unsigned)blocks, threads, 0, cur_stream()>>>(reinterpret_cast<const uint4*>(a.data_ptr()),
                                                                    reinterpret_cast<const uint4*>(b.data_ptr()),
                                                                    dest_row.data_ptr<int>(), out.data_ptr<float>(), (int)n,
                                                                    (int)(a.size(1) / 8));
  count_launch();
  check_cuda(cudaGetLastError(), "moe_rowdot launch");
  return out;
}

void scale_rows_(Tensor& x, const Tensor& w, const c10::optional<Tensor>& tile_owner, int64_t owners) {
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.size(1) % 8 == 0, "bf16 rows");
  TORCH_CHECK(w.scalar_type() == torch::kFloat32 && w.numel() == x.size(0), "one fp32 factor per row");
  const c10::cuda::CUDAGuard guard(x.device());
  const long long total = x.size(0) * (x.size(1) / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  scale_rows_kernel<<<(unsigned)blocks, 256, 0, cur_stream()>>>(reinterpret_cast<uint4*>(x.data_ptr()), w.data_ptr<float>(),
                                                                x.size(0), (int)(x.size(1) / 8),
                                                                tile_owner.has_value() ? tile_owner->data_ptr<int>() : nullptr, (int)owners);
  count_launch();
  check_cuda(cudaGetLastError(), "scale_rows launch");
}

// (act_w [rows, I], dfc [rows, 2I], dot [rows] fp32) from fc [rows, 2I], dact [rows, I], row_weight [rows] fp32.
// Rows of skipped tiles are left unwritten in act_w / dfc; dot is zero there.
std::vector<Tensor> moe_swiglu_bwd(const Tensor& fc, const Tensor& dact, const Tensor& row_weight,
                                   const c10::optional<Tensor>& tile_owner, int64_t owners) {
  TORCH_CHECK(fc.scalar_type() == torch::kBFloat16 && dact.scalar_type() == torch::kBFloat16 && fc.is_contiguous() && dact.is_contiguous(), "bf16 rows");
  TORCH_CHECK(fc.dim() == 2 && dact.dim() == 2 && fc.size(0) == dact.size(0) && fc.size(1) == 2 * dact.size(1) && dact.size(1) % 8 == 0, "fc: [rows, 2I], dact: [rows, I]");
  TORCH_CHECK(row_weight.scalar_type() == torch::kFloat32 && row_weight.numel() == fc.size(0) && row_weight.is_contiguous(), "one fp32 weight per row");
  const int64_t rows = fc.size(0);
  if (tile_owner.has_value())
    TORCH_CHECK(tile_owner->scalar_type() == torch::kInt32 && tile_owner->numel() * 128 >= rows, "tile_owner: int32, one per 128 rows");
  const c10::cuda::CUDAGuard guard(fc.device());
  Tensor act_w = torch::empty_like(dact);
  Tensor dfc = torch::empty_like(fc);
  Tensor dot = torch::zeros({rows}, fc.options().dtype(torch::kFloat32));
  if (rows == 0) return {act_w, dfc, dot};
  const int threads = 256;
  const long long blocks = (rows * 32 + threads - 1) / threads;
  moe_swiglu_bwd_kernel<<<(unsigned)blocks, threads, 0, cur_stream()>>>(
      reinterpret_cast<const uint4*>(fc.data_ptr()), reinterpret_cast<const uint4*>(dact.data_ptr()), row_weight.data_ptr<float>(),
      reinterpret_cast<uint4*>(act_w.data_ptr()), reinterpret_cast<uint4*>(dfc.data_ptr()), dot.data_ptr<float>(), rows,
      (int)(dact.size(1) / 8), tile_owner.has_value() ? tile_owner->data_ptr<int>() : nullptr, (int)owners);
  count_launch();
  check_cuda(cudaGetLastError(), "moe_swiglu_bwd launch");
  return {act_w, dfc, dot};
}

// out[rows, N] = a[rows, K] * op(W[tile expert]); w: [E, N, K] (w_mn = false) or [E, K, N] (w_mn = true)
// `out` (optional): a contiguous [rows, N] bf16 buffer to write into (for instance a view of symmetric memory).
Tensor grouped_rows(const Tensor& a, const Tensor& w, const Tensor& tile_expert, bool w_mn, const c10::optional<Tensor>& status,
                    const c10::optional<Tensor>& out_buffer) {
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16 && a.is_contiguous() && w.is_contiguous(), "bf16 contiguous");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && a.size(0) % 128 == 0, "a: [128 * tiles, K], w: 3-D");
  const int64_t K = a.size(1);
  const int64_t N = w_mn ? w.size(2) : w.size(1);
  TORCH_CHECK((w_mn ? w.size(1) : w.size(2)) == K, "contraction size mismatch");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "sizes must be multiples of 8");
  const int64_t tiles = a.size(0) / 128;
  TORCH_CHECK(tile_expert.scalar_type() == torch::kInt32 && tile_expert.numel() >= tiles, "tile_expert: int32, one per tile");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out;
  if (out_buffer.has_value()) {
    out = *out_buffer;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.dim() == 2 && out.size(0) == a.size(0) && out.size(1) == N,
                "out: contiguous bf16 [rows, N]");
  } else {
    out = torch::empty({a.size(0), N}, a.options());
  }
  grouped_rows_gemm(a.data_ptr(), K, w.data_ptr(), out.data_ptr(), N, tile_expert.data_ptr<int>(), (int)tiles, (int)w.size(0),
                    (int)N, (int)K, w_mn, status_of(status), cur_stream());
  return out;
}

// Dispatch fused into the grouped GEMM: the rows named by `src_entry` are pulled from the per-rank token buffers by gather CTAs
// of the GEMM kernel itself, tile by tile, while the other CTAs multiply the tiles that have arrived.
// -> (gathered rows [rows, K], out [rows, N]); `out` may be given (for instance a view of symmetric memory).
std::vector<Tensor> grouped_rows_dispatch(const std::vector<int64_t>& src_ptrs, const Tensor& src_entry, int64_t entries_per_rank, int64_t k,
                                          const Tensor& w, const Tensor& tile_expert, bool w_mn, const c10::optional<Tensor>& status,
                                          int64_t copy_ctas, const c10::optional<Tensor>& out_buffer) {
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.dim() == 3, "w: contiguous bf16 [E, ., .]");
  TORCH_CHECK(src_entry.is_cuda() && src_entry.scalar_type() == torch::kInt32 && src_entry.is_contiguous() && src_entry.numel() % 128 == 0, "src_entry: int32, one per row, 128-row tiles");
  TORCH_CHECK(src_ptrs.size() >= 1 && src_ptrs.size() <= MAX_RANKS, "between 1 and 16 source buffers");
  const int64_t rows = src_entry.numel();
  const int64_t K = w_mn ? w.size(1) : w.size(2);
  const int64_t N = w_mn ? w.size(2) : w.size(1);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0 && K * 2 <= 16384, "sizes must be multiples of 8, rows at most 16 KB");
  const int64_t tiles = rows / 128;
  TORCH_CHECK(tile_expert.scalar_type() == torch::kInt32 && tile_expert.numel() >= tiles, "tile_expert: int32, one per tile");
  const c10::cuda::CUDAGuard guard(w.device());
  Tensor a_rows = torch::empty({rows, K}, w.options());
  Tensor out;
  if (out_buffer.has_value()) {
    out = *out_buffer;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.dim() == 2 && out.size(0) == rows && out.size(1) == N,
                "out: contiguous bf16 [rows, N]");
  } else {
    out = torch::empty({rows, N}, w.options());
  }
  Tensor ready = torch::zeros({tiles}, src_entry.options());
  const void* ptrs[MAX_RANKS];
  for (size_t i = 0; i < src_ptrs.size(); ++i) ptrs[i] = reinterpret_cast<const void*>(src_ptrs[i]);
  grouped_rows_dispatch_gemm(ptrs, (int)src_ptrs.size(), src_entry.data_ptr<int>(), (int)entries_per_rank, (int)k, a_rows.data_ptr(),
                             ready.data_ptr<int>(), (int)copy_ctas, w.data_ptr(), out.data_ptr(), N, tile_expert.data_ptr<int>(), (int)tiles,
                             (int)w.size(0), (int)N, (int)K, w_mn, status_of(status), cur_stream());
  return {a_rows, out};
}

// dw[E, Nw, Kw] (+)= dy[rows, Nw]^T x[rows, Kw] per expert row range
void grouped_wgrad(const Tensor& dy, const Tensor& x, Tensor& dw, const Tensor& padded_offsets, bool accumulate,
                   const c10::optional<Tensor>& status) {
  TORCH_CHECK(dy.scalar_type() == torch::kBFloat16 && x.scalar_type() == torch::kBFloat16 && dy.is_contiguous() && x.is_contiguous(), "bf16 contiguous");
  TORCH_CHECK(dw.scalar_type() == torch::kFloat32 && dw.is_contiguous() && dw.dim() == 3, "dw: fp32 [E, Nw, Kw]");
  TORCH_CHECK(dy.size(0) == x.size(0) && dw.size(1) == dy.size(1) && dw.size(2) == x.size(1), "shape mismatch");
  TORCH_CHECK(padded_offsets.scalar_type() == torch::kInt32 && padded_offsets.numel() == dw.size(0) + 1, "padded_offsets: int32 [E + 1]");
  const c10::cuda::CUDAGuard guard(dy.device());
  grouped_wgrad_gemm(dy.data_ptr(), x.data_ptr(), dw.data_ptr<float>(), padded_offsets.data_ptr<int>(), dy.size(0),
                     (int)dw.size(0), (int)dw.size(1), (int)dw.size(2), accumulate, status_of(status), cur_stream());
}

}  // namespace

void register_moe(pybind11::module_& m) {
  m.def("moe_gather", &moe_gather, pybind11::arg("src_ptrs"), pybind11::arg("scale_ptrs"), pybind11::arg("src_entry"), pybind11::arg("H"),
        pybind11::arg("entries_per_rank"), pybind11::arg("k"), pybind11::arg("like"), pybind11::arg("tile_owner") = pybind11::none(),
        pybind11::arg("owners") = 0);
  m.def("moe_combine", &moe_combine);
  m.def("moe_rowdot", &moe_rowdot);
  m.def("scale_rows_", &scale_rows_, pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("tile_owner") = pybind11::none(), pybind11::arg("owners") = 0);
  m.def("moe_swiglu_bwd", &moe_swiglu_bwd, pybind11::arg("fc"), pybind11::arg("dact"), pybind11::arg("row_weight"),
        pybind11::arg("tile_owner") = pybind11::none(), pybind11::arg("owners") = 0);
  m.def("grouped_rows", &grouped_rows, pybind11::arg("a"), pybind11::arg("w"), pybind11::arg("tile_expert"), pybind11::arg("w_mn"),
        pybind11::arg("status"), pybind11::arg("out") = pybind11::none());
  m.def("grouped_rows_dispatch", &grouped_rows_dispatch, pybind11::arg("src_ptrs"), pybind11::arg("src_entry"), pybind11::arg("entries_per_rank"),
        pybind11::arg("k"), pybind11::arg("w"), pybind11::arg("tile_expert"), pybind11::arg("w_mn"), pybind11::arg("status"),
        pybind11::arg("copy_ctas") = 16, pybind11::arg("out") = pybind11::none());
  m.def("grouped_wgrad", &grouped_wgrad);
}

}  // namespace b200

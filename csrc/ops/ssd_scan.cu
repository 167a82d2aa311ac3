// Selective state-space (Mamba-2 SSD) recurrence as a state-resident scan (sm_100a).
//
//   h_t = exp(a_t) * h_{t-1} + x_t b_t^T        (h: [P, N] per head),        y_t = h_t c_t
//
// One generic kernel runs the recurrence  s_t = decay * s_prev + u_t v_t^T,  o_t[q] = sum_r s_t[q, r] w_t[r]  forwards or
// backwards in time with the [Q, R] state held in registers for the whole sequence (one CTA per (batch, head), every
// thread owns a 4 x RS register tile of it; the lanes that share rows finish the output with shuffles).
// Forward and backward of the layer are four instances of it:
//   y  : forwards,  (q, r) = (p, n), u = x,  v = b,  w = c
//   dc : forwards,  (q, r) = (n, p), u = b,  v = x,  w = dy      (the transposed state times dy)
//   dx : backwards, (q, r) = (p, n), u = dy, v = c,  w = b       (the adjoint state dh_t = dy_t c_t^T + exp(a_{t+1}) dh_{t+1})
//   db : backwards, (q, r) = (n, p), u = c,  v = dy, w = x
// and the gradient of a needs no state at all: da_t = <dy_t, y_t> - <x_t, dx_t> + da_{t+1} (a reversed cumulative sum
// done by the caller). No chunking, no checkpoints: the state never leaves the SM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "../common/launch.h"

namespace py = pybind11;
using torch::Tensor;

namespace b200 {
namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

struct Operand {
  const float* ptr;  // [B, L, heads, dim]
  int heads;         // H, or the number of groups when the operand is shared by the heads of a group
  int dim;
};

__device__ __forceinline__ const float* row_of(const Operand& op, int b, int t, int h, int H, int L) {
  const int hh = op.heads == H ? h : h / (H / op.heads);
  return op.ptr + (((size_t)b * L + t) * op.heads + hh) * op.dim;
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int TC = 16;  // time steps staged in shared memory per chunk (two chunks in flight)

constexpr int QS = 4;  // state rows per thread

// Thread (g, k) owns a QS x RS register tile of the state: rows g * QS .. + QS, and the RS columns
// {(i * NT + k) * 4 + j : i < RS / 4, j < 4} with NT = R / RS lanes per row group, so that the NT lanes of a row group read
// consecutive 16-byte pieces of v_t and w_t from shared memory (no bank conflicts) and every v / w value a thread loads
// serves QS rows. Threads = (Q / QS) * NT. The operands of TC consecutive time steps are copied to shared memory with
// cp.async while the previous chunk is consumed, so the sequential loop never waits on global memory.
template <int RS, bool REVERSE>
__global__ void ssd_scan_kernel(Operand u, Operand v, Operand w, const float* __restrict__ a, float* __restrict__ out,
                                const float* __restrict__ s0, float* __restrict__ s_last, int L, int H, int Q, int R) {
  extern __shared__ __align__(16) float stage[];  // [2][TC * (Q + 2 R) + TC]
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int NT = R / RS;
  const int g = threadIdx.x / NT, k = threadIdx.x - g * NT;
  const int per_step = Q + 2 * R;
  const int chunk_floats = TC * per_step + TC;
  float s[QS][RS];
  const size_t state_base = (((size_t)b * H + h) * Q + (size_t)g * QS) * R;
#pragma unroll
  for (int jq = 0; jq < QS; ++jq)
#pragma unroll
    for (int i = 0; i < RS / 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[jq][4 * i + j] = s0 != nullptr ? s0[state_base + (size_t)jq * R + (i * NT + k) * 4 + j] : 0.f;

  const int chunks = (L + TC - 1) / TC;
  // copy the operands of chunk `ci` (steps ci * TC ... in processing order) into buffer `buf`
  auto issue = [&](int ci, int buf) {
    float* base = stage + (size_t)buf * chunk_floats;
    const int vec_per_step = per_step / 4;
    for (int idx = threadIdx.x; idx < TC * vec_per_step; idx += blockDim.x) {
      const int j = idx / vec_per_step, e = (idx - j * vec_per_step) * 4;
      const int step = ci * TC + j;
      if (step >= L) continue;
      const int t = REVERSE ? L - 1 - step : step;
      const float* src = e < Q ? row_of(u, b, t, h, H, L) + e : (e < Q + R ? row_of(v, b, t, h, H, L) + (e - Q) : row_of(w, b, t, h, H, L) + (e - Q - R));
      cp_async_16(base + j * per_step + e, src);
    }
    for (int j = threadIdx.x; j < TC; j += blockDim.x) {
      const int step = ci * TC + j;
      if (step < L) cp_async_4(base + TC * per_step + j, a + ((size_t)b * L + (REVERSE ? L - 1 - step : step)) * H + h);
    }
    cp_async_commit();
  };

  float carry_decay = 1.f;  // REVERSE: exp(a_{t+1}), applied to the state before step t adds its term
  issue(0, 0);
  for (int ci = 0; ci < chunks; ++ci) {
    if (ci + 1 < chunks) {
      issue(ci + 1, (ci + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* base = stage + (size_t)(ci & 1) * chunk_floats;
    const int steps = min(TC, L - ci * TC);
    for (int j = 0; j < steps; ++j) {
      const int step = ci * TC + j;
      const int t = REVERSE ? L - 1 - step : step;
      const float decay_t = __expf(base[TC * per_step + j]);
      const float decay = REVERSE ? carry_decay : decay_t;
      carry_decay = decay_t;
      const float* row = base + j * per_step;
      const float4 u4 = *reinterpret_cast<const float4*>(row + g * QS);
      const float uq[QS] = {u4.x, u4.y, u4.z, u4.w};
      const float4* v4 = reinterpret_cast<const float4*>(row + Q) + k;
      const float4* w4 = reinterpret_cast<const float4*>(row + Q + R) + k;
      float acc[QS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < RS / 4; ++i) {
        const float4 vv = v4[i * NT], ww = w4[i * NT];
#pragma unroll
        for (int jq = 0; jq < QS; ++jq) {
          float* sr = &s[jq][4 * i];
          sr[0] = fmaf(decay, sr[0], uq[jq] * vv.x);
          sr[1] = fmaf(decay, sr[1], uq[jq] * vv.y);
          sr[2] = fmaf(decay, sr[2], uq[jq] * vv.z);
          sr[3] = fmaf(decay, sr[3], uq[jq] * vv.w);
          acc[jq] = fmaf(sr[0], ww.x, fmaf(sr[1], ww.y, fmaf(sr[2], ww.z, fmaf(sr[3], ww.w, acc[jq]))));
        }
      }
      for (int off = NT >> 1; off > 0; off >>= 1) {
#pragma unroll
        for (int jq = 0; jq < QS; ++jq) acc[jq] += __shfl_xor_sync(0xffffffffu, acc[jq], off);
      }
      if (k == 0) *reinterpret_cast<float4*>(out + (((size_t)b * L + t) * H + h) * Q + g * QS) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
    __syncthreads();  // the buffer is refilled two chunks later
  }
  if (s_last != nullptr) {
#pragma unroll
    for (int jq = 0; jq < QS; ++jq)
#pragma unroll
      for (int i = 0; i < RS / 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s_last[state_base + (size_t)jq * R + (i * NT + k) * 4 + j] = s[jq][4 * i + j];
  }
}

Operand operand_of(const Tensor& t, int64_t B, int64_t L, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous() && t.dim() == 4 && t.size(0) == B && t.size(1) == L,
              name, ": contiguous fp32 [B, L, heads, dim]");
  return Operand{t.data_ptr<float>(), (int)t.size(2), (int)t.size(3)};
}

// out[b, t, h, q] of the recurrence above. u: [B, L, Hu, Q]; v, w: [B, L, Hv, R]; a: [B, L, H]; s0: [B, H, Q, R] or none.
// Returns (out [B, L, H, Q], last state [B, H, Q, R]).
std::vector<Tensor> ssd_scan(const Tensor& u, const Tensor& v, const Tensor& w, const Tensor& a, const c10::optional<Tensor>& s0, bool reverse) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kFloat32 && a.is_contiguous() && a.dim() == 3, "a: contiguous fp32 [B, L, H]");
  const int64_t B = a.size(0), L = a.size(1), H = a.size(2);
  const Operand ou = operand_of(u, B, L, "u"), ov = operand_of(v, B, L, "v"), ow = operand_of(w, B, L, "w");
  const int Q = ou.dim, R = ov.dim;
  TORCH_CHECK(ow.dim == R, "v and w must have the same width");
  for (const Operand& op : {ou, ov, ow}) TORCH_CHECK(op.heads >= 1 && H % op.heads == 0, "operand heads must divide the number of heads");
  // columns per thread: as many as keep the CTA between 128 and 512 threads with a power-of-two number of lanes per row group
  TORCH_CHECK(Q % QS == 0 && R % 4 == 0, "state shape must be a multiple of 4 in both directions");
  int rs = 0;
  for (int cand : {8, 16, 4, 32}) {
    if (R % cand != 0) continue;
    const int nt = R / cand;
    if ((nt & (nt - 1)) != 0 || nt > 32) continue;
    const int threads = (Q / QS) * nt;
    if (threads > 1024 || (threads % 32 != 0 && threads > 32) || (threads < 32 && 32 % threads != 0)) continue;
    if (threads < 32) continue;
    rs = cand;
    if (threads >= 128 && threads <= 512) break;
  }
  TORCH_CHECK(rs != 0, "unsupported state shape ", Q, " x ", R);
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out = torch::empty({B, L, H, (int64_t)Q}, a.options());
  Tensor last = torch::empty({B, H, (int64_t)Q, (int64_t)R}, a.options());
  const float* s0p = nullptr;
  if (s0.has_value()) {
    TORCH_CHECK(s0->scalar_type() == torch::kFloat32 && s0->is_contiguous() && s0->numel() == B * H * Q * R, "s0: contiguous fp32 [B, H, Q, R]");
    s0p = s0->data_ptr<float>();
  }
  if (B * H == 0) return {out, last};
  const int threads = (Q / QS) * (R / rs);
  const dim3 grid((unsigned)(B * H));
  const size_t smem = (size_t)2 * (TC * (Q + 2 * R) + TC) * sizeof(float);
  TORCH_CHECK(Q % 4 == 0 && smem <= 200 * 1024, "state rows must be a multiple of 4 and fit the staging buffer");
#define B200_SSD_LAUNCH(RS_)                                                                                                              \
  do {                                                                                                                                    \
    if (smem > 48 * 1024) {                                                                                                               \
      check_cuda(cudaFuncSetAttribute(ssd_scan_kernel<RS_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "ssd smem");   \
      check_cuda(cudaFuncSetAttribute(ssd_scan_kernel<RS_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "ssd smem");  \
    }                                                                                                                                     \
    if (reverse)                                                                                                                          \
      ssd_scan_kernel<RS_, true><<<grid, threads, smem, cur_stream()>>>(ou, ov, ow, a.data_ptr<float>(), out.data_ptr<float>(), s0p,        \
                                                                     last.data_ptr<float>(), (int)L, (int)H, Q, R);                       \
    else                                                                                                                                  \
      ssd_scan_kernel<RS_, false><<<grid, threads, smem, cur_stream()>>>(ou, ov, ow, a.data_ptr<float>(), out.data_ptr<float>(), s0p,       \
                                                                      last.data_ptr<float>(), (int)L, (int)H, Q, R);                      \
  } while (0)
  switch (rs) {
    case 4: B200_SSD_LAUNCH(4); break;
    case 8: B200_SSD_LAUNCH(8); break;
    case 16: B200_SSD_LAUNCH(16); break;
    default: B200_SSD_LAUNCH(32); break;
  }
#undef B200_SSD_LAUNCH
  count_launch();
  check_cuda(cudaGetLastError(), "ssd_scan launch");
  return {out, last};
}

}  // namespace

void register_ssd(py::module_& m) { m.def("ssd_scan", &ssd_scan); }

}  // namespace b200

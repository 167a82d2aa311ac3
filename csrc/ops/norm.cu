// RMSNorm forward/backward for bf16 activations (fp32 math), with the residual
// add fused on both sides:
//   forward : h = x (+ residual) ; y = h * rsqrt(mean(h^2) + eps) * w
//   backward: dh = d(norm path) (+ incoming residual-stream gradient) ; dw partials per CTA
// Memory bound: one pass over each operand with 16-byte accesses; rows stay in registers.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "ops.h"

namespace b200 {

namespace {


template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}

template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
    rmsnorm_fwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res, const uint4* __restrict__ w,
                       uint4* __restrict__ y, uint4* __restrict__ h_out, float* __restrict__ rstd, int T, int H,
                       float eps) {
  __shared__ float red[THREADS / 32];
  const int nv = H >> 3;
  const int row = blockIdx.x;
  if (row >= T) return;
  const uint4* xr = x + (size_t)row * nv;
  const uint4* rr = res ? res + (size_t)row * nv : nullptr;
  uint4 hv[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nv) {
      uint4 a = xr[i];
      if (rr) {
        const uint4 b = rr[i];
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
        const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
        a.x = pack_bf16x2(a0.x + b0.x, a0.y + b0.y);
        a.y = pack_bf16x2(a1.x + b1.x, a1.y + b1.y);
        a.z = pack_bf16x2(a2.x + b2.x, a2.y + b2.y);
        a.w = pack_bf16x2(a3.x + b3.x, a3.y + b3.y);
        if (h_out) h_out[(size_t)row * nv + i] = a;
      }
      hv[j] = a;
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
    }
  }
  ss = block_sum<THREADS>(ss, red);
  const float r = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nv) {
      const uint4 a = hv[j];
      const uint4 g = w[i];
      const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
      const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
      uint4 o;
      o.x = pack_bf16x2(f0.x * r * g0.x, f0.y * r * g0.y);
      o.y = pack_bf16x2(f1.x * r * g1.x, f1.y * r * g1.y);
      o.z = pack_bf16x2(f2.x * r * g2.x, f2.y * r * g2.y);
      o.w = pack_bf16x2(f3.x * r * g3.x, f3.y * r * g3.y);
      y[(size_t)row * nv + i] = o;
    }
  }
}

// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its share of
// dw in registers; partial[blockIdx.x, :] receives it at the end.
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
    rmsnorm_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ h, const uint4* __restrict__ w,
                       const float* __restrict__ rstd, const uint4* __restrict__ dres, uint4* __restrict__ dh,
                       float* __restrict__ partial, int T, int H) {
  __shared__ float red[THREADS / 32];
  const int nv = H >> 3;
  float dw[MAXV][8];
  float wf[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) dw[j][e] = 0.f;
    if (i < nv) {
      const uint4 g = w[i];
      const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
      wf[j][0] = g0.x; wf[j][1] = g0.y; wf[j][2] = g1.x; wf[j][3] = g1.y;
      wf[j][4] = g2.x; wf[j][5] = g2.y; wf[j][6] = g3.x; wf[j][7] = g3.y;
    }
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float r = rstd[row];
    float xh[MAXV][8], wd[MAXV][8];
    float c = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nv) {
        const uint4 a = h[(size_t)row * nv + i];
        const uint4 d = dy[(size_t)row * nv + i];
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
        const float2 d0 = unpack_bf16x2(d.x), d1 = unpack_bf16x2(d.y), d2 = unpack_bf16x2(d.z), d3 = unpack_bf16x2(d.w);
        const float av[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
        const float dv[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = av[e] * r;
          wd[j][e] = dv[e] * wf[j][e];
          dw[j][e] += dv[e] * xh[j][e];
          c += xh[j][e] * wd[j][e];
        }
      }
    }
    c = block_sum<THREADS>(c, red) / (float)H;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nv) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (wd[j][e] - xh[j][e] * c) * r;
        if (dres) {
          const uint4 q = dres[(size_t)row * nv + i];
          const float2 q0 = unpack_bf16x2(q.x), q1 = unpack_bf16x2(q.y), q2 = unpack_bf16x2(q.z), q3 = unpack_bf16x2(q.w);
          o[0] += q0.x; o[1] += q0.y; o[2] += q1.x; o[3] += q1.y;
          o[4] += q2.x; o[5] += q2.y; o[6] += q3.x; o[7] += q3.y;
        }
        uint4 ov;
        ov.x = pack_bf16x2(o[0], o[1]);
        ov.y = pack_bf16x2(o[2], o[3]);
        ov.z = pack_bf16x2(o[4], o[5]);
        ov.w = pack_bf16x2(o[6], o[7]);
        dh[(size_t)row * nv + i] = ov;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nv) {
      float4* p = reinterpret_cast<float4*>(partial + (size_t)blockIdx.x * H + (size_t)i * 8);
      p[0] = make_float4(dw[j][0], dw[j][1], dw[j][2], dw[j][3]);
      p[1] = make_float4(dw[j][4], dw[j][5], dw[j][6], dw[j][7]);
    }
  }
}

// out[c] (+)= sum_r partial[r, c]. Block = 32 columns x 8 row lanes: every row lane sums its rows with coalesced
// 128-byte reads, shared memory folds the eight partial sums.
__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int cols,
                                                         int accumulate) {
  __shared__ float fold[8][33];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + x;
  float s = 0.f;
  if (c < cols) {
    for (int r = y; r < rows; r += 8) s += partial[(size_t)r * cols + c];
  }
  fold[y][x] = s;
  __syncthreads();
  if (y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += fold[k][x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

}  // namespace

int rmsnorm_bwd_partial_rows(int T) {
  const int cap = sm_count() * 4;
  return T < cap ? T : cap;
}

void rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd, int T, int H,
                 float eps, cudaStream_t stream) {
  if (T == 0) return;
  if (H % 8 != 0 || H > 32768) throw std::runtime_error("rmsnorm: H must be a multiple of 8 and <= 32768");
  auto X = reinterpret_cast<const uint4*>(x);
  auto R = reinterpret_cast<const uint4*>(residual);
  auto W = reinterpret_cast<const uint4*>(w);
  auto Y = reinterpret_cast<uint4*>(y);
  auto HO = reinterpret_cast<uint4*>(h_out);
  const int nv = H / 8;
#define FWD(TH, V) rmsnorm_fwd_kernel<TH, V><<<T, TH, 0, stream>>>(X, R, W, Y, HO, rstd, T, H, eps)
  if (nv <= 256) FWD(256, 1);
  else if (nv <= 512) FWD(256, 2);
  else if (nv <= 1024) FWD(256, 4);
  else if (nv <= 2048) FWD(512, 4);
  else FWD(1024, 4);
#undef FWD
  count_launch();
  check_cuda(cudaGetLastError(), "rmsnorm_fwd launch");
}

// `partial` is scratch of rmsnorm_bwd_partial_rows(T) * H floats. dw (fp32, [H]) is
// overwritten or accumulated into.
void rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dh,
                 float* partial, float* dw, bool accumulate_dw, int T, int H, cudaStream_t stream) {
  if (T == 0) return;
  if (H % 8 != 0 || H > 32768) throw std::runtime_error("rmsnorm: H must be a multiple of 8 and <= 32768");
  int rows = rmsnorm_bwd_partial_rows(T);
  auto DY = reinterpret_cast<const uint4*>(dy);
  auto HH = reinterpret_cast<const uint4*>(h);
  auto W = reinterpret_cast<const uint4*>(w);
  auto DR = reinterpret_cast<const uint4*>(dres);
  auto DH = reinterpret_cast<uint4*>(dh);
  const int nv = H / 8;
  // one wave of CTAs: as many as are resident at a time (a partly filled second wave would double the kernel's time)
#define BWD(TH, V)                                                                                                        \
  do {                                                                                                                    \
    static int resident = 0;                                                                                              \
    if (resident == 0) {                                                                                                  \
      int per_sm = 0;                                                                                                     \
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_bwd_kernel<TH, V>, TH, 0);                            \
      resident = sm_count() * (per_sm > 0 ? per_sm : 1);                                                                  \
    }                                                                                                                     \
    if (rows > resident) rows = resident;                                                                                 \
    rmsnorm_bwd_kernel<TH, V><<<rows, TH, 0, stream>>>(DY, HH, W, rstd, DR, DH, partial, T, H);                            \
  } while (0)
  if (nv <= 256) BWD(256, 1);
  else if (nv <= 512) BWD(256, 2);
  else if (nv <= 1024) BWD(256, 4);
  else if (nv <= 2048) BWD(512, 4);
  else BWD(1024, 4);
#undef BWD
  column_sum_kernel<<<(H + 31) / 32, 256, 0, stream>>>(partial, dw, rows, H, accumulate_dw ? 1 : 0);
  count_launch(2);
  check_cuda(cudaGetLastError(), "rmsnorm_bwd launch");
}

}  // namespace b200

// ----------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the RMSNorm backward (declared in noalloc.h).
//
// The regular entry point takes its per-CTA partial-sum scratch from the caller (the Python binding allocates it
// from the tensor allocator on every call). Callers that must not allocate device memory - a C host loop that has
// handed all device memory to its own arena, code running where a device allocation would synchronise or fail -
// use this one instead: the scratch is a fixed array that lives in the library image.
// ----------------------------------------------------------------------------------------------------------------
#include <mutex>

#include "noalloc.h"

namespace b200 {
namespace {

// kNoAllocMaxRows x kNoAllocMaxH floats = 5 MiB, resident on every GPU that loads this library until process exit.
static __device__ __align__(256) float g_noalloc_rmsnorm_partial[B200_NOALLOC_RMSNORM_MAX_ROWS * B200_NOALLOC_RMSNORM_MAX_H];

constexpr int kMaxDevices = 64;
float* g_noalloc_partial_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

void copy_message(char* dst, int len, const char* msg) {
  if (dst == nullptr || len <= 0) return;
  int i = 0;
  for (; i < len - 1 && msg[i] != '\0'; ++i) dst[i] = msg[i];
  dst[i] = '\0';
}

template <int TH, int V>
void launch_noalloc_bwd(int rows, const uint4* DY, const uint4* HH, const uint4* W, const float* rstd, const uint4* DR,
                        uint4* DH, float* partial, int T, int H, cudaStream_t stream) {
  rmsnorm_bwd_kernel<TH, V><<<rows, TH, 0, stream>>>(DY, HH, W, rstd, DR, DH, partial, T, H);
}

}  // namespace
}  // namespace b200

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                                        void* dh, float* dw, int accumulate_dw, int T, int H, void* stream,
                                        char* error_message, int error_message_len) {
  using namespace b200;
  if (T < 0 || H <= 0 || H % 8 != 0) {
    copy_message(error_message, error_message_len, "b200_rmsnorm_bwd_noalloc: T must be >= 0 and H a positive multiple of 8");
    return 1;
  }
  if (H > B200_NOALLOC_RMSNORM_MAX_H) {
    copy_message(error_message, error_message_len,
                 "b200_rmsnorm_bwd_noalloc: H exceeds B200_NOALLOC_RMSNORM_MAX_H (8192); use the allocating entry point");
    return 2;
  }
  if (T == 0) return 0;
  {
    // The kernels read and write 16 bytes at a time: a missing or misaligned pointer would otherwise surface as a
    // device-side fault instead of an error code.
    const void* required[] = {dy, h, w, rstd, dh, dw};
    for (const void* p : required) {
      if (p == nullptr) {
        copy_message(error_message, error_message_len, "b200_rmsnorm_bwd_noalloc: dy, h, w, rstd, dh and dw must not be NULL");
        return 6;
      }
    }
    const void* vectors[] = {dy, h, w, dres, dh, dw};
    for (const void* p : vectors) {
      if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) {
        copy_message(error_message, error_message_len, "b200_rmsnorm_bwd_noalloc: dy, h, w, dres, dh and dw must be 16-byte aligned");
        return 7;
      }
    }
    if ((reinterpret_cast<uintptr_t>(rstd) & 3u) != 0) {
      copy_message(error_message, error_message_len, "b200_rmsnorm_bwd_noalloc: rstd must be 4-byte aligned");
      return 7;
    }
  }

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    copy_message(error_message, error_message_len, "b200_rmsnorm_bwd_noalloc: cannot identify the current device");
    return 3;
  }
  float* partial = nullptr;
  {
    // First call on a device: resolve the device address of the scratch array with that device current.
    // (In host code the array's name is only a handle; a kernel must be given the resolved address.)
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_partial_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_rmsnorm_partial);
      if (e != cudaSuccess || p == nullptr) {
        copy_message(error_message, error_message_len, cudaGetErrorString(e));
        return 4;
      }
      g_noalloc_partial_ptr[dev] = static_cast<float*>(p);
    }
    partial = g_noalloc_partial_ptr[dev];
  }

  const int rows = T < B200_NOALLOC_RMSNORM_MAX_ROWS ? T : B200_NOALLOC_RMSNORM_MAX_ROWS;
  auto DY = reinterpret_cast<const uint4*>(dy);
  auto HH = reinterpret_cast<const uint4*>(h);
  auto W = reinterpret_cast<const uint4*>(w);
  auto DR = reinterpret_cast<const uint4*>(dres);
  auto DH = reinterpret_cast<uint4*>(dh);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int nv = H / 8;
  // Every partial row that the reduction reads is fully overwritten by its CTA first, so nothing needs clearing.
  if (nv <= 256) launch_noalloc_bwd<256, 1>(rows, DY, HH, W, rstd, DR, DH, partial, T, H, s);
  else if (nv <= 512) launch_noalloc_bwd<256, 2>(rows, DY, HH, W, rstd, DR, DH, partial, T, H, s);
  else launch_noalloc_bwd<256, 4>(rows, DY, HH, W, rstd, DR, DH, partial, T, H, s);
  column_sum_kernel<<<(H + 31) / 32, 256, 0, s>>>(partial, dw, rows, H, accumulate_dw ? 1 : 0);
  count_launch(2);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    copy_message(error_message, error_message_len, cudaGetErrorString(e));
    return 5;
  }
  return 0;
}

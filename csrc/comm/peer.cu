// Collectives of this engine over NVLink peer memory (no NCCL on these paths).
//
// Buffers live in symmetric memory: every rank allocates the same layout and maps every peer's copy, so a kernel
// receives one pointer per rank (plus, when the NVSwitch supports it, one multicast address that stands for all
// copies at once). Two access modes per kernel:
//   * multimem: `multimem.ld_reduce` sums the copies inside the switch, `multimem.st` stores to all copies at once;
//   * plain peer loads/stores with 16-byte accesses, summed in rank order (bit-reproducible).
// No load here is a TMA load, so nothing is multicast across a cluster.
//
// Cross-rank ordering uses flags in a symmetric control block: `peer_barrier` publishes a monotonically increasing
// epoch to every peer with a system-scope release store and waits with acquire loads until every peer has published
// it. The wait is bounded by wall time (%globaltimer); on expiry the kernel records kStatusWaitTimeoutPeer in the
// status word and returns, so a missing rank shows up as an error code on the host and never as a hang.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdexcept>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "peer.h"

namespace b200 {
namespace {

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint4 ld_peer_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_peer_u4(uint4* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float4* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ void multimem_st_u4(uint4* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// One block; thread p talks to rank p. Flags: word [writer] of the control block of rank [reader].
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, uint32_t epoch, unsigned long long timeout_ns, int* status) {
  const int p = threadIdx.x;
  if (p >= flags.n) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<uint32_t*>(flags.p[p]) + rank, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + p;
  const unsigned long long start = global_timer_ns();
  while (true) {
    const uint32_t seen = ld_acquire_sys(mine);
    if (static_cast<int32_t>(seen - epoch) >= 0) break;
    if (global_timer_ns() - start > timeout_ns) {
      atomicCAS(status, kStatusOk, kStatusWaitTimeoutPeer);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

// out[i] = sum over ranks of src[r][offset + i], i in float4 units. `out` may be this rank's own region.
__global__ void reduce_scatter_f32_kernel(PeerPtrs src, const float4* __restrict__ multicast, float4* __restrict__ out,
                                          long long offset_v, long long nv, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float4 acc;
    if (multicast != nullptr) {
      acc = multimem_ld_reduce_f4(multicast + offset_v + i);
    } else {
      acc = ld_peer_f4(reinterpret_cast<const float4*>(src.p[0]) + offset_v + i);
      for (int r = 1; r < src.n; ++r) {
        const float4 v = ld_peer_f4(reinterpret_cast<const float4*>(src.p[r]) + offset_v + i);
        acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
      }
    }
    out[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
  }
}

// Every rank pulls the shards of the others into its own copy: buf[r][shard r] -> buf[self][shard r].
__global__ void all_gather_pull_kernel(PeerPtrs buf, int rank, long long shard_v) {
  uint4* mine = reinterpret_cast<uint4*>(buf.p[rank]);
  const long long total = shard_v * (buf.n - 1);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int r = static_cast<int>(i / shard_v);
    const long long e = i - r * shard_v;
    r = (rank + 1 + r) % buf.n;  // start with the next rank so that the peers are not all hit in the same order
    mine[r * shard_v + e] = ld_peer_u4(reinterpret_cast<const uint4*>(buf.p[r]) + r * shard_v + e);
  }
}

// AdamW on this rank's fp32 shard whose bf16 result goes to the same place of every rank's compute copy: the
// parameter all-gather is the store of the optimizer. Eight elements per thread so that peer stores are 16 bytes.
__global__ void adamw_bcast_kernel(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v, float4* __restrict__ g,
                                   PeerPtrs dst, uint4* __restrict__ multicast, long long dst_offset_v8, long long n8, float lr,
                                   float b1, float b2, float eps, float wd, float bc1, float bc2_sqrt,
                                   const float* __restrict__ grad_scale, float grad_mul, int zero_grad) {
  const float gs = (grad_scale ? grad_scale[0] : 1.f) * grad_mul;
  const float step = lr / bc1;
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint32_t packed[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long j = 2 * i + h;
      const float4 P = p[j], M = m[j], V = v[j], G = g[j];
      float pp[4] = {P.x, P.y, P.z, P.w}, mm[4] = {M.x, M.y, M.z, M.w}, vv[4] = {V.x, V.y, V.z, V.w};
      const float gg[4] = {G.x * gs, G.y * gs, G.z * gs, G.w * gs};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pp[e] *= decay;
        mm[e] = b1 * mm[e] + (1.f - b1) * gg[e];
        vv[e] = b2 * vv[e] + (1.f - b2) * gg[e] * gg[e];
        const float denom = sqrtf(vv[e]) / bc2_sqrt + eps;
        pp[e] -= step * mm[e] / denom;
      }
      p[j] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      m[j] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      v[j] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (zero_grad) g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      packed[2 * h] = pack_bf16x2(pp[0], pp[1]);
      packed[2 * h + 1] = pack_bf16x2(pp[2], pp[3]);
    }
    const uint4 out = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    if (multicast != nullptr) {
      multimem_st_u4(multicast + dst_offset_v8 + i, out);
    } else {
      for (int r = 0; r < dst.n; ++r) st_peer_u4(reinterpret_cast<uint4*>(dst.p[r]) + dst_offset_v8 + i, out);
    }
  }
}

inline int comm_grid(long long work_items, int threads) {
  const long long want = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

void peer_barrier(const PeerPtrs& flags, int rank, uint32_t epoch, double timeout_seconds, int* status, cudaStream_t stream) {
  if (flags.n < 1 || flags.n > kMaxPeers || rank < 0 || rank >= flags.n) throw std::runtime_error("peer_barrier: bad rank table");
  const unsigned long long timeout_ns = (unsigned long long)(timeout_seconds * 1e9);
  peer_barrier_kernel<<<1, 32, 0, stream>>>(flags, rank, epoch, timeout_ns, status);
  count_launch();
  check_cuda(cudaGetLastError(), "peer_barrier launch");
}

void peer_reduce_scatter_f32(const PeerPtrs& src, const void* multicast, float* out, long long elem_offset, long long n, float scale,
                             cudaStream_t stream) {
  if (n == 0) return;
  if (n % 4 || elem_offset % 4) throw std::runtime_error("peer_reduce_scatter: offset and length must be multiples of 4 floats");
  reduce_scatter_f32_kernel<<<comm_grid(n / 4, 256), 256, 0, stream>>>(src, reinterpret_cast<const float4*>(multicast),
                                                                     reinterpret_cast<float4*>(out), elem_offset / 4, n / 4, scale);
  count_launch();
  check_cuda(cudaGetLastError(), "peer_reduce_scatter launch");
}

void peer_all_gather(const PeerPtrs& buf, int rank, long long shard_bytes, cudaStream_t stream) {
  if (buf.n <= 1 || shard_bytes == 0) return;
  if (shard_bytes % 16) throw std::runtime_error("peer_all_gather: shard size must be a multiple of 16 bytes");
  const long long shard_v = shard_bytes / 16;
  all_gather_pull_kernel<<<comm_grid(shard_v * (buf.n - 1), 256), 256, 0, stream>>>(buf, rank, shard_v);
  count_launch();
  check_cuda(cudaGetLastError(), "peer_all_gather launch");
}

void adamw_step_bcast(float* p, float* m, float* v, float* g, const PeerPtrs& dst, void* multicast, long long dst_elem_offset,
                      long long n, float lr, float beta1, float beta2, float eps, float weight_decay, float bias_c1, float bias_c2,
                      const float* grad_scale, float grad_mul, bool zero_grad, cudaStream_t stream) {
  if (n == 0) return;
  if (n % 8 || dst_elem_offset % 8) throw std::runtime_error("adamw_step_bcast: offset and length must be multiples of 8");
  adamw_bcast_kernel<<<comm_grid(n / 8, 256), 256, 0, stream>>>(
      reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v), reinterpret_cast<float4*>(g), dst,
      reinterpret_cast<uint4*>(multicast), dst_elem_offset / 8, n / 8, lr, beta1, beta2, eps, weight_decay, bias_c1,
      sqrtf(bias_c2), grad_scale, grad_mul, zero_grad ? 1 : 0);
  count_launch();
  check_cuda(cudaGetLastError(), "adamw_step_bcast launch");
}

}  // namespace b200

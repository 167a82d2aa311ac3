// Host entry points of the peer-memory collectives (see peer.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMaxPeers = 16;

// One device pointer per rank of the group (the local rank included), passed to kernels by value.
struct PeerPtrs {
  void* p[kMaxPeers];
  int n;
};

void peer_barrier(const PeerPtrs& flags, int rank, uint32_t epoch, double timeout_seconds, int* status, cudaStream_t stream);
void peer_reduce_scatter_f32(const PeerPtrs& src, const void* multicast, float* out, long long elem_offset, long long n, float scale,
                             cudaStream_t stream);
void peer_all_gather(const PeerPtrs& buf, int rank, long long shard_bytes, cudaStream_t stream);
void adamw_step_bcast(float* p, float* m, float* v, float* g, const PeerPtrs& dst, void* multicast, long long dst_elem_offset,
                      long long n, float lr, float beta1, float beta2, float eps, float weight_decay, float bias_c1, float bias_c2,
                      const float* grad_scale, float grad_mul, bool zero_grad, cudaStream_t stream);

// Fused tensor-parallel GEMMs (tp_gemm.cu).
void ag_gemm_bf16(const PeerPtrs& x_ptrs, void* staging, int* ready, int epoch, const void* W, void* Y, int M, int N, int K, long long ldw,
                  long long ldc, bool w_mn, int rank, int copy_ctas, int* status, cudaStream_t stream);
void gemm_rs_bf16(const void* X, const void* W, const PeerPtrs& out_ptrs, int M, int N, int K, long long ldx, long long ldw, long long ldc,
                  bool w_mn, int rank, int* status, cudaStream_t stream);

void sum_slots_bf16(const void* slots, void* out, long long n, int world, cudaStream_t stream);

}  // namespace b200

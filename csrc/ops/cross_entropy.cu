// Row-wise softmax cross-entropy over bf16 logits with the gradient written in
// place of the logits, used by the chunked fused linear + cross-entropy path:
//   z = logit_scale * logits ; loss = logsumexp(z) - z[label]
//   dlogits = grad_scale * logit_scale * (softmax(z) - onehot(label))   (zero for ignored rows)
// One CTA per row: pass 1 keeps a running (max, sum) per thread, pass 2 re-reads the
// row (still resident in L2) and overwrites it.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "ops.h"

namespace b200 {

namespace {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_update(float& m, float& s, float x) {
  if (x > m) {
    s = s * __expf(m - x) + 1.f;
    m = x;
  } else {
    s += __expf(x - m);
  }
}

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) return;
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

__global__ void __launch_bounds__(CE_THREADS)
    ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ loss,
              float* __restrict__ lse_out, int V, long long row_stride, float logit_scale, float grad_scale,
              long long ignore_index, int write_grad) {
  __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
  __shared__ float sh_lse;
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (long long)row * row_stride;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const bool vec_ok = (row_stride % 8 == 0) && (reinterpret_cast<uintptr_t>(logits) % 16 == 0);
  const int nv = vec_ok ? V / 8 : 0;
  uint4* l4 = reinterpret_cast<uint4*>(lr);

  float m = -INFINITY, s = 0.f;
  if (!ignored || lse_out) {
    for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
      const uint4 v = l4[i];
      const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(vv[e]);
        online_update(m, s, f.x * logit_scale);
        online_update(m, s, f.y * logit_scale);
      }
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += CE_THREADS) online_update(m, s, __bfloat162float(lr[i]) * logit_scale);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) {
      red_m[threadIdx.x >> 5] = m;
      red_s[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = red_m[0], S = red_s[0];
      for (int w = 1; w < CE_THREADS / 32; ++w) online_merge(M, S, red_m[w], red_s[w]);
      const float lse = M + __logf(S);
      sh_lse = lse;
      if (lse_out) lse_out[row] = lse;
      if (loss) loss[row] = ignored ? 0.f : lse - __bfloat162float(lr[label]) * logit_scale;
    }
    __syncthreads();
  } else if (threadIdx.x == 0 && loss) {
    loss[row] = 0.f;
  }
  if (!write_grad) return;

  if (ignored) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < nv; i += CE_THREADS) l4[i] = z;
    for (int i = nv * 8 + threadIdx.x; i < V; i += CE_THREADS) lr[i] = __float2bfloat16(0.f);
    return;
  }
  const float lse = sh_lse;
  const float gs = grad_scale * logit_scale;
  const int lab = (int)label;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    const uint4 v = l4[i];
    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
    float g[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(vv[e]);
      g[2 * e] = __expf(f.x * logit_scale - lse) * gs;
      g[2 * e + 1] = __expf(f.y * logit_scale - lse) * gs;
    }
    if ((lab >> 3) == i) g[lab & 7] -= gs;
    l4[i] = make_uint4(pack_bf16x2(g[0], g[1]), pack_bf16x2(g[2], g[3]), pack_bf16x2(g[4], g[5]), pack_bf16x2(g[6], g[7]));
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[i]) * logit_scale - lse) * gs;
    if (i == lab) g -= gs;
    lr[i] = __float2bfloat16(g);
  }
}

// ---- vocabulary-parallel form: every rank holds the logits of the vocabulary slice [vocab_start, vocab_start + V) -------
// Pass 1 per rank: (row maximum, sum of exponentials relative to it, target logit if the label lies in the slice).
// The ranks' triples are combined outside (one all-gather of [T, 3] floats), which yields the row's log-sum-exp;
// pass 2 writes this rank's slice of the gradient  row_scale * (exp(z - lse) - onehot).
__global__ void __launch_bounds__(CE_THREADS)
    ce_shard_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ stats, int V,
                          long long row_stride, long long vocab_start, long long ignore_index) {
  __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + (long long)row * row_stride;
  const bool vec_ok = (row_stride % 8 == 0) && (reinterpret_cast<uintptr_t>(logits) % 16 == 0);
  const int nv = vec_ok ? V / 8 : 0;
  const uint4* l4 = reinterpret_cast<const uint4*>(lr);
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    const uint4 v = l4[i];
    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(vv[e]);
      online_update(m, s, f.x);
      online_update(m, s, f.y);
    }
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += CE_THREADS) online_update(m, s, __bfloat162float(lr[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) {
    red_m[threadIdx.x >> 5] = m;
    red_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = red_m[0], S = red_s[0];
    for (int w = 1; w < CE_THREADS / 32; ++w) online_merge(M, S, red_m[w], red_s[w]);
    const long long label = labels[row];
    const long long local = label - vocab_start;
    const bool mine = label != ignore_index && local >= 0 && local < V;
    stats[3 * row] = M;
    stats[3 * row + 1] = S;
    stats[3 * row + 2] = mine ? __bfloat162float(lr[local]) : 0.f;
  }
}

__global__ void __launch_bounds__(CE_THREADS)
    ce_shard_grad_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ lse,
                         const float* __restrict__ row_scale, __nv_bfloat16* __restrict__ grad, int V, long long row_stride,
                         long long vocab_start, long long ignore_index) {
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + (long long)row * row_stride;
  __nv_bfloat16* gr = grad + (long long)row * V;
  const long long label = labels[row];
  const bool ignored = label == ignore_index;
  const float gs = ignored ? 0.f : row_scale[row];
  const float l = lse[row];
  const long long local = label - vocab_start;
  const int lab = (!ignored && local >= 0 && local < V) ? (int)local : -1;
  const bool vec_ok = (row_stride % 8 == 0) && (V % 8 == 0) && (reinterpret_cast<uintptr_t>(logits) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(grad) % 16 == 0);
  const int nv = vec_ok ? V / 8 : 0;
  const uint4* l4 = reinterpret_cast<const uint4*>(lr);
  uint4* g4 = reinterpret_cast<uint4*>(gr);
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    const uint4 v = l4[i];
    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
    float g[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(vv[e]);
      g[2 * e] = __expf(f.x - l) * gs;
      g[2 * e + 1] = __expf(f.y - l) * gs;
    }
    if (lab >= 0 && (lab >> 3) == i) g[lab & 7] -= gs;
    g4[i] = make_uint4(pack_bf16x2(g[0], g[1]), pack_bf16x2(g[2], g[3]), pack_bf16x2(g[4], g[5]), pack_bf16x2(g[6], g[7]));
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[i]) - l) * gs;
    if (i == lab) g -= gs;
    gr[i] = __float2bfloat16(g);
  }
}

}  // namespace

void cross_entropy_shard_stats(const void* logits, const long long* labels, float* stats, int T, int V, long long row_stride,
                               long long vocab_start, long long ignore_index, cudaStream_t stream) {
  if (T == 0) return;
  ce_shard_stats_kernel<<<T, CE_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels, stats, V, row_stride,
                                                      vocab_start, ignore_index);
  count_launch();
  check_cuda(cudaGetLastError(), "cross_entropy_shard_stats launch");
}

void cross_entropy_shard_grad(const void* logits, const long long* labels, const float* lse, const float* row_scale, void* grad, int T,
                              int V, long long row_stride, long long vocab_start, long long ignore_index, cudaStream_t stream) {
  if (T == 0) return;
  ce_shard_grad_kernel<<<T, CE_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels, lse, row_scale,
                                                     reinterpret_cast<__nv_bfloat16*>(grad), V, row_stride, vocab_start, ignore_index);
  count_launch();
  check_cuda(cudaGetLastError(), "cross_entropy_shard_grad launch");
}

// logits: [T, V] bf16 with `row_stride` elements between rows; overwritten by the gradient
// when write_grad is set. loss / lse: optional fp32 [T] outputs.
void cross_entropy_fwd_bwd(void* logits, const long long* labels, float* loss, float* lse, int T, int V,
                           long long row_stride, float logit_scale, float grad_scale, long long ignore_index,
                           bool write_grad, cudaStream_t stream) {
  if (T == 0) return;
  ce_kernel<<<T, CE_THREADS, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(logits), labels, loss, lse, V, row_stride,
                                          logit_scale, grad_scale, ignore_index, write_grad ? 1 : 0);
  count_launch();
  check_cuda(cudaGetLastError(), "cross_entropy launch");
}

}  // namespace b200

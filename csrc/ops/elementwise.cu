// Memory-bound kernels: SwiGLU, rotary embedding, embedding gather/scatter,
// casts, gradient-norm reduction, gradient clipping and the fused AdamW step.
// All of them use 16-byte accesses and grid-stride loops sized from the SM count.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "ops.h"

namespace b200 {

namespace {

__device__ __forceinline__ float silu_f(float x) { return silu_fast(x); }

inline int ew_grid(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// ------------------------------------------------------------------------- SwiGLU
// x is [T, 2I] with up = x[:, :I], gate = x[:, I:]; y = up * silu(gate).
// `tile_owner` (optional): one entry per 128 rows; rows of tiles whose entry is >= `owners` hold no data and are skipped
// (expert-grouped buffers are sized for the worst case, only the used tiles are touched).
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long T, int Iv,
                                  const int* __restrict__ tile_owner, int owners) {
  const long long total = T * Iv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / Iv;
    if (tile_owner != nullptr && tile_owner[t >> 7] >= owners) continue;
    const int c = (int)(idx - t * Iv);
    const uint4 u = x[t * 2 * Iv + c];
    const uint4 g = x[t * 2 * Iv + Iv + c];
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w}, gg[4] = {g.x, g.y, g.z, g.w};
    uint32_t oo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(uu[e]), b = unpack_bf16x2(gg[e]);
      oo[e] = pack_bf16x2(a.x * silu_f(b.x), a.y * silu_f(b.y));
    }
    y[idx] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
  }
}

// dx[:, :I] = dy * silu(gate); dx[:, I:] = dy * up * dsilu(gate); optionally re-emits y.
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, uint4* __restrict__ dx,
                                  uint4* __restrict__ y, long long T, int Iv, const int* __restrict__ tile_owner, int owners) {
  const long long total = T * Iv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / Iv;
    if (tile_owner != nullptr && tile_owner[t >> 7] >= owners) continue;
    const int c = (int)(idx - t * Iv);
    const uint4 u = x[t * 2 * Iv + c];
    const uint4 g = x[t * 2 * Iv + Iv + c];
    const uint4 d = dy[idx];
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w}, gg[4] = {g.x, g.y, g.z, g.w}, dd[4] = {d.x, d.y, d.z, d.w};
    uint32_t du[4], dg[4], yy[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(uu[e]), b = unpack_bf16x2(gg[e]), q = unpack_bf16x2(dd[e]);
      const float s0 = sigmoid_fast(b.x), s1 = sigmoid_fast(b.y);
      const float act0 = b.x * s0, act1 = b.y * s1;
      const float dact0 = s0 * (1.f + b.x * (1.f - s0)), dact1 = s1 * (1.f + b.y * (1.f - s1));
      du[e] = pack_bf16x2(q.x * act0, q.y * act1);
      dg[e] = pack_bf16x2(q.x * a.x * dact0, q.y * a.y * dact1);
      yy[e] = pack_bf16x2(a.x * act0, a.y * act1);
    }
    dx[t * 2 * Iv + c] = make_uint4(du[0], du[1], du[2], du[3]);
    dx[t * 2 * Iv + Iv + c] = make_uint4(dg[0], dg[1], dg[2], dg[3]);
    if (y) y[idx] = make_uint4(yy[0], yy[1], yy[2], yy[3]);
  }
}

// ------------------------------------------------------------------------- RoPE
// In place on a fused projection buffer whose row holds `groups` blocks of
// (q_per_group query heads | one key head | one value head), each head `d` wide.
// Query and key heads are rotated on their last `rd` channels (half-rotation form).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, int T, long long row_stride,
                            int groups, int qpg, int d, int rd, float sign) {
  const int half_v = rd >> 4;  // uint4 vectors in one half of the rotated span
  const int rot_heads = groups * (qpg + 1);
  const long long total = (long long)T * rot_heads * half_v;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int vi = (int)(idx % half_v);
    const long long r = idx / half_v;
    const int hh = (int)(r % rot_heads);
    const int t = (int)(r / rot_heads);
    const int grp = hh / (qpg + 1), slot = hh % (qpg + 1);
    __nv_bfloat16* base = qkv + (long long)t * row_stride + ((long long)grp * (qpg + 2) + slot) * d + (d - rd);
    uint4* p1 = reinterpret_cast<uint4*>(base) + vi;
    uint4* p2 = reinterpret_cast<uint4*>(base + (rd >> 1)) + vi;
    const int p = pos ? pos[t] : t;
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * (rd >> 1) + vi * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * (rd >> 1) + vi * 8);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float cc[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float ss[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    const uint4 a = *p1, b = *p2;
    const uint32_t aa[4] = {a.x, a.y, a.z, a.w}, bb[4] = {b.x, b.y, b.z, b.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x1 = unpack_bf16x2(aa[e]), x2 = unpack_bf16x2(bb[e]);
      const float s0 = ss[2 * e] * sign, s1 = ss[2 * e + 1] * sign;
      o1[e] = pack_bf16x2(x1.x * cc[2 * e] - x2.x * s0, x1.y * cc[2 * e + 1] - x2.y * s1);
      o2[e] = pack_bf16x2(x2.x * cc[2 * e] + x1.x * s0, x2.y * cc[2 * e + 1] + x1.y * s1);
    }
    *p1 = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *p2 = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

// ------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const uint4* __restrict__ w, const long long* __restrict__ ids,
                                     uint4* __restrict__ out, int T, int Hv, float scale) {
  const long long total = (long long)T * Hv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / Hv);
    const int c = (int)(idx - (long long)t * Hv);
    uint4 v = w[ids[t] * Hv + c];
    if (scale != 1.f) {
      uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(vv[e]);
        vv[e] = pack_bf16x2(f.x * scale, f.y * scale);
      }
      v = make_uint4(vv[0], vv[1], vv[2], vv[3]);
    }
    out[idx] = v;
  }
}

__global__ void embedding_bwd_kernel(const uint4* __restrict__ dy, const long long* __restrict__ ids,
                                     float* __restrict__ dw, int T, int Hv, float scale) {
  const long long total = (long long)T * Hv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / Hv);
    const int c = (int)(idx - (long long)t * Hv);
    const uint4 v = dy[idx];
    float* dst = dw + (ids[t] * Hv + c) * 8;
    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(vv[e]);
      atomicAdd(dst + 2 * e, f.x * scale);
      atomicAdd(dst + 2 * e + 1, f.y * scale);
    }
  }
}

// ------------------------------------------------------------------------- casts / adds
__global__ void cast_f32_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, long long nv,
                                     const float* __restrict__ src_s, __nv_bfloat16* __restrict__ dst_s, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const float4 f = src[i];
    dst[i] = make_uint2(pack_bf16x2(f.x, f.y), pack_bf16x2(f.z, f.w));
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) dst_s[i] = __float2bfloat16(src_s[i]);
  }
}

__global__ void cast_bf16_f32_kernel(const uint2* __restrict__ src, float4* __restrict__ dst, long long nv,
                                     const __nv_bfloat16* __restrict__ src_s, float* __restrict__ dst_s, long long n,
                                     int accumulate, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const uint2 v = src[i];
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
    float4 o = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
    if (accumulate) {
      const float4 old = dst[i];
      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
    }
    dst[i] = o;
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) {
      const float f = __bfloat162float(src_s[i]) * scale;
      dst_s[i] = accumulate ? dst_s[i] + f : f;
    }
  }
}

__global__ void add_bf16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                long long nv) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = a[i], y = b[i];
    const uint32_t xx[4] = {x.x, x.y, x.z, x.w}, yy[4] = {y.x, y.y, y.z, y.w};
    uint32_t oo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 p = unpack_bf16x2(xx[e]), q = unpack_bf16x2(yy[e]);
      oo[e] = pack_bf16x2(p.x + q.x, p.y + q.y);
    }
    out[i] = make_uint4(oo[0], oo[1], oo[2], oo[3]);
  }
}

// ------------------------------------------------------------------------- gradient norm
constexpr int SUMSQ_THREADS = 512;

__global__ void __launch_bounds__(SUMSQ_THREADS)
    sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partials) {
  __shared__ float red[SUMSQ_THREADS / 32];
  float s = 0.f;
  const long long nv = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    const float4 f = x4[i];
    s += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
  }
  if (blockIdx.x == 0) {
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < SUMSQ_THREADS / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

__global__ void sum_partials_kernel(const float* __restrict__ partials, int count, float* __restrict__ out,
                                    int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) s += partials[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
  }
}

__global__ void clip_coef_kernel(const float* __restrict__ total_sq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm) {
  const float nrm = sqrtf(total_sq[0]);
  if (norm) norm[0] = nrm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (nrm + 1e-6f));
  coef[0] = c;
}

// ------------------------------------------------------------------------- AdamW
// Decoupled weight decay, bias-corrected moments (the update rule of torch.optim.AdamW).
// The gradient is multiplied by grad_mul and by *grad_scale (the clipping coefficient,
// resident on the device) before use; the bf16 working copy of the parameter is refreshed
// in the same pass and the gradient is optionally cleared for the next accumulation.
__global__ void adamw_kernel(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v,
                             float4* __restrict__ g, uint2* __restrict__ pb, long long nv, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2_sqrt, const float* __restrict__ grad_scale,
                             float grad_mul, int zero_grad) {
  const float gs = (grad_scale ? grad_scale[0] : 1.f) * grad_mul;
  const float step = lr / bc1;
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float4 P = p[i], M = m[i], V = v[i];
    const float4 G = g[i];
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
    p[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    m[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    v[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (pb) pb[i] = make_uint2(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]));
    if (zero_grad) g[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

}  // namespace

void swiglu_fwd(const void* x, void* y, long long T, int I, cudaStream_t stream, const int* tile_owner, int owners) {
  if (T == 0) return;
  if (I % 8) throw std::runtime_error("swiglu: intermediate size must be a multiple of 8");
  const int Iv = I / 8;
  swiglu_fwd_kernel<<<ew_grid(T * Iv, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(x),
                                                             reinterpret_cast<uint4*>(y), T, Iv, tile_owner, owners);
  count_launch();
  check_cuda(cudaGetLastError(), "swiglu_fwd launch");
}

void swiglu_bwd(const void* dy, const void* x, void* dx, void* y_recompute, long long T, int I, cudaStream_t stream,
                const int* tile_owner, int owners) {
  if (T == 0) return;
  if (I % 8) throw std::runtime_error("swiglu: intermediate size must be a multiple of 8");
  const int Iv = I / 8;
  swiglu_bwd_kernel<<<ew_grid(T * Iv, 256), 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(dy), reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(dx),
      reinterpret_cast<uint4*>(y_recompute), T, Iv, tile_owner, owners);
  count_launch();
  check_cuda(cudaGetLastError(), "swiglu_bwd launch");
}

void rope_inplace(void* qkv, const float* cos_t, const float* sin_t, const int* position_ids, int T, long long row_stride,
                  int num_kv_groups, int q_per_group, int head_dim, int rope_dim, bool inverse, cudaStream_t stream) {
  if (T == 0) return;
  if (rope_dim % 16 || head_dim % 8 || (head_dim - rope_dim) % 8 || row_stride % 8)
    throw std::runtime_error("rope: rope_dim must be a multiple of 16 and head_dim/row_stride multiples of 8");
  const long long total = (long long)T * num_kv_groups * (q_per_group + 1) * (rope_dim / 16);
  rope_kernel<<<ew_grid(total, 256), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(qkv), cos_t, sin_t, position_ids,
                                                      T, row_stride, num_kv_groups, q_per_group, head_dim, rope_dim,
                                                      inverse ? -1.f : 1.f);
  count_launch();
  check_cuda(cudaGetLastError(), "rope launch");
}

void embedding_fwd(const void* weight, const long long* ids, void* out, int T, int H, float scale, cudaStream_t stream) {
  if (T == 0) return;
  if (H % 8) throw std::runtime_error("embedding: hidden size must be a multiple of 8");
  embedding_fwd_kernel<<<ew_grid((long long)T * (H / 8), 256), 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(weight), ids, reinterpret_cast<uint4*>(out), T, H / 8, scale);
  count_launch();
  check_cuda(cudaGetLastError(), "embedding_fwd launch");
}

void embedding_bwd(const void* dy, const long long* ids, float* dweight, int T, int H, float scale,
                   cudaStream_t stream) {
  if (T == 0) return;
  if (H % 8) throw std::runtime_error("embedding: hidden size must be a multiple of 8");
  embedding_bwd_kernel<<<ew_grid((long long)T * (H / 8), 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(dy), ids,
                                                                                dweight, T, H / 8, scale);
  count_launch();
  check_cuda(cudaGetLastError(), "embedding_bwd launch");
}

void cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n == 0) return;
  const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) && (reinterpret_cast<uintptr_t>(dst) % 8 == 0);
  const long long nv = aligned ? n / 4 : 0;
  cast_f32_bf16_kernel<<<ew_grid(nv > 0 ? nv : n, 256), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(src), reinterpret_cast<uint2*>(dst), nv, src, reinterpret_cast<__nv_bfloat16*>(dst),
      n);
  count_launch();
  check_cuda(cudaGetLastError(), "cast_f32_to_bf16 launch");
}

void cast_bf16_to_f32(const void* src, float* dst, long long n, bool accumulate, float scale, cudaStream_t stream) {
  if (n == 0) return;
  const bool aligned = (reinterpret_cast<uintptr_t>(dst) % 16 == 0) && (reinterpret_cast<uintptr_t>(src) % 8 == 0);
  const long long nv = aligned ? n / 4 : 0;
  cast_bf16_f32_kernel<<<ew_grid(nv > 0 ? nv : n, 256), 256, 0, stream>>>(
      reinterpret_cast<const uint2*>(src), reinterpret_cast<float4*>(dst), nv,
      reinterpret_cast<const __nv_bfloat16*>(src), dst, n, accumulate ? 1 : 0, scale);
  count_launch();
  check_cuda(cudaGetLastError(), "cast_bf16_to_f32 launch");
}

void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n == 0) return;
  if (n % 8) throw std::runtime_error("add_bf16: element count must be a multiple of 8");
  add_bf16_kernel<<<ew_grid(n / 8, 256), 256, 0, stream>>>(reinterpret_cast<const uint4*>(a),
                                                          reinterpret_cast<const uint4*>(b),
                                                          reinterpret_cast<uint4*>(out), n / 8);
  count_launch();
  check_cuda(cudaGetLastError(), "add_bf16 launch");
}

int sumsq_partial_count(long long n) {
  long long blocks = (n / 4 + SUMSQ_THREADS - 1) / SUMSQ_THREADS;
  const long long cap = (long long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// partials: scratch of sumsq_partial_count(n) floats. out[0] (+)= sum(x^2), in a fixed order.
void sumsq_f32(const float* x, long long n, float* partials, float* out, bool accumulate, cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(x) % 16) throw std::runtime_error("sumsq: input must be 16-byte aligned");
  const int blocks = sumsq_partial_count(n);
  sumsq_partial_kernel<<<blocks, SUMSQ_THREADS, 0, stream>>>(x, n, partials);
  sum_partials_kernel<<<1, 1024, 0, stream>>>(partials, blocks, out, accumulate ? 1 : 0);
  count_launch(2);
  check_cuda(cudaGetLastError(), "sumsq launch");
}

void clip_coef(const float* total_sq, float max_norm, float* coef, float* norm, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(total_sq, max_norm, coef, norm);
  count_launch();
  check_cuda(cudaGetLastError(), "clip_coef launch");
}

void adamw_step(float* p, float* m, float* v, float* g, void* p_bf16, long long n, float lr, float beta1, float beta2,
                float eps, float weight_decay, float bias_c1, float bias_c2, const float* grad_scale, float grad_mul,
                bool zero_grad, cudaStream_t stream) {
  if (n == 0) return;
  if (n % 4) throw std::runtime_error("adamw: segment length must be a multiple of 4");
  adamw_kernel<<<ew_grid(n / 4, 256), 256, 0, stream>>>(
      reinterpret_cast<float4*>(p), reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v),
      reinterpret_cast<float4*>(g), reinterpret_cast<uint2*>(p_bf16), n / 4, lr, beta1, beta2, eps, weight_decay,
      bias_c1, sqrtf(bias_c2), grad_scale, grad_mul, zero_grad ? 1 : 0);
  count_launch();
  check_cuda(cudaGetLastError(), "adamw launch");
}

}  // namespace b200

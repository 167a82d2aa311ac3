// Launch interface of the packed-sequence attention kernels (attention_fwd.cu, attention_bwd.cu).
#pragma once

#include <cuda_runtime.h>

namespace b200 {

// qkv: fused projection [T, groups * (qpg + 2) * head_dim] bf16 (row stride qkv_stride elements).
// out: [T, groups * qpg * head_dim] bf16. lse: [groups * qpg, T] fp32 (natural log).
void attn_varlen_fwd(const void* qkv, long long qkv_stride, void* out, long long out_stride, float* lse,
                     const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale,
                     bool causal, int* status, cudaStream_t stream);

// dout/out: [T, groups * qpg * head_dim] bf16; dqkv: same layout as qkv (every element is written).
// delta: scratch [groups * qpg, T] fp32; dq_accum: scratch [T, groups * qpg * head_dim] fp32.
void attn_varlen_bwd(const void* dout, const void* qkv, long long qkv_stride, const void* out, long long out_stride,
                     const float* lse, float* delta, float* dq_accum, void* dqkv, long long dqkv_stride,
                     const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale,
                     bool causal, int* status, cudaStream_t stream);

// Cycle counters of the first CTA of every following attn_varlen_bwd launch go to `words` (16 int64; nullptr turns it off).
void attn_bwd_set_trace(long long* words);

// Stick-breaking attention forward (sb_attention_fwd.cu): same buffers; rem: [groups * qpg, T] fp32 = 1 - sum of weights.
void sb_attn_varlen_fwd(const void* qkv, long long qkv_stride, void* out, long long out_stride, float* rem, const int* cu_seqlens,
                        int num_docs, int T, int groups, int qpg, int head_dim, float scale, int* status, cudaStream_t stream);

// Stick-breaking attention backward (sb_attention_bwd.cu). rem / drem: [groups * qpg, T] fp32 (forward output and its
// gradient); gtot: scratch [groups * qpg, T] fp32; dk_accum / dv_accum: scratch [T, groups * head_dim] fp32; dqkv: layout of qkv.
void sb_attn_varlen_bwd(const void* dout, const void* qkv, long long qkv_stride, const void* out, long long out_stride, const float* rem,
                        const float* drem, float* gtot, float* dk_accum, float* dv_accum, void* dqkv, long long dqkv_stride,
                        const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale, int* status,
                        cudaStream_t stream);

}  // namespace b200

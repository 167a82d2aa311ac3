// Plain C++ launch interface of every kernel in this library (raw pointers and a
// stream; no tensor library types) so that the Python binding layer and C callers
// share one set of entry points.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---- gemm/gemm_bf16.cu
void gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
               bool a_mn, bool b_mn, int epi, float alpha, int* status, int max_ctas, cudaStream_t stream);

// ---- gemm/gemm_bf16_2sm.cu (CTA pairs, 256 x 256 tiles)
void gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                   bool a_mn, bool b_mn, int epi, float alpha, int* status, int max_ctas, cudaStream_t stream);
// fc[M, 2I] = A W^T with W = [up rows | gate rows] and act[M, I] = fc[:, :I] * silu(fc[:, I:]) from one kernel
// (needs I % 128 == 0 and M >= 256).
void gemm_bf16_swiglu(const void* A, const void* W, void* fc, void* act, int M, int I, int K, long long lda, long long ldw,
                      long long ldfc, long long ldact, int* status, cudaStream_t stream);
// d(fc)[M, 2I] and act[M, I] from d(act) = dy[M, K] . W[K, I] and the saved projection fc = [up | gate]: the SwiGLU backward in the
// epilogue of the down-projection's data-gradient GEMM (needs I % 64 == 0 and M >= 256).
void gemm_bf16_swiglu_bwd(const void* dy, const void* W, const void* fc, void* dfc, void* act, int M, int I, int K, long long lddy,
                          long long ldw, long long ldfc, long long lddfc, long long ldact, int* status, cudaStream_t stream);
// Process-wide knobs of the CTA-pair kernel (0 / null = built-in choice); meant for micro-benchmarks.
struct PairGemmTuning {
  int group = 0;               // tile raster: > 0 row panels of that many 256-row tiles, < 0 column panels
  int k_skew = 0;              // start the walk over K at a tile-dependent k-block
  int direct_store = 0;        // epilogue writes from registers instead of bulk tensor stores
  int split_k = 0;             // accumulating epilogues: partial sums over K per tile (0 = built-in choice, 1 = none)
  long long* trace = nullptr;  // device buffer of 8 cycle counters per CTA, filled by the traced build of the kernel
};
PairGemmTuning& pair_gemm_tuning();

// ---- ops/norm.cu
int rmsnorm_bwd_partial_rows(int T);
void rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd, int T, int H,
                 float eps, cudaStream_t stream);
void rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dh,
                 float* partial, float* dw, bool accumulate_dw, int T, int H, cudaStream_t stream);

// ---- ops/elementwise.cu
// tile_owner / owners (optional): rows of 128-row tiles whose owner entry is >= owners are skipped.
void swiglu_fwd(const void* x, void* y, long long T, int I, cudaStream_t stream, const int* tile_owner = nullptr, int owners = 0);
void swiglu_bwd(const void* dy, const void* x, void* dx, void* y_recompute, long long T, int I, cudaStream_t stream,
                const int* tile_owner = nullptr, int owners = 0);
void rope_inplace(void* qkv, const float* cos_t, const float* sin_t, const int* position_ids, int T, long long row_stride,
                  int num_kv_groups, int q_per_group, int head_dim, int rope_dim, bool inverse, cudaStream_t stream);
void embedding_fwd(const void* weight, const long long* ids, void* out, int T, int H, float scale, cudaStream_t stream);
void embedding_bwd(const void* dy, const long long* ids, float* dweight, int T, int H, float scale,
                   cudaStream_t stream);
void cast_f32_to_bf16(const float* src, void* dst, long long n, cudaStream_t stream);
void cast_bf16_to_f32(const void* src, float* dst, long long n, bool accumulate, float scale, cudaStream_t stream);
void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream);
int sumsq_partial_count(long long n);
void sumsq_f32(const float* x, long long n, float* partials, float* out, bool accumulate, cudaStream_t stream);
void clip_coef(const float* total_sq, float max_norm, float* coef, float* norm, cudaStream_t stream);
void adamw_step(float* p, float* m, float* v, float* g, void* p_bf16, long long n, float lr, float beta1, float beta2,
                float eps, float weight_decay, float bias_c1, float bias_c2, const float* grad_scale, float grad_mul,
                bool zero_grad, cudaStream_t stream);

// ---- ops/cross_entropy.cu
void cross_entropy_fwd_bwd(void* logits, const long long* labels, float* loss, float* lse, int T, int V,
                           long long row_stride, float logit_scale, float grad_scale, long long ignore_index,
                           bool write_grad, cudaStream_t stream);

// vocabulary-parallel form: per-rank (max, sum-exp, target logit) triples of a vocabulary slice, and the slice of the gradient
void cross_entropy_shard_stats(const void* logits, const long long* labels, float* stats, int T, int V, long long row_stride,
                               long long vocab_start, long long ignore_index, cudaStream_t stream);
void cross_entropy_shard_grad(const void* logits, const long long* labels, const float* lse, const float* row_scale, void* grad, int T,
                              int V, long long row_stride, long long vocab_start, long long ignore_index, cudaStream_t stream);

// fp8 GEMM (gemm/gemm_fp8.cu): a_fmt / b_fmt 0 = e4m3, 1 = e5m2; scale_a / scale_b device fp32 scalars or null.
void gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc, bool a_mn,
              bool b_mn, int a_fmt, int b_fmt, int epi, float alpha, const float* scale_a, const float* scale_b, int* status,
              cudaStream_t stream);

// MXFP8 GEMM (gemm/gemm_mxfp8.cu): 8-bit payloads with one UE8M0 scale per 32 elements along K, scale codes in 512-byte
// tiles of 128 rows x 4 blocks; mx_scale_bytes gives the size of such a buffer.
long long mx_scale_bytes(long long rows, long long k);
void gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long long lda,
                long long ldb, long long ldc, bool a_mn, bool b_mn, int a_fmt, int b_fmt, int epi, float alpha, int* status,
                cudaStream_t stream);

}  // namespace b200

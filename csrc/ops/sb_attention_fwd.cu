// Stick-breaking attention forward over packed variable-length sequences (sm_100a), arXiv 2410.17980:
//
//   A[i, j] = sigmoid(z_ij) * prod_{j < k < i} (1 - sigmoid(z_ik)),   z = scale * q k^T,   j < i (strictly causal)
//   out_i = sum_j A[i, j] v_j,       rem_i = 1 - sum_j A[i, j]
//
// Same machinery as the softmax kernel (attention_fwd.cu): q, k, v read in place from the fused projection buffer through
// one strided TMA map, one CTA per 128 query rows of one document and one head, warp 0 = TMA, warp 1 = tcgen05 MMA
// (S = Q K^T into two TMEM buffers, O += A V into a third; the bf16 weights A are written over the S columns they were
// computed from and read there as the A operand of the second product), warps 2-5 = one thread per query row. The
// differences:
//   * key tiles are visited from the diagonal towards the start of the document, because the weight of key j depends on
//     all keys between j and i: every row keeps the product of (1 - sigma(z_ik)) over the keys seen so far, and
//     A[i, j] = sigma(z_ij) * product before the product shrinks by (1 - sigma(z_ij));
//   * the weights are absolute (no normalisation), so O is never rescaled and accumulates across all tiles;
//   * the kernel returns rem (fp32 [heads, T]) instead of a log-sum-exp.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace b200 {

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 128;
constexpr int KV_STAGES = 2;
constexpr int FWD_THREADS = 192;

template <int D>
struct FwdSmem {
  static constexpr int Q_BYTES = BLOCK_M * D * 2;
  static constexpr int K_BYTES = BLOCK_N * D * 2;
  static constexpr int V_BYTES = BLOCK_N * D * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * K_BYTES;
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * V_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

// barrier indices
enum { B_Q = 0, B_KV_FULL = 1, B_KV_EMPTY = 3, B_S_FULL = 5, B_P_READY = 7, B_PV_DONE = 8, B_COUNT = 9 };

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    sb_attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ rem,
                    const int* __restrict__ cu_seqlens, int num_docs, int T, int groups, int qpg, long long out_stride,
                    float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = FwdSmem<D>;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_slot + 2);  // [doc_start, doc_len, q_tile] or doc_len = -1

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x;  // query head (fastest grid index: the long tiles of every head are scheduled first)
  const int grp = head / qpg;
  const int q_col = (grp * (qpg + 2) + (head - grp * qpg)) * D;
  const int k_col = (grp * (qpg + 2) + qpg) * D;
  const int v_col = k_col + D;

  if (threadIdx.x == 0) {
    // Map this CTA to (document, query tile); heavy (late) tiles of each document are handed out first.
    const int want = gridDim.y - 1 - blockIdx.y;
    int acc = 0, found = -1, start = 0, len = -1, qt = 0;
    for (int b = 0; b < num_docs; ++b) {
      const int s = cu_seqlens[b], e = cu_seqlens[b + 1];
      const int nt = (e - s + BLOCK_M - 1) / BLOCK_M;
      if (want < acc + nt) {
        found = b;
        start = s;
        len = e - s;
        qt = want - acc;
        break;
      }
      acc += nt;
    }
    s_tile[0] = start;
    s_tile[1] = found < 0 ? -1 : len;
    s_tile[2] = qt;
    mbar_init(&bars[B_Q], 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars[B_KV_FULL + s], 1);
      mbar_init(&bars[B_KV_EMPTY + s], 1);
      mbar_init(&bars[B_S_FULL + s], 1);
    }
    mbar_init(&bars[B_P_READY], 128);
    mbar_init(&bars[B_PV_DONE], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const int doc_start = s_tile[0];
  const int doc_len = s_tile[1];
  const int q_tile = s_tile[2];
  if (doc_len <= 0) return;  // uniform: surplus CTA of the upper-bound grid

  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;             // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 2 * BLOCK_N;  // D columns

  const int q0 = q_tile * BLOCK_M;  // first query row of this tile, relative to the document
  const int kv_end = min(doc_len, q0 + BLOCK_M);
  const int n_tiles = (kv_end + BLOCK_N - 1) / BLOCK_N;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      mbar_arrive_expect_tx(&bars[B_Q], L::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < D / 64; ++kb) tma_load_2d(sQ + kb * (BLOCK_M * 128), &tm_qkv, &bars[B_Q], q_col + kb * 64, doc_start + q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&bars[B_KV_EMPTY + st], ph ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
          break;
        }
        mbar_arrive_expect_tx(&bars[B_KV_FULL + st], L::K_BYTES + L::V_BYTES);
        const int row = doc_start + (n_tiles - 1 - j) * BLOCK_N;  // from the diagonal backwards
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) {
          tma_load_2d(sK + st * L::K_BYTES + kb * (BLOCK_N * 128), &tm_qkv, &bars[B_KV_FULL + st], k_col + kb * 64, row);
          tma_load_2d(sV + st * L::V_BYTES + kb * (BLOCK_N * 128), &tm_qkv, &bars[B_KV_FULL + st], v_col + kb * 64, row);
        }
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BLOCK_M, BLOCK_N, 0, 0);  // S = Q K^T, both K-major
      constexpr uint32_t idesc_o = umma_idesc_bf16(BLOCK_M, D, 0, 1);        // O = P V, V is MN-major
      const uint32_t q_base = smem_u32(sQ);
      bool ok = mbar_wait(&bars[B_Q], 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int st = j % KV_STAGES;
        if (!mbar_wait(&bars[B_KV_FULL + st], (j / KV_STAGES) & 1, abort_flag)) return false;
        tc_fence_after_sync();
        // No wait for the S buffer: it last held S(j-2) and then the weights of tile j-2, which O += A V(j-2) has read;
        // that product was issued by this thread before this one, and the tensor cores retire in order.
        const uint32_t k_base = smem_u32(sK + st * L::K_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BLOCK_M * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_S0 + st * BLOCK_N, umma_smem_desc_sw128(q_base + off, 16, 1024),
                      umma_smem_desc_sw128(k_base + off, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_S_FULL + st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait(&bars[B_P_READY], j & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int st = j % KV_STAGES;
        const uint32_t v_base = smem_u32(sV + st * L::V_BYTES);
#pragma unroll
        for (int k = 0; k < BLOCK_N / 16; ++k) {
          // 16 keys per step: their bf16 weights are 8 columns of the tile's S buffer
          const uint64_t db = umma_smem_desc_sw128(v_base + k * 16 * 128, BLOCK_N * 128, 1024);
          umma_f16_ts(tmem_O, tmem_S0 + st * BLOCK_N + k * 8, db, idesc_o, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_KV_EMPTY + st]);
        umma_commit(&bars[B_PV_DONE]);
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutMma, abort_flag);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int q = warp & 3;              // TMEM lane quarter of this warp
    const int r = q * 32 + lane;         // row inside the tile
    const int q_local = q0 + r;          // row inside the document
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    float keep = 1.f;     // product of (1 - sigmoid(z)) over the keys already visited (those between the current key and the query)
    const float scale_log2 = scale * 1.4426950408889634f;
    float a_total = 0.f;  // sum of the weights
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j % KV_STAGES;
      if (!mbar_wait(&bars[B_S_FULL + st], (j / 2) & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t s[BLOCK_N];
#pragma unroll
      for (int c = 0; c < BLOCK_N / 32; ++c) B200_TMEM_LD_32((s + c * 32), tmem_S0 + lane_addr + st * BLOCK_N + c * 32);
      tmem_ld_wait();

      const int kv0 = (n_tiles - 1 - j) * BLOCK_N;
      uint32_t p[BLOCK_N / 2];
      float row_sum = 0.f;
#pragma unroll
      for (int c = BLOCK_N - 2; c >= 0; c -= 2) {
        float w[2];
#pragma unroll
        for (int h = 1; h >= 0; --h) {  // the later key first
          const int kv = kv0 + c + h;
          if (kv < q_local && kv < doc_len) {
            // sigma = e^z / (1 + e^z), 1 - sigma = 1 / (1 + e^z): one exponential and one reciprocal per element; the
            // product of (1 - sigma) over the keys already visited is carried in the linear domain (z clamped at 60)
            const float ez = fast_exp2(fminf(__uint_as_float(s[c + h]) * scale_log2, 86.f));
            const float inv = fast_rcp(1.f + ez);
            w[h] = ez * inv * keep;
            keep *= inv;
          } else {
            w[h] = 0.f;
          }
        }
        row_sum += w[0] + w[1];
        p[c / 2] = pack_bf16x2(w[0], w[1]);
      }
      a_total += row_sum;

      // weights (bf16 pairs) over the first 64 of the 128 S columns this thread has read: the A operand of the second product
      B200_TMEM_ST_32(tmem_S0 + lane_addr + st * BLOCK_N, p);
      B200_TMEM_ST_32(tmem_S0 + lane_addr + st * BLOCK_N + 32, (p + 32));
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[B_P_READY]);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(&bars[B_PV_DONE], (n_tiles - 1) & 1, abort_flag);
    if (!ok) {
      raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
    } else {
      tc_fence_after_sync();
      const float inv_l = 1.f;
      const bool valid = q_local < doc_len;
      __nv_bfloat16* orow = out + (long long)(doc_start + q_local) * out_stride + (long long)head * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        B200_TMEM_LD_32(o, tmem_O + lane_addr + c * 32);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * e + 0]) * inv_l, __uint_as_float(o[8 * e + 1]) * inv_l);
            w.y = pack_bf16x2(__uint_as_float(o[8 * e + 2]) * inv_l, __uint_as_float(o[8 * e + 3]) * inv_l);
            w.z = pack_bf16x2(__uint_as_float(o[8 * e + 4]) * inv_l, __uint_as_float(o[8 * e + 5]) * inv_l);
            w.w = pack_bf16x2(__uint_as_float(o[8 * e + 6]) * inv_l, __uint_as_float(o[8 * e + 7]) * inv_l);
            reinterpret_cast<uint4*>(orow + c * 32)[e] = w;
          }
        }
      }
      if (valid) rem[(long long)head * T + doc_start + q_local] = 1.f - a_total;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
void launch_fwd(const CUtensorMap& tm, void* out, float* rem, const int* cu_seqlens, int num_docs, int T, int groups,
                int qpg, long long out_stride, float scale, int* status, cudaStream_t stream) {
  auto kernel = sb_attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::TOTAL), "sb_attn_fwd smem attr");
    configured = true;
  }
  const int tiles_upper = (T + BLOCK_M - 1) / BLOCK_M + num_docs;
  dim3 grid(groups * qpg, tiles_upper);
  kernel<<<grid, FWD_THREADS, FwdSmem<D>::TOTAL, stream>>>(tm, reinterpret_cast<__nv_bfloat16*>(out), rem, cu_seqlens, num_docs, T,
                                                           groups, qpg, out_stride, scale, status);
  count_launch();
  check_cuda(cudaGetLastError(), "sb_attn_fwd launch");
}

}  // namespace

void sb_attn_varlen_fwd(const void* qkv, long long qkv_stride, void* out, long long out_stride, float* rem, const int* cu_seqlens,
                        int num_docs, int T, int groups, int qpg, int head_dim, float scale, int* status, cudaStream_t stream) {
  if (T == 0 || num_docs == 0) return;
  const long long width = (long long)groups * (qpg + 2) * head_dim;
  const CUtensorMap tm = make_tensor_map_2d_b16(qkv, width, T, qkv_stride, 64, BLOCK_M);
  if (head_dim == 128) launch_fwd<128>(tm, out, rem, cu_seqlens, num_docs, T, groups, qpg, out_stride, scale, status, stream);
  else if (head_dim == 64) launch_fwd<64>(tm, out, rem, cu_seqlens, num_docs, T, groups, qpg, out_stride, scale, status, stream);
  else throw std::runtime_error("sb_attn_varlen_fwd: head_dim must be 64 or 128");
}

}  // namespace b200

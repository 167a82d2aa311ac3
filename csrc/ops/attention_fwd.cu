// Causal softmax attention forward over packed variable-length sequences (sm_100a).
//
// q, k and v are read in place from the fused projection buffer
//   qkv[T, groups * (q_per_group + 2) * D]   (per key/value group: its query heads, then k, then v)
// through one strided TMA tensor map; nothing is split or copied beforehand.
//
// One CTA owns 128 consecutive query rows of one document and one query head:
//   warp 0      TMA producer: Q once, then K tiles and V tiles of 128 keys through two separate 2-stage rings
//   warp 1      MMA issuer : S = Q K^T into one of two TMEM buffers, O += P V into a third
//   warps 2..9  256 softmax threads, two per query row (TMEM lane), each owning half of the key columns: online softmax with lazy
//               rescaling of O (only when the running maximum grew by more than 2^8), P written as bf16 over
//               the S columns of tensor memory it was computed from (the second MMA reads its A operand there,
//               so P never visits shared memory), final O / l and lse
// All waits are bounded; a timeout raises the status word and the CTA unwinds.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace b200 {

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 128;
constexpr int KV_STAGES = 2;
constexpr int SOFTMAX_WARPS = 8;  // two warps per TMEM lane quarter: each thread owns half of the columns of its row
constexpr int FWD_THREADS = 64 + SOFTMAX_WARPS * 32;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

template <int D>
struct FwdSmem {
  static constexpr int Q_BYTES = BLOCK_M * D * 2;
  static constexpr int K_BYTES = BLOCK_N * D * 2;
  static constexpr int V_BYTES = BLOCK_N * D * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * K_BYTES;
  static constexpr int OFF_BAR = OFF_V + KV_STAGES * V_BYTES;
  static constexpr int OFF_X = OFF_BAR + 256;  // row statistics exchanged between the two threads of a row: [2][2][128] floats
  static constexpr int TOTAL = OFF_X + 2 * 2 * BLOCK_M * 4 + 1024;
};

// barrier indices
enum { B_Q = 0, B_K_FULL = 1, B_K_EMPTY = 3, B_V_FULL = 5, B_V_EMPTY = 7, B_S_FULL = 9, B_P_READY = 11, B_PV_DONE = 12, B_COUNT = 13 };

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                    const int* __restrict__ cu_seqlens, int num_docs, int T, int groups, int qpg, long long out_stride,
                    float scale_log2, int causal, int* status) {
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
  float* s_x = reinterpret_cast<float*>(smem + L::OFF_X);

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
      mbar_init(&bars[B_K_FULL + s], 1);
      mbar_init(&bars[B_K_EMPTY + s], 1);
      mbar_init(&bars[B_V_FULL + s], 1);
      mbar_init(&bars[B_V_EMPTY + s], 1);
      mbar_init(&bars[B_S_FULL + s], 1);
    }
    mbar_init(&bars[B_P_READY], SOFTMAX_WARPS * 32);
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
  const int kv_end = causal ? min(doc_len, q0 + BLOCK_M) : doc_len;
  const int n_tiles = (kv_end + BLOCK_N - 1) / BLOCK_N;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      mbar_arrive_expect_tx(&bars[B_Q], L::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < D / 64; ++kb) tma_load_2d(sQ + kb * (BLOCK_M * 128), &tm_qkv, &bars[B_Q], q_col + kb * 64, doc_start + q0);
      // K and V tiles travel through separate 2-stage rings: a K stage is free as soon as its S = Q K^T has retired,
      // long before the V stage of the same tile, so the next-but-one K tile is in flight while this one's softmax runs.
      auto load_tile = [&](int j, bool is_k) -> bool {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        uint64_t* full = &bars[(is_k ? B_K_FULL : B_V_FULL) + st];
        if (!mbar_wait(&bars[(is_k ? B_K_EMPTY : B_V_EMPTY) + st], ph ^ 1, abort_flag)) return false;
        mbar_arrive_expect_tx(full, L::K_BYTES);
        const int row = doc_start + j * BLOCK_N;
        uint8_t* dst = is_k ? sK + st * L::K_BYTES : sV + st * L::V_BYTES;
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) tma_load_2d(dst + kb * (BLOCK_N * 128), &tm_qkv, full, (is_k ? k_col : v_col) + kb * 64, row);
        return true;
      };
      bool ok = load_tile(0, true);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = load_tile(j + 1, true);
        if (ok) ok = load_tile(j, false);
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
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
        if (!mbar_wait(&bars[B_K_FULL + st], (j / KV_STAGES) & 1, abort_flag)) return false;
        tc_fence_after_sync();
        // No wait for the S buffer: it last held S(j-2) and then P(j-2), which O += P V(j-2) has read; that product was
        // issued by this thread before this one (and only after the softmax threads had finished with S(j-2)), and the
        // tensor cores retire in order.
        const uint32_t k_base = smem_u32(sK + st * L::K_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BLOCK_M * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_S0 + st * BLOCK_N, umma_smem_desc_sw128(q_base + off, 16, 1024),
                      umma_smem_desc_sw128(k_base + off, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_K_EMPTY + st]);
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
        const int st = j % KV_STAGES;
        if (!mbar_wait(&bars[B_V_FULL + st], (j / KV_STAGES) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t v_base = smem_u32(sV + st * L::V_BYTES);
#pragma unroll
        for (int k = 0; k < BLOCK_N / 16; ++k) {
          // 16 keys per step; the bf16 P of keys [64 h, 64 h + 64) sits in the first 32 of this tile's S columns [64 h, 64 h + 64)
          const uint64_t db = umma_smem_desc_sw128(v_base + k * 16 * 128, BLOCK_N * 128, 1024);
          umma_f16_ts(tmem_O, tmem_S0 + st * BLOCK_N + (k / 4) * 64 + (k % 4) * 8, db, idesc_o, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_V_EMPTY + st]);
        umma_commit(&bars[B_PV_DONE]);
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutMma, abort_flag);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    constexpr int HALF_N = BLOCK_N / 2;
    const int q = warp & 3;              // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;    // which half of the key columns (and of the output columns) this thread owns
    const int r = q * 32 + lane;         // row inside the tile
    const int q_local = q0 + r;          // row inside the document
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const int pair_bar = 1 + q;          // named barrier of the two warps that share these rows
    float m_used = -INFINITY, l_sum = 0.f;  // l_sum: this thread's columns only
    bool ok = true;
    bool failed = false;  // a bounded wait ran out: carried to the next pair barrier so that both warps of a pair leave together
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j % KV_STAGES;
      const bool got = !failed && mbar_wait(&bars[B_S_FULL + st], (j / 2) & 1, abort_flag);
      tc_fence_after_sync();
      uint32_t s[HALF_N];
#pragma unroll
      for (int c = 0; c < HALF_N / 32; ++c) B200_TMEM_LD_32((s + c * 32), tmem_S0 + lane_addr + st * BLOCK_N + half * HALF_N + c * 32);
      tmem_ld_wait();

      const int kv0 = j * BLOCK_N + half * HALF_N;
      const bool needs_mask = (j * BLOCK_N + BLOCK_N > doc_len) || (causal && j * BLOCK_N + BLOCK_N - 1 > q0);
      if (needs_mask) {
#pragma unroll
        for (int c = 0; c < HALF_N; ++c) {
          const int kv = kv0 + c;
          if (kv >= doc_len || (causal && kv > q_local)) s[c] = __float_as_uint(-INFINITY);
        }
      }
      // maximum of the raw scores (the scale is positive, so it commutes with the maximum), then across the two halves
      float m_raw[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < HALF_N; c += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          m_raw[u] = fmaxf(m_raw[u], fmaxf(__uint_as_float(s[c + 2 * u]), __uint_as_float(s[c + 2 * u + 1])));
      }
      float* x_mine = s_x + ((j & 1) * 2 + half) * BLOCK_M;
      const float* x_other = s_x + ((j & 1) * 2 + (half ^ 1)) * BLOCK_M;
      const float m_half = fmaxf(fmaxf(m_raw[0], m_raw[1]), fmaxf(m_raw[2], m_raw[3]));
      x_mine[r] = m_half;
      // the barrier also carries the outcome of the bounded wait above, so that both warps of a pair leave together
      if (named_barrier_or(pair_bar, 64, !got)) { ok = false; break; }
      const float m_tile = fmaxf(m_half, x_other[r]) * scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_used = m_tile;
      } else if (m_tile > m_used + RESCALE_THRESHOLD) {
        alpha = fast_exp2(m_used - m_tile);
        m_used = m_tile;
        rescale = true;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      // p = 2^(s * scale*log2e - m): one packed multiply-add per pair, one special-function instruction per element
      const float2 scale2 = make_float2(scale_log2, scale_log2), neg_m2 = make_float2(-m_sub, -m_sub);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t p[HALF_N / 2];
#pragma unroll
      for (int c = 0; c < HALF_N; c += 4) {
        const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), scale2, neg_m2);
        const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])), scale2, neg_m2);
        const float2 e0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
        const float2 e1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
        sum2[0] = __fadd2_rn(sum2[0], e0);
        sum2[1] = __fadd2_rn(sum2[1], e1);
        p[c / 2] = pack_bf16x2(e0.x, e0.y);
        p[c / 2 + 1] = pack_bf16x2(e1.x, e1.y);
      }
      const float row_sum = (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      l_sum = l_sum * alpha + row_sum;

      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        // O must be stable: PV of the previous tile retired
        if (!mbar_wait(&bars[B_PV_DONE], (j - 1) & 1, abort_flag)) {
          failed = true;
          *abort_flag = 1;
          continue;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;
          uint32_t o[32];
          B200_TMEM_LD_32(o, tmem_O + lane_addr + c * 32);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          B200_TMEM_ST_32(tmem_O + lane_addr + c * 32, o);
        }
      }
      // P (bf16 pairs) over the first 32 of the 64 S columns this thread has read: the A operand of the second product
      B200_TMEM_ST_32(tmem_S0 + lane_addr + st * BLOCK_N + half * HALF_N, p);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[B_P_READY]);
    }
    ok = ok && !failed;
    if (ok && n_tiles > 0) ok = mbar_wait(&bars[B_PV_DONE], (n_tiles - 1) & 1, abort_flag);
    // total of the two halves of every row (also the point where a pair agrees on having finished)
    float* x_mine = s_x + ((n_tiles & 1) * 2 + half) * BLOCK_M;
    const float* x_other = s_x + ((n_tiles & 1) * 2 + (half ^ 1)) * BLOCK_M;
    x_mine[r] = l_sum;
    if (named_barrier_or(pair_bar, 64, !ok)) ok = false;
    if (!ok) {
      raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
    } else {
      tc_fence_after_sync();
      const float l_row = l_sum + x_other[r];
      const float inv_l = l_row > 0.f ? 1.f / l_row : 0.f;
      const bool valid = q_local < doc_len;
      __nv_bfloat16* orow = out + (long long)(doc_start + q_local) * out_stride + (long long)head * D;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;
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
      if (valid && half == 0) lse[(long long)head * T + doc_start + q_local] = (m_used + log2f(l_row)) * 0.6931471805599453f;
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
void launch_fwd(const CUtensorMap& tm, void* out, float* lse, const int* cu_seqlens, int num_docs, int T, int groups,
                int qpg, long long out_stride, float scale, bool causal, int* status, cudaStream_t stream) {
  auto kernel = attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::TOTAL), "attn_fwd smem attr");
    configured = true;
  }
  const int tiles_upper = (T + BLOCK_M - 1) / BLOCK_M + num_docs;
  dim3 grid(groups * qpg, tiles_upper);
  kernel<<<grid, FWD_THREADS, FwdSmem<D>::TOTAL, stream>>>(tm, reinterpret_cast<__nv_bfloat16*>(out), lse, cu_seqlens,
                                                           num_docs, T, groups, qpg, out_stride,
                                                           scale * 1.4426950408889634f, causal ? 1 : 0, status);
  count_launch();
  check_cuda(cudaGetLastError(), "attn_fwd launch");
}

}  // namespace

void attn_varlen_fwd(const void* qkv, long long qkv_stride, void* out, long long out_stride, float* lse,
                     const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale,
                     bool causal, int* status, cudaStream_t stream) {
  if (T == 0 || num_docs == 0) return;
  const long long width = (long long)groups * (qpg + 2) * head_dim;
  const CUtensorMap tm = make_tensor_map_2d_b16(qkv, width, T, qkv_stride, 64, BLOCK_M);
  if (head_dim == 128) launch_fwd<128>(tm, out, lse, cu_seqlens, num_docs, T, groups, qpg, out_stride, scale, causal, status, stream);
  else if (head_dim == 64) launch_fwd<64>(tm, out, lse, cu_seqlens, num_docs, T, groups, qpg, out_stride, scale, causal, status, stream);
  else throw std::runtime_error("attn_varlen_fwd: head_dim must be 64 or 128");
}

}  // namespace b200

// Causal softmax attention backward over packed variable-length sequences (sm_100a).
//
// One CTA owns 128 keys of one document and one key/value head. K and V stay resident in shared memory;
// the CTA walks the query heads of the group and, for each, the query tiles that can see these keys:
//   S^T  = K Q^T,  dP^T = V dO^T                      (tcgen05, fp32 in TMEM)
//   P^T  = exp2(S^T * scale*log2e - lse*log2e),  dS^T = P^T o (dP^T - delta) * scale   (256 threads: row = key, two warps share a row and split its columns)
//   dV  += P^T dO,  dK += dS^T Q,  dQ_tile = dS K       (tcgen05; dQ is added to an fp32 buffer by bulk tensor reductions)
// The tiles of dS^T / Q / dO / K are each loaded or written once and reused through a second descriptor with
// the other major-ness (e.g. dS^T is the K-major A operand of dK and the MN-major A operand of dQ).
// Two small kernels bracket it: delta = rowsum(dO o O) before, fp32 dQ -> bf16 into the fused gradient after.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace b200 {

namespace {

constexpr int BT = 128;  // tile edge for both queries and keys
constexpr int SOFTMAX_WARPS = 8;  // two warps per TMEM lane quarter, each taking half of the columns
constexpr int BWD_THREADS = 64 + SOFTMAX_WARPS * 32;

template <int D>
struct BwdSmem {
  static constexpr int TILE_D = BT * D * 2;    // a [128 x D] bf16 tile
  static constexpr int TILE_S = BT * BT * 2;   // a [128 x 128] bf16 tile
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_D;
  static constexpr int OFF_Q = OFF_V + TILE_D;
  static constexpr int OFF_DO = OFF_Q + TILE_D;
  static constexpr int OFF_P = OFF_DO + TILE_D;
  static constexpr int OFF_DS = OFF_P + TILE_S;
  static constexpr int OFF_ROW = OFF_DS + TILE_S;       // per softmax warp: lse[64], delta[64] floats
  static constexpr int OFF_BAR = OFF_ROW + 8 * BT * 4;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

enum { B_KV = 0, B_QDO_FULL = 1, B_QDO_EMPTY = 2, B_SDP_FULL = 3, B_PDS_READY = 4, B_MMA2_DONE = 5, B_DQ_DRAINED = 6, B_PDS_FIRST = 7, B_COUNT = 8 };

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dq, const float* __restrict__ lse, const float* __restrict__ delta,
                    __nv_bfloat16* __restrict__ dqkv, long long dqkv_stride, const int* __restrict__ cu_seqlens,
                    int num_docs, int T, int groups, int qpg, float scale, float scale_log2, int causal, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = BwdSmem<D>;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sP = smem + L::OFF_P;
  uint8_t* sDS = smem + L::OFF_DS;
  float* s_rows = reinterpret_cast<float*>(smem + L::OFF_ROW);  // [8 warps][lse 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grp = blockIdx.x;  // key/value head (fastest grid index: the long key tiles of every head are scheduled first)
  const int k_col = (grp * (qpg + 2) + qpg) * D;
  const int v_col = k_col + D;

  if (threadIdx.x == 0) {
    const int want = blockIdx.y;  // early key tiles see the most queries: hand them out first
    int acc = 0, found = -1, start = 0, len = -1, kt = 0;
    for (int b = 0; b < num_docs; ++b) {
      const int s = cu_seqlens[b], e = cu_seqlens[b + 1];
      const int nt = (e - s + BT - 1) / BT;
      if (want < acc + nt) {
        found = b;
        start = s;
        len = e - s;
        kt = want - acc;
        break;
      }
      acc += nt;
    }
    s_tile[0] = start;
    s_tile[1] = found < 0 ? -1 : len;
    s_tile[2] = kt;
    mbar_init(&bars[B_KV], 1);
    mbar_init(&bars[B_QDO_FULL], 1);
    mbar_init(&bars[B_QDO_EMPTY], 1);
    mbar_init(&bars[B_SDP_FULL], 1);
    mbar_init(&bars[B_PDS_READY], SOFTMAX_WARPS * 32);
    mbar_init(&bars[B_PDS_FIRST], SOFTMAX_WARPS * 32);
    mbar_init(&bars[B_MMA2_DONE], 1);
    mbar_init(&bars[B_DQ_DRAINED], SOFTMAX_WARPS * 32);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const int doc_start = s_tile[0];
  const int doc_len = s_tile[1];
  const int kv_tile = s_tile[2];
  if (doc_len <= 0) return;

  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;             // 128 cols, later reused for dQ (D cols)
  const uint32_t tmem_dP = tmem_base + BT;       // 128 cols
  const uint32_t tmem_dV = tmem_base + 2 * BT;   // D cols
  const uint32_t tmem_dK = tmem_base + 2 * BT + D;  // D cols

  const int kv0 = kv_tile * BT;
  const int n_q_tiles = (doc_len + BT - 1) / BT;
  const int first_q_tile = causal ? kv_tile : 0;
  const int tiles_per_head = n_q_tiles - first_q_tile;
  const int n_iter = tiles_per_head * qpg;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(&bars[B_KV], 2 * L::TILE_D);
#pragma unroll
      for (int kb = 0; kb < D / 64; ++kb) {
        tma_load_2d(sK + kb * (BT * 128), &tm_qkv, &bars[B_KV], k_col + kb * 64, doc_start + kv0);
        tma_load_2d(sV + kb * (BT * 128), &tm_qkv, &bars[B_KV], v_col + kb * 64, doc_start + kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int qh = it / tiles_per_head;
        const int qt = first_q_tile + it % tiles_per_head;
        if (!mbar_wait(&bars[B_QDO_EMPTY], (it & 1) ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
          break;
        }
        mbar_arrive_expect_tx(&bars[B_QDO_FULL], 2 * L::TILE_D);
        const int q_col = (grp * (qpg + 2) + qh) * D;
        const int do_col = (grp * qpg + qh) * D;
        const int row = doc_start + qt * BT;
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) {
          tma_load_2d(sQ + kb * (BT * 128), &tm_qkv, &bars[B_QDO_FULL], q_col + kb * 64, row);
          tma_load_2d(sDO + kb * (BT * 128), &tm_do, &bars[B_QDO_FULL], do_col + kb * 64, row);
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
      constexpr uint32_t idesc_st = umma_idesc_bf16(BT, BT, 0, 0);  // S^T = K Q^T, dP^T = V dO^T
      constexpr uint32_t idesc_kv = umma_idesc_bf16(BT, D, 0, 1);   // dV = P^T dO, dK = dS^T Q   (B MN-major)
      constexpr uint32_t idesc_dq = umma_idesc_bf16(BT, D, 1, 1);   // dQ = dS K                 (A and B MN-major)
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
      const uint32_t p_base = smem_u32(sP), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&bars[B_KV], 0, abort_flag);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(&bars[B_QDO_FULL], ph, abort_flag)) { ok = false; break; }
        if (it > 0 && !mbar_wait(&bars[B_DQ_DRAINED], (it - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_S, umma_smem_desc_sw128(k_base + off, 16, 1024), umma_smem_desc_sw128(q_base + off, 16, 1024),
                      idesc_st, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_dP, umma_smem_desc_sw128(v_base + off, 16, 1024), umma_smem_desc_sw128(do_base + off, 16, 1024),
                      idesc_st, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_SDP_FULL]);

        // Every softmax warp produces its first 32 query columns, then its second 32: the dV / dK steps over the first
        // columns (queries 0..31 and 64..95) run while the second ones are still being computed.
        const uint32_t acc = it > 0 ? 1u : 0u;
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          if (!mbar_wait(&bars[part == 0 ? B_PDS_FIRST : B_PDS_READY], ph, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int k = (kk >> 1) * 4 + part * 2 + (kk & 1);
            const uint32_t a_off = (k / 4) * (BT * 128) + (k % 4) * 32;  // K-major A: 16 query columns per step
            const uint32_t b_off = k * 16 * 128;                          // MN-major B: 16 query rows per step
            umma_f16_ss(tmem_dV, umma_smem_desc_sw128(p_base + a_off, 16, 1024),
                        umma_smem_desc_sw128(do_base + b_off, BT * 128, 1024), idesc_kv, (acc | (part | kk) != 0) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int k = (kk >> 1) * 4 + part * 2 + (kk & 1);
            const uint32_t a_off = (k / 4) * (BT * 128) + (k % 4) * 32;
            const uint32_t b_off = k * 16 * 128;
            umma_f16_ss(tmem_dK, umma_smem_desc_sw128(ds_base + a_off, 16, 1024),
                        umma_smem_desc_sw128(q_base + b_off, BT * 128, 1024), idesc_kv, (acc | (part | kk) != 0) ? 1u : 0u);
          }
        }
        if (!ok) break;
        umma_commit(&bars[B_QDO_EMPTY]);  // Q and dO are free once dV and dK have retired: the next tiles load under dQ
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t off = k * 16 * 128;  // 16 key rows per step for both operands
          umma_f16_ss(tmem_S, umma_smem_desc_sw128(ds_base + off, BT * 128, 1024),
                      umma_smem_desc_sw128(k_base + off, BT * 128, 1024), idesc_dq, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_MMA2_DONE]);
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutMma, abort_flag);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- P / dS producers, dQ drain, final dK / dV
    const int q4 = warp & 3;            // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // which half of the columns (of S^T / dP^T, dQ, dK, dV) this warp takes
    const bool is_issuer = warp == 2 && lane == 0;  // issues the bulk reductions of dQ
    const int r = q4 * 32 + lane;  // key row inside the tile (S^T, dV, dK) / query row inside the tile (dQ)
    const int kv_local = kv0 + r;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const bool kv_valid = kv_local < doc_len;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int qh = it / tiles_per_head;
      const int qt = first_q_tile + it % tiles_per_head;
      const int head = grp * qpg + qh;
      const int q0 = qt * BT;
      // Each warp stages the per-query statistics of this tile for itself (no cross-warp barrier needed).
      float* w_lse = s_rows + (half * 4 + q4) * BT;
      float* w_delta = w_lse + BT / 2;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < BT / 64; ++i) {
        const int col = i * 32 + lane;  // relative to this warp's first column
        const int ql = q0 + half * (BT / 2) + col;
        const bool v = ql < doc_len;
        // stored negated (and delta pre-multiplied by the softmax scale) so that each element below is one fused multiply-add
        w_lse[col] = v ? lse[(long long)head * T + doc_start + ql] * -1.4426950408889634f : -INFINITY;
        w_delta[col] = v ? delta[(long long)head * T + doc_start + ql] * -scale : 0.f;
      }
      __syncwarp();
      bool got = mbar_wait(&bars[B_SDP_FULL], it & 1, abort_flag);
      tc_fence_after_sync();
      // Only the diagonal tile and the last key tile of a document mask anything: every other tile takes the short path.
      const bool masked = !kv_valid || (causal && (q0 < kv0 + BT - 1));
      const int first_visible = kv_valid ? (causal ? kv_local - q0 : 0) : BT;  // query columns below this see nothing of this key
      const float2 scale_log2_2 = make_float2(scale_log2, scale_log2), scale_2 = make_float2(scale, scale);
#pragma unroll 1
      for (int cc = 0; cc < BT / 64; ++cc) {
        const int c = half * (BT / 64) + cc;
        uint32_t sv[32], dpv[32];
        B200_TMEM_LD_32(sv, tmem_S + lane_addr + c * 32);
        B200_TMEM_LD_32(dpv, tmem_dP + lane_addr + c * 32);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
        const float4* nl4 = reinterpret_cast<const float4*>(w_lse + cc * 32);
        const float4* nd4 = reinterpret_cast<const float4*>(w_delta + cc * 32);
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 nl = nl4[e / 4], nd = nd4[e / 4];
          // packed fp32 pairs: t = s * scale*log2e - lse*log2e, g = dP * scale - delta * scale
          const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), scale_log2_2, make_float2(nl.x, nl.y));
          const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(sv[e + 2]), __uint_as_float(sv[e + 3])), scale_log2_2, make_float2(nl.z, nl.w));
          const float2 g0 = __ffma2_rn(make_float2(__uint_as_float(dpv[e]), __uint_as_float(dpv[e + 1])), scale_2, make_float2(nd.x, nd.y));
          const float2 g1 = __ffma2_rn(make_float2(__uint_as_float(dpv[e + 2]), __uint_as_float(dpv[e + 3])), scale_2, make_float2(nd.z, nd.w));
          float2 p0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
          float2 p1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
          if (masked) {
            const int col = c * 32 + e;  // query column inside the tile
            if (col < first_visible) p0.x = 0.f;
            if (col + 1 < first_visible) p0.y = 0.f;
            if (col + 2 < first_visible) p1.x = 0.f;
            if (col + 3 < first_visible) p1.y = 0.f;
          }
          const float2 d0 = __fmul2_rn(p0, g0), d1 = __fmul2_rn(p1, g1);
          pp[e / 2] = pack_bf16x2(p0.x, p0.y);
          pp[e / 2 + 1] = pack_bf16x2(p1.x, p1.y);
          dd[e / 2] = pack_bf16x2(d0.x, d0.y);
          dd[e / 2 + 1] = pack_bf16x2(d1.x, d1.y);
        }
        if (cc == 0) {
          // the P / dS tiles double as the staging buffer of the previous dQ tile: its bulk reduction must have read them
          if (is_issuer) tma_store_wait_read<0>();
          if (named_barrier_or(1, SOFTMAX_WARPS * 32, !got)) { ok = false; break; }
        }
        // 32 columns = half of a 64-column K block: four 16-byte chunks of this thread's row
        const int kb = c >> 1;
        uint8_t* prow = sP + kb * (BT * 128) + r * 128;
        uint8_t* drow = sDS + kb * (BT * 128) + r * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c & 1) * 4 + ch) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
          *reinterpret_cast<uint4*>(drow + chunk * 16) = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
        }
        if (cc == 0) {
          fence_proxy_async_smem();
          tc_fence_before_sync();
          mbar_arrive(&bars[B_PDS_FIRST]);
        }
      }
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[B_PDS_READY]);

      got = mbar_wait(&bars[B_MMA2_DONE], it & 1, abort_flag);
      tc_fence_after_sync();
      if (got) {
        // dQ tile -> fp32 staging in shared memory (one 128-byte-swizzled [128 x 32] box per 32 columns, over the P / dS
        // tiles the MMAs have finished with), then one bulk add per box into the fp32 accumulator: full lines at L2
        // instead of scattered 16-byte atomics. Query rows past the document are exact zeros (their P is 0).
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;
          uint32_t o[32];
          B200_TMEM_LD_32(o, tmem_S + lane_addr + c * 32);
          tmem_ld_wait();
          uint8_t* row = sP + c * (BT * 128) + r * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(row + ((ch ^ (r & 7)) * 16)) = make_uint4(o[4 * ch], o[4 * ch + 1], o[4 * ch + 2], o[4 * ch + 3]);
        }
        tc_fence_before_sync();
        mbar_arrive(&bars[B_DQ_DRAINED]);  // the S / dQ columns of TMEM can take the next tile
        fence_proxy_async_smem();
      }
      if (named_barrier_or(2, SOFTMAX_WARPS * 32, !got)) { ok = false; break; }
      if (is_issuer) {
        const int row0 = doc_start + q0;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tma_reduce_add_2d(&tm_dq, sP + c * (BT * 128), head * D + c * 32, row0);
        tma_store_commit();
      }
    }
    if (is_issuer) tma_store_wait<0>();
    if (!ok) {
      raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
    } else {
      // dK and dV of this key tile (all MMAs retired: the last MMA2_DONE wait above)
      tc_fence_after_sync();
      __nv_bfloat16* krow = dqkv + (long long)(doc_start + kv_local) * dqkv_stride + k_col;
      __nv_bfloat16* vrow = krow + D;
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const int c = half * (D / 64) + cc;
        uint32_t a[32], b[32];
        B200_TMEM_LD_32(a, tmem_dK + lane_addr + c * 32);
        B200_TMEM_LD_32(b, tmem_dV + lane_addr + c * 32);
        tmem_ld_wait();
        if (kv_valid) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 wk, wv;
            wk.x = pack_bf16x2(__uint_as_float(a[8 * e + 0]), __uint_as_float(a[8 * e + 1]));
            wk.y = pack_bf16x2(__uint_as_float(a[8 * e + 2]), __uint_as_float(a[8 * e + 3]));
            wk.z = pack_bf16x2(__uint_as_float(a[8 * e + 4]), __uint_as_float(a[8 * e + 5]));
            wk.w = pack_bf16x2(__uint_as_float(a[8 * e + 6]), __uint_as_float(a[8 * e + 7]));
            wv.x = pack_bf16x2(__uint_as_float(b[8 * e + 0]), __uint_as_float(b[8 * e + 1]));
            wv.y = pack_bf16x2(__uint_as_float(b[8 * e + 2]), __uint_as_float(b[8 * e + 3]));
            wv.z = pack_bf16x2(__uint_as_float(b[8 * e + 4]), __uint_as_float(b[8 * e + 5]));
            wv.w = pack_bf16x2(__uint_as_float(b[8 * e + 6]), __uint_as_float(b[8 * e + 7]));
            reinterpret_cast<uint4*>(krow + c * 32)[e] = wk;
            reinterpret_cast<uint4*>(vrow + c * 32)[e] = wv;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ delta, int T, int H, int D, long long stride) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const int t = w / H, h = w - t * H;
  const __nv_bfloat16* a = dout + (long long)t * stride + (long long)h * D;
  const __nv_bfloat16* b = out + (long long)t * stride + (long long)h * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(long long)h * T + t] = s;
}

// dqkv[t, q columns] = bf16(dq_accum[t, :]) for every query head of every group.
__global__ void attn_dq_convert_kernel(const float* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dqkv,
                                       long long dqkv_stride, int T, int groups, int qpg, int D) {
  const int per_row = groups * qpg * D / 4;
  const long long total = (long long)T * per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_row);
    const int c = (int)(idx - (long long)t * per_row) * 4;  // column inside [hq * D]
    const int head = c / D, within = c - head * D;
    const int grp = head / qpg, qh = head - grp * qpg;
    const float4 v = reinterpret_cast<const float4*>(dq_accum)[idx];
    __nv_bfloat16* dst = dqkv + (long long)t * dqkv_stride + ((long long)grp * (qpg + 2) + qh) * D + within;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

template <int D>
void launch_bwd(const CUtensorMap& tm_qkv, const CUtensorMap& tm_do, const CUtensorMap& tm_dq, const float* lse, const float* delta,
                void* dqkv, long long dqkv_stride, const int* cu_seqlens, int num_docs, int T, int groups, int qpg,
                float scale, bool causal, int* status, cudaStream_t stream) {
  auto kernel = attn_bwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::TOTAL), "attn_bwd smem attr");
    configured = true;
  }
  const int tiles_upper = (T + BT - 1) / BT + num_docs;
  dim3 grid(groups, tiles_upper);
  kernel<<<grid, BWD_THREADS, BwdSmem<D>::TOTAL, stream>>>(tm_qkv, tm_do, tm_dq, lse, delta,
                                                           reinterpret_cast<__nv_bfloat16*>(dqkv), dqkv_stride, cu_seqlens,
                                                           num_docs, T, groups, qpg, scale, scale * 1.4426950408889634f,
                                                           causal ? 1 : 0, status);
  check_cuda(cudaGetLastError(), "attn_bwd launch");
}

}  // namespace

void attn_varlen_bwd(const void* dout, const void* qkv, long long qkv_stride, const void* out, long long out_stride,
                     const float* lse, float* delta, float* dq_accum, void* dqkv, long long dqkv_stride,
                     const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale,
                     bool causal, int* status, cudaStream_t stream) {
  if (T == 0 || num_docs == 0) return;
  const int hq = groups * qpg;
  const long long width = (long long)groups * (qpg + 2) * head_dim;
  {
    const long long warps = (long long)T * hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                reinterpret_cast<const __nv_bfloat16*>(out), delta, T, hq,
                                                                head_dim, out_stride);
  }
  check_cuda(cudaMemsetAsync(dq_accum, 0, (size_t)T * hq * head_dim * sizeof(float), stream), "dq_accum memset");
  const CUtensorMap tm_qkv = make_tensor_map_2d_b16(qkv, width, T, qkv_stride, 64, BT);
  const CUtensorMap tm_do = make_tensor_map_2d_b16(dout, (long long)hq * head_dim, T, out_stride, 64, BT);
  const CUtensorMap tm_dq = make_tensor_map_2d_f32(dq_accum, (long long)hq * head_dim, T, (long long)hq * head_dim, 32, BT);
  if (head_dim == 128) launch_bwd<128>(tm_qkv, tm_do, tm_dq, lse, delta, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, causal, status, stream);
  else if (head_dim == 64) launch_bwd<64>(tm_qkv, tm_do, tm_dq, lse, delta, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, causal, status, stream);
  else throw std::runtime_error("attn_varlen_bwd: head_dim must be 64 or 128");
  {
    const long long total = (long long)T * hq * head_dim / 4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    attn_dq_convert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dq_accum, reinterpret_cast<__nv_bfloat16*>(dqkv), dqkv_stride,
                                                                T, groups, qpg, head_dim);
  }
  count_launch(3);
  check_cuda(cudaGetLastError(), "attn_bwd tail launch");
}

}  // namespace b200

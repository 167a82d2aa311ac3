// Stick-breaking attention backward over packed variable-length sequences (sm_100a).
//
// Forward (sb_attention_fwd.cu):  A[i, j] = sigma(z_ij) * prod_{j < k < i} (1 - sigma(z_ik)),  z = scale * q k^T,  j < i,
//                                 out_i = sum_j A[i, j] v_j,   rem_i = 1 - sum_j A[i, j].
// With G[i, j] = A[i, j] * (dO_i . v_j - drem_i) the gradient of the logits is
//   dz_ij = G_ij * (1 - sigma_ij) - sigma_ij * sum_{j' < j} G_ij',    sum_{j' < j} G_ij' = Gtot_i - sum_{j' >= j} G_ij',
//   Gtot_i = dO_i . out_i - drem_i * (1 - rem_i)                      (a row quantity known before the kernel starts),
// so a row can be walked from the diagonal towards the start of the document exactly like the forward pass, carrying the
// running product prod (1 - sigma) and the running sum of G.
//
// One CTA owns 128 query rows of one document and one query head: Q and dO stay in shared memory, the key / value tiles
// stream past from right to left. Per tile:
//   S = Q K^T, dP = dO V^T                        (tcgen05, fp32 in TMEM, lane = query row)
//   A, dS = dz * scale                            (128 threads, one per query row, sequential along the keys)
//   dV_tile = A^T dO, dK_tile = dS^T Q, dQ += dS K (tcgen05; dV / dK tiles reuse the S / dP columns of TMEM)
// dQ stays in TMEM until the end; the dV / dK tiles of every (query tile, head) are added into fp32 buffers with bulk
// tensor reductions from shared memory (several query heads and all later query tiles contribute to one key tile).
// Two small kernels bracket it: Gtot before, fp32 dK / dV -> bf16 into the fused gradient after.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace b200 {

namespace {

constexpr int BT = 128;
constexpr int ROW_THREADS = 128;
constexpr int SB_BWD_THREADS = 64 + ROW_THREADS;

template <int D>
struct SbBwdSmem {
  static constexpr int TILE_D = BT * D * 2;
  static constexpr int TILE_S = BT * BT * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + TILE_D;
  static constexpr int OFF_K = OFF_DO + TILE_D;
  static constexpr int OFF_V = OFF_K + TILE_D;
  static constexpr int OFF_A = OFF_V + TILE_D;     // A (bf16), later the fp32 staging of the dV / dK tiles together with dS
  static constexpr int OFF_DS = OFF_A + TILE_S;
  static constexpr int OFF_BAR = OFF_DS + TILE_S;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

enum { S_QDO = 0, S_KV_FULL = 1, S_KV_EMPTY = 2, S_SDP_FULL = 3, S_PDS_READY = 4, S_MMA2_DONE = 5, S_DRAINED = 6, S_COUNT = 7 };

template <int D>
__global__ void __launch_bounds__(SB_BWD_THREADS, 1)
    sb_attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                       const float* __restrict__ gtot, const float* __restrict__ drem, __nv_bfloat16* __restrict__ dqkv,
                       long long dqkv_stride, const int* __restrict__ cu_seqlens, int num_docs, int T, int groups, int qpg, float scale,
                       int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = SbBwdSmem<D>;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sA = smem + L::OFF_A;
  uint8_t* sDS = smem + L::OFF_DS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x;  // query head (fastest grid index: the long tiles of every head are scheduled first)
  const int grp = head / qpg;
  const int q_col = (grp * (qpg + 2) + (head - grp * qpg)) * D;
  const int k_col = (grp * (qpg + 2) + qpg) * D;
  const int v_col = k_col + D;

  if (threadIdx.x == 0) {
    const int want = gridDim.y - 1 - blockIdx.y;  // late query tiles see the most keys: hand them out first
    int acc = 0, found = -1, start = 0, len = -1, qt = 0;
    for (int b = 0; b < num_docs; ++b) {
      const int s = cu_seqlens[b], e = cu_seqlens[b + 1];
      const int nt = (e - s + BT - 1) / BT;
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
    mbar_init(&bars[S_QDO], 1);
    mbar_init(&bars[S_KV_FULL], 1);
    mbar_init(&bars[S_KV_EMPTY], 1);
    mbar_init(&bars[S_SDP_FULL], 1);
    mbar_init(&bars[S_PDS_READY], ROW_THREADS);
    mbar_init(&bars[S_MMA2_DONE], 1);
    mbar_init(&bars[S_DRAINED], ROW_THREADS);
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
  const uint32_t tmem_S = tmem_base;            // 128 columns: S, then the dV tile (D columns)
  const uint32_t tmem_dP = tmem_base + BT;      // 128 columns: dP, then the dK tile (D columns)
  const uint32_t tmem_dQ = tmem_base + 2 * BT;  // D columns, accumulates over all key tiles

  const int q0 = q_tile * BT;
  const int kv_end = min(doc_len, q0 + BT);  // strictly causal: keys below the last query row of the tile
  const int n_tiles = (kv_end + BT - 1) / BT;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_qkv);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(&bars[S_QDO], 2 * L::TILE_D);
#pragma unroll
      for (int kb = 0; kb < D / 64; ++kb) {
        tma_load_2d(sQ + kb * (BT * 128), &tm_qkv, &bars[S_QDO], q_col + kb * 64, doc_start + q0);
        tma_load_2d(sDO + kb * (BT * 128), &tm_do, &bars[S_QDO], head * D + kb * 64, doc_start + q0);
      }
      for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait(&bars[S_KV_EMPTY], (j & 1) ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
          break;
        }
        mbar_arrive_expect_tx(&bars[S_KV_FULL], 2 * L::TILE_D);
        const int row = doc_start + (n_tiles - 1 - j) * BT;
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) {
          tma_load_2d(sK + kb * (BT * 128), &tm_qkv, &bars[S_KV_FULL], k_col + kb * 64, row);
          tma_load_2d(sV + kb * (BT * 128), &tm_qkv, &bars[S_KV_FULL], v_col + kb * 64, row);
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
      constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BT, 0, 0);   // S = Q K^T, dP = dO V^T (all K-major)
      constexpr uint32_t idesc_t = umma_idesc_bf16(BT, D, 1, 1);    // dV = A^T dO, dK = dS^T Q (A and B MN-major)
      constexpr uint32_t idesc_q = umma_idesc_bf16(BT, D, 0, 1);    // dQ += dS K (B MN-major)
      const uint32_t q_base = smem_u32(sQ), do_base = smem_u32(sDO), k_base = smem_u32(sK), v_base = smem_u32(sV);
      const uint32_t a_base = smem_u32(sA), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&bars[S_QDO], 0, abort_flag);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(&bars[S_KV_FULL], ph, abort_flag)) { ok = false; break; }
        if (j > 0 && !mbar_wait(&bars[S_DRAINED], (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_S, umma_smem_desc_sw128(q_base + off, 16, 1024), umma_smem_desc_sw128(k_base + off, 16, 1024), idesc_s,
                      k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_dP, umma_smem_desc_sw128(do_base + off, 16, 1024), umma_smem_desc_sw128(v_base + off, 16, 1024), idesc_s,
                      k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[S_SDP_FULL]);

        if (!mbar_wait(&bars[S_PDS_READY], ph, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t off = k * 16 * 128;  // 16 query rows per step for both operands
          umma_f16_ss(tmem_S, umma_smem_desc_sw128(a_base + off, BT * 128, 1024), umma_smem_desc_sw128(do_base + off, BT * 128, 1024),
                      idesc_t, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t off = k * 16 * 128;
          umma_f16_ss(tmem_dP, umma_smem_desc_sw128(ds_base + off, BT * 128, 1024), umma_smem_desc_sw128(q_base + off, BT * 128, 1024),
                      idesc_t, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t a_off = (k / 4) * (BT * 128) + (k % 4) * 32;  // K-major A: 16 key columns per step
          const uint32_t b_off = k * 16 * 128;                          // MN-major B: 16 key rows per step
          umma_f16_ss(tmem_dQ, umma_smem_desc_sw128(ds_base + a_off, 16, 1024), umma_smem_desc_sw128(k_base + b_off, BT * 128, 1024),
                      idesc_q, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&bars[S_KV_EMPTY]);
        umma_commit(&bars[S_MMA2_DONE]);
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutMma, abort_flag);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- one thread per query row
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;        // query row inside the tile; also the key row of the dV / dK tiles it drains
    const int q_local = q0 + r;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const bool is_issuer = warp == 2 && lane == 0;
    const bool row_valid = q_local < doc_len;
    const float g_total = row_valid ? gtot[(long long)head * T + doc_start + q_local] : 0.f;
    const float d_rem = row_valid ? drem[(long long)head * T + doc_start + q_local] : 0.f;
    const float scale_log2 = scale * 1.4426950408889634f;
    float prod = 1.f;   // prod of (1 - sigma) over the keys between the current key and the query
    float g_run = 0.f;  // sum of G over the same keys
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int kv0 = (n_tiles - 1 - j) * BT;
      bool got = mbar_wait(&bars[S_SDP_FULL], j & 1, abort_flag);
      tc_fence_after_sync();
      // the A / dS tiles double as the staging buffer of the previous dK tile: its bulk reduction must have read them
      if (is_issuer) tma_store_wait_read<0>();
      if (named_barrier_or(1, ROW_THREADS, !got)) { ok = false; break; }
#pragma unroll 1
      for (int c = BT / 32 - 1; c >= 0; --c) {
        uint32_t sv[32], dpv[32];
        B200_TMEM_LD_32(sv, tmem_S + lane_addr + c * 32);
        B200_TMEM_LD_32(dpv, tmem_dP + lane_addr + c * 32);
        tmem_ld_wait();
        uint32_t pa[16], pd[16];
#pragma unroll
        for (int e = 30; e >= 0; e -= 2) {
          float av[2], dv[2];
#pragma unroll
          for (int u = 1; u >= 0; --u) {  // the later key first
            const int kv = kv0 + c * 32 + e + u;
            const bool valid = row_valid && kv < q_local;
            const float ez = fast_exp2(fminf(__uint_as_float(sv[e + u]) * scale_log2, 86.f));  // exp(z), z clamped at 60
            const float inv = fast_rcp(1.f + ez);                                             // 1 - sigma
            const float sig = ez * inv;
            const float a = valid ? sig * prod : 0.f;
            const float g = a * (__uint_as_float(dpv[e + u]) - d_rem);
            g_run += g;  // now includes this key
            const float dz = valid ? g * inv - sig * (g_total - g_run) : 0.f;
            if (valid) prod *= inv;
            av[u] = a;
            dv[u] = dz * scale;
          }
          pa[e / 2] = pack_bf16x2(av[0], av[1]);
          pd[e / 2] = pack_bf16x2(dv[0], dv[1]);
        }
        const int kb = c >> 1;
        uint8_t* arow = sA + kb * (BT * 128) + r * 128;
        uint8_t* drow = sDS + kb * (BT * 128) + r * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c & 1) * 4 + ch) ^ (r & 7);
          *reinterpret_cast<uint4*>(arow + chunk * 16) = make_uint4(pa[4 * ch], pa[4 * ch + 1], pa[4 * ch + 2], pa[4 * ch + 3]);
          *reinterpret_cast<uint4*>(drow + chunk * 16) = make_uint4(pd[4 * ch], pd[4 * ch + 1], pd[4 * ch + 2], pd[4 * ch + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[S_PDS_READY]);

      got = mbar_wait(&bars[S_MMA2_DONE], j & 1, abort_flag);
      tc_fence_after_sync();
      // dV tile, then dK tile: TMEM -> fp32 staging (128-byte-swizzled [128 x 32] boxes over the A / dS tiles, which the
      // MMAs have finished with) -> one bulk add per box into the fp32 accumulators of this key / value head.
      // Key rows past the document hold exact zeros (their A and dS columns are 0).
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        if (got) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            B200_TMEM_LD_32(o, (which == 0 ? tmem_S : tmem_dP) + lane_addr + c * 32);
            tmem_ld_wait();
            uint8_t* row = sA + c * (BT * 128) + r * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(row + ((ch ^ (r & 7)) * 16)) = make_uint4(o[4 * ch], o[4 * ch + 1], o[4 * ch + 2], o[4 * ch + 3]);
          }
          if (which == 1) {
            tc_fence_before_sync();
            mbar_arrive(&bars[S_DRAINED]);  // both TMEM tiles have been read: the next S / dP may overwrite them
          }
          fence_proxy_async_smem();
        }
        if (named_barrier_or(2, ROW_THREADS, !got)) { ok = false; break; }
        if (is_issuer) {
          const int row0 = doc_start + kv0;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) tma_reduce_add_2d(which == 0 ? &tm_dv : &tm_dk, sA + c * (BT * 128), grp * D + c * 32, row0);
          tma_store_commit();
          if (which == 0) tma_store_wait_read<0>();  // the dK tile is staged in the same buffer
        }
        if (which == 0 && named_barrier_or(3, ROW_THREADS, false)) { ok = false; break; }
      }
      if (!ok) break;
    }
    if (is_issuer) tma_store_wait<0>();
    if (!ok) {
      raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
    } else {
      // dQ of this query tile (all MMAs retired: the last MMA2_DONE wait above)
      tc_fence_after_sync();
      __nv_bfloat16* qrow = dqkv + (long long)(doc_start + q_local) * dqkv_stride + q_col;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t a[32];
        B200_TMEM_LD_32(a, tmem_dQ + lane_addr + c * 32);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(a[8 * e + 0]), __uint_as_float(a[8 * e + 1]));
            w.y = pack_bf16x2(__uint_as_float(a[8 * e + 2]), __uint_as_float(a[8 * e + 3]));
            w.z = pack_bf16x2(__uint_as_float(a[8 * e + 4]), __uint_as_float(a[8 * e + 5]));
            w.w = pack_bf16x2(__uint_as_float(a[8 * e + 6]), __uint_as_float(a[8 * e + 7]));
            reinterpret_cast<uint4*>(qrow + c * 32)[e] = w;
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

// gtot[h, t] = sum_d dO[t, h, d] * O[t, h, d] - drem[h, t] * (1 - rem[h, t]); one warp per (t, h).
__global__ void sb_gtot_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, const float* __restrict__ drem,
                               const float* __restrict__ rem, float* __restrict__ gtot, int T, int H, int D, long long stride) {
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
  if (lane == 0) {
    const long long at = (long long)h * T + t;
    gtot[at] = s - drem[at] * (1.f - rem[at]);
  }
}

// dqkv[t, k / v columns of every group] = bf16(dk_accum[t, :]), bf16(dv_accum[t, :])
__global__ void sb_dkv_convert_kernel(const float* __restrict__ dk_accum, const float* __restrict__ dv_accum, __nv_bfloat16* __restrict__ dqkv,
                                      long long dqkv_stride, int T, int groups, int qpg, int D) {
  const int per_row = groups * D / 4;
  const long long total = (long long)T * per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_row);
    const int c = (int)(idx - (long long)t * per_row) * 4;  // column inside [groups * D]
    const int grp = c / D, within = c - grp * D;
    const float4 k = reinterpret_cast<const float4*>(dk_accum)[idx];
    const float4 v = reinterpret_cast<const float4*>(dv_accum)[idx];
    __nv_bfloat16* dst = dqkv + (long long)t * dqkv_stride + ((long long)grp * (qpg + 2) + qpg) * D + within;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(k.x, k.y), pack_bf16x2(k.z, k.w));
    *reinterpret_cast<uint2*>(dst + D) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

template <int D>
void launch_sb_bwd(const CUtensorMap& tm_qkv, const CUtensorMap& tm_do, const CUtensorMap& tm_dk, const CUtensorMap& tm_dv, const float* gtot,
                   const float* drem, void* dqkv, long long dqkv_stride, const int* cu_seqlens, int num_docs, int T, int groups, int qpg,
                   float scale, int* status, cudaStream_t stream) {
  auto kernel = sb_attn_bwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SbBwdSmem<D>::TOTAL), "sb_attn_bwd smem attr");
    configured = true;
  }
  const int tiles_upper = (T + BT - 1) / BT + num_docs;
  dim3 grid(groups * qpg, tiles_upper);
  kernel<<<grid, SB_BWD_THREADS, SbBwdSmem<D>::TOTAL, stream>>>(tm_qkv, tm_do, tm_dk, tm_dv, gtot, drem, reinterpret_cast<__nv_bfloat16*>(dqkv),
                                                                dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, status);
  check_cuda(cudaGetLastError(), "sb_attn_bwd launch");
}

}  // namespace

void sb_attn_varlen_bwd(const void* dout, const void* qkv, long long qkv_stride, const void* out, long long out_stride, const float* rem,
                        const float* drem, float* gtot, float* dk_accum, float* dv_accum, void* dqkv, long long dqkv_stride,
                        const int* cu_seqlens, int num_docs, int T, int groups, int qpg, int head_dim, float scale, int* status,
                        cudaStream_t stream) {
  if (T == 0 || num_docs == 0) return;
  const int hq = groups * qpg;
  const long long width = (long long)groups * (qpg + 2) * head_dim;
  {
    const long long warps = (long long)T * hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    sb_gtot_kernel<<<(unsigned)blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(out),
                                                             drem, rem, gtot, T, hq, head_dim, out_stride);
  }
  const size_t accum_bytes = (size_t)T * groups * head_dim * sizeof(float);
  check_cuda(cudaMemsetAsync(dk_accum, 0, accum_bytes, stream), "dk_accum memset");
  check_cuda(cudaMemsetAsync(dv_accum, 0, accum_bytes, stream), "dv_accum memset");
  const CUtensorMap tm_qkv = make_tensor_map_2d_b16(qkv, width, T, qkv_stride, 64, BT);
  const CUtensorMap tm_do = make_tensor_map_2d_b16(dout, (long long)hq * head_dim, T, out_stride, 64, BT);
  const CUtensorMap tm_dk = make_tensor_map_2d_f32(dk_accum, (long long)groups * head_dim, T, (long long)groups * head_dim, 32, BT);
  const CUtensorMap tm_dv = make_tensor_map_2d_f32(dv_accum, (long long)groups * head_dim, T, (long long)groups * head_dim, 32, BT);
  if (head_dim == 128) launch_sb_bwd<128>(tm_qkv, tm_do, tm_dk, tm_dv, gtot, drem, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, status, stream);
  else if (head_dim == 64) launch_sb_bwd<64>(tm_qkv, tm_do, tm_dk, tm_dv, gtot, drem, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, status, stream);
  else throw std::runtime_error("sb_attn_varlen_bwd: head_dim must be 64 or 128");
  {
    const long long total = (long long)T * groups * head_dim / 4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    sb_dkv_convert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dk_accum, dv_accum, reinterpret_cast<__nv_bfloat16*>(dqkv), dqkv_stride, T, groups,
                                                               qpg, head_dim);
  }
  count_launch(4);
  check_cuda(cudaGetLastError(), "sb_attn_bwd tail launch");
}

}  // namespace b200

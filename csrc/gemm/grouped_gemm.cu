// Grouped bf16 GEMMs for mixture-of-experts layers (tcgen05, TMA, TMEM; one CTA per SM, persistent).
//
// Token rows are stored grouped by expert in one buffer whose per-expert ranges start at multiples of 128 rows and
// are zero-padded up to the next multiple (see lm_engine/ops/moe.py). Every 128-row tile therefore belongs to
// exactly one expert, listed in `tile_expert`; tiles past the last used one carry an id >= num_experts and are
// skipped by all warp roles alike. No host synchronisation is needed to size the launch: the grid is persistent
// and the tile table has a fixed upper-bound length.
//
//   grouped_rows : C[rows, N] = A[rows, K] * op(W[expert(row)])      forward (W K-major) and data gradient (W MN-major)
//   grouped_wgrad: dW[e][N, K] (+)= sum over rows of expert e of dY[row, N]^T X[row, K]     (both operands MN-major)
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 + 256;

struct Smem {
  uint8_t* sA;
  uint8_t* sB;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* acc_full;
  uint64_t* acc_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

__device__ __forceinline__ Smem carve(uint8_t* raw) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  Smem s;
  s.sA = smem;
  s.sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  s.full = bars;
  s.empty = bars + STAGES;
  s.acc_full = bars + 2 * STAGES;
  s.acc_empty = bars + 2 * STAGES + 2;
  s.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
  return s;
}

__device__ __forceinline__ void init_common(const Smem& s, int warp) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s.acc_full[b], 1);
      mbar_init(&s.acc_empty[b], 4);
    }
    *s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
}

// Writes one 128 x 256 fp32 accumulator (this thread's row) to global memory.
template <bool F32_OUT, bool ACCUMULATE>
__device__ __forceinline__ void store_row(uint32_t t_row, void* Cv, long long row_offset, int n0, int N, bool row_valid) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    const int col0 = n0 + c * 32;
    if (col0 >= N) break;
    uint32_t v[32];
    B200_TMEM_LD_32(v, t_row + c * 32);
    tmem_ld_wait();
    if (!row_valid) continue;
    if (F32_OUT) {
      float* dst = reinterpret_cast<float*>(Cv) + row_offset + col0;
      if (col0 + 32 <= N) {
        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
          if (ACCUMULATE) {
            const float4 old = d4[j];
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          d4[j] = o;
        }
      } else {
        for (int e = 0; e < 32 && col0 + e < N; ++e) dst[e] = __uint_as_float(v[e]) + (ACCUMULATE ? dst[e] : 0.f);
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + row_offset + col0;
      if (col0 + 32 <= N) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          d4[j] = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
        }
      } else {
        for (int e = 0; e < 32 && col0 + e < N; ++e) dst[e] = __float2bfloat16(__uint_as_float(v[e]));
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------------------------
// C[rows, N] = A[rows, K] * op(W[expert])
// With DISPATCH the A rows do not exist yet when the kernel starts: the first `copy_ctas` CTAs gather them, 128-row tile by
// tile, from the token buffers of all ranks (peer pointers; bulk copies peer -> shared-memory ring -> this GPU's A buffer)
// and publish one ready flag per tile; the GEMM CTAs visit the tiles in the same order and wait for the flag of a tile
// before their first TMA load of it, so the transfer of tile t + 1 runs under the MMAs of tile t. All CTAs are resident
// (one per SM), every wait is bounded.
struct DispatchArgs {
  const void* src[16];     // per rank: [tokens, K] bf16 token rows
  const int* src_entry;    // per row: global entry (rank * entries_per_rank + token * k + slot) or -1 for a padding row
  void* a_rows;            // [max_m_tiles * 128, K] bf16: the gathered rows (kept by the caller for the weight gradient)
  int* ready;              // one flag per tile, zero at launch
  int entries_per_rank, k, copy_ctas, epoch;
};

constexpr uint32_t kReadySpinLimit = 1u << 24;  // x ~100 ns sleep: a couple of seconds
constexpr int RING_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);

__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void bulk_store_row(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

// One warp of a gather CTA. Lane l owns two row slots of the shared-memory ring and its own mbarriers, and runs its own
// two-deep pipeline over the rows l, l + rb, l + 2 rb, ... of every tile this CTA gathers: the load of its next row is in
// flight while the current one is stored, so about 2 * rb rows per CTA are in flight at any time.
__device__ void gather_tiles(uint8_t* ring, volatile int* abort_flag, const DispatchArgs& da, const int* tile_expert, int max_m_tiles,
                             int num_experts, int K, int* status) {
  const int lane = threadIdx.x & 31;
  const uint32_t row_bytes = (uint32_t)K * 2;
  const int rb = min(32, (int)((RING_BYTES - row_bytes - 512) / 2 / row_bytes));  // lanes that take rows
  uint8_t* zero = ring + (size_t)2 * rb * row_bytes;  // one row of zeros: the source of the padding rows
  uint64_t* bars = reinterpret_cast<uint64_t*>(zero + row_bytes);  // [2][rb]
  const bool active = lane < rb;
  if (active) {
    mbar_init(&bars[lane], 1);
    mbar_init(&bars[rb + lane], 1);
  }
  if (lane == 0) *abort_flag = 0;
  fence_barrier_init();
  for (uint32_t i = lane * 16; i < row_bytes; i += 32 * 16) *reinterpret_cast<uint4*>(zero + i) = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  __syncwarp();
  uint32_t parity[2] = {0, 0};
  uint32_t slot = 0;     // slot of the row whose load is in flight (or that is a padding row)
  bool ok = true;
  const int per_lane = (BM - lane + rb - 1) / rb;  // rows of a tile that fall to this lane

  // first used tile at or after `mt` in this CTA's sequence (max_m_tiles if none)
  auto next_tile = [&](int mt) -> int {
    for (; mt < max_m_tiles; mt += da.copy_ctas) {
      const int te = tile_expert[mt];
      if (te >= 0 && te < num_experts) break;
    }
    return mt;
  };
  // start the load of row (mt, r) into `s`; returns the entry (-1: padding row, nothing to load)
  auto start_row = [&](int mt, int r, uint32_t s) -> int {
    const int e = da.src_entry[mt * BM + r];
    if (e >= 0) {
      tma_store_wait_read<0>();  // the store that last used this slot (the previous row of this lane) has left shared memory
      const int rank = e / da.entries_per_rank;
      const int token = (e - rank * da.entries_per_rank) / da.k;
      uint64_t* bar = &bars[s * rb + lane];
      mbar_arrive_expect_tx(bar, row_bytes);
      bulk_load_row(ring + (size_t)(s * rb + lane) * row_bytes, reinterpret_cast<const uint8_t*>(da.src[rank]) + (size_t)token * row_bytes, row_bytes, bar);
    }
    return e;
  };

  int mt = next_tile(blockIdx.x);
  int e_cur = -1;
  if (mt < max_m_tiles && active) e_cur = start_row(mt, lane, slot);
  while (mt < max_m_tiles) {
    const int mt_next = next_tile(mt + da.copy_ctas);
    uint8_t* dst_tile = reinterpret_cast<uint8_t*>(da.a_rows) + (size_t)mt * BM * row_bytes;
    if (active) {
      for (int jrow = 0; jrow < per_lane; ++jrow) {
        const int r = lane + jrow * rb;
        // the next row of this lane: in this tile, or the first one of the next tile
        int e_next = -1;
        const bool more = jrow + 1 < per_lane;
        if (more) e_next = start_row(mt, r + rb, slot ^ 1);
        else if (mt_next < max_m_tiles) e_next = start_row(mt_next, lane, slot ^ 1);
        if (e_cur >= 0) {
          if (ok && !mbar_wait(&bars[slot * rb + lane], parity[slot], abort_flag)) ok = false;
          parity[slot] ^= 1;
        }
        if (ok) bulk_store_row(dst_tile + (size_t)r * row_bytes, e_cur >= 0 ? ring + (size_t)(slot * rb + lane) * row_bytes : zero, row_bytes);
        tma_store_commit();
        e_cur = e_next;
        slot ^= 1;
      }
      tma_store_wait<0>();  // this lane's rows of the tile are in this GPU's memory (its next load stays in flight)
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    if (lane == 0) {
      __threadfence();
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(da.ready + mt), "r"(da.epoch) : "memory");
    }
    mt = mt_next;
  }
  if (!ok) {
    if (lane == 0) raise_status(status, kStatusWaitTimeoutPeer, abort_flag);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // bounded grace for copies still in flight
    tma_store_wait<0>();
  }
}

template <int B_MN, bool DISPATCH>
__global__ void __launch_bounds__(THREADS, 1)
    grouped_rows_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        __nv_bfloat16* __restrict__ C, const int* __restrict__ tile_expert, int max_m_tiles,
                        int num_experts, int N, int K, long long ldc, int* status, const __grid_constant__ DispatchArgs da) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int copy_ctas = DISPATCH ? da.copy_ctas : 0;
  if (DISPATCH && (int)blockIdx.x < copy_ctas) {
    if (warp == 0) gather_tiles(s.sA, s.abort_flag, da, tile_expert, max_m_tiles, num_experts, K, status);
    return;
  }
  init_common(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int n_tiles = (N + BN - 1) / BN;
  const int k_blocks = (K + BK - 1) / BK;
  const int total = max_m_tiles * n_tiles;
  const int first_tile = (int)blockIdx.x - copy_ctas, tile_step = (int)gridDim.x - copy_ctas;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_mt = -1;
      for (int tile = first_tile; tile < total && ok; tile += tile_step) {
        const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
        const int e = tile_expert[mt];
        if (e < 0 || e >= num_experts) continue;
        if (DISPATCH && mt != ready_mt) {
          // the rows of this tile are being gathered by another CTA: wait for its flag, bounded
          uint32_t spins = 0;
          int seen;
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(da.ready + mt) : "memory");
            if (seen == da.epoch) break;
            __nanosleep(100);
          } while (++spins < kReadySpinLimit && !*s.abort_flag);
          if (seen != da.epoch) {
            raise_status(status, kStatusWaitTimeoutPeer, s.abort_flag);
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // the TMA loads below must see the rows written by bulk copies
          ready_mt = mt;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, s.abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, s.abort_flag);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.full[st], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(s.sA + st * A_STAGE_BYTES, &tmA, &s.full[st], kb * BK, mt * BM);
          uint8_t* b_dst = s.sB + st * B_STAGE_BYTES;
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * (BK * 128), &tmB, &s.full[st], nt * BN + j * 64, kb * BK, e);
          } else {
            tma_load_3d(b_dst, &tmB, &s.full[st], kb * BK, nt * BN, e);
          }
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, B_MN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step) {
        const int mt = tile / n_tiles;
        const int e = tile_expert[mt];
        if (e < 0 || e >= num_experts) continue;
        const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait(&s.acc_empty[buf], aph ^ 1, s.abort_flag)) {
          raise_status(status, kStatusWaitTimeoutMma, s.abort_flag);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.full[st], ph, s.abort_flag)) {
            raise_status(status, kStatusWaitTimeoutMma, s.abort_flag);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(s.sA + st * A_STAGE_BYTES), b_base = smem_u32(s.sB + st * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(b_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&s.empty[st]);
        }
        if (ok) umma_commit(&s.acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    uint32_t tcount = 0;
    for (int tile = first_tile; tile < total; tile += tile_step) {
      const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
      const int e = tile_expert[mt];
      if (e < 0 || e >= num_experts) continue;
      const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&s.acc_full[buf], aph, s.abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, s.abort_flag);
        break;
      }
      tc_fence_after_sync();
      const long long row = (long long)mt * BM + q * 32 + lane;
      store_row<false, false>(tmem_base + (uint32_t(q * 32) << 16) + buf * BN, C, row * ldc, nt * BN, N, true);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------------------------------------
// dW[e][Nw, Kw] (+)= dY[rows_e, Nw]^T X[rows_e, Kw]; rows_e = [padded_offsets[e], padded_offsets[e + 1])
template <bool ACCUMULATE>
__global__ void __launch_bounds__(THREADS, 1)
    grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmDY, const __grid_constant__ CUtensorMap tmX,
                         float* __restrict__ dW, const int* __restrict__ padded_offsets, int num_experts, int Nw, int Kw,
                         int* status) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  init_common(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int m_tiles = (Nw + BM - 1) / BM;   // output rows  = weight rows (out features)
  const int n_tiles = (Kw + BN - 1) / BN;   // output cols  = weight cols (in features)
  const int per_expert = m_tiles * n_tiles;
  const int total = num_experts * per_expert;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int e = tile / per_expert, r = tile - e * per_expert;
        const int mt = r / n_tiles, nt = r - mt * n_tiles;
        const int row0 = padded_offsets[e], row1 = padded_offsets[e + 1];
        for (int row = row0; row < row1; row += BK, ++it) {
          const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, s.abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, s.abort_flag);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.full[st], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = s.sA + st * A_STAGE_BYTES;
          uint8_t* b_dst = s.sB + st * B_STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmDY, &s.full[st], mt * BM + j * 64, row);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmX, &s.full[st], nt * BN + j * 64, row);
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 1, 1);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int e = tile / per_expert;
        const int row0 = padded_offsets[e], row1 = padded_offsets[e + 1];
        if (row1 <= row0) continue;
        const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait(&s.acc_empty[buf], aph ^ 1, s.abort_flag)) {
          raise_status(status, kStatusWaitTimeoutMma, s.abort_flag);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool first = true;
        for (int row = row0; row < row1; row += BK, ++it) {
          const uint32_t st = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(&s.full[st], ph, s.abort_flag)) {
            raise_status(status, kStatusWaitTimeoutMma, s.abort_flag);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(s.sA + st * A_STAGE_BYTES), b_base = smem_u32(s.sB + st * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16_ss(d_tmem, umma_smem_desc_sw128(a_base + k * 16 * 128, BK * 128, 1024),
                        umma_smem_desc_sw128(b_base + k * 16 * 128, BK * 128, 1024), idesc, (first && k == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit(&s.empty[st]);
        }
        if (ok) umma_commit(&s.acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const int e = tile / per_expert, r = tile - e * per_expert;
      const int mt = r / n_tiles, nt = r - mt * n_tiles;
      if (padded_offsets[e + 1] <= padded_offsets[e]) continue;
      const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&s.acc_full[buf], aph, s.abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, s.abort_flag);
        break;
      }
      tc_fence_after_sync();
      const int wrow = mt * BM + q * 32 + lane;
      store_row<true, ACCUMULATE>(tmem_base + (uint32_t(q * 32) << 16) + buf * BN, dW,
                                  ((long long)e * Nw + wrow) * Kw, nt * BN, Kw, wrow < Nw);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename KernelT>
void configure(KernelT kernel) {
  check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "grouped gemm smem attr");
}

}  // namespace

// A: grouped rows [max_m_tiles * 128, K] bf16 contiguous (row stride lda). W: [E, N, K] (w_mn = false, forward) or
// [E, K, N] read as the MN-major operand (w_mn = true: C = A * W[e] with W[e] of shape [K, N]). C: [rows, N] bf16.
void grouped_rows_gemm(const void* A, long long lda, const void* W, void* C, long long ldc, const int* tile_expert,
                       int max_m_tiles, int num_experts, int N, int K, bool w_mn, int* status, cudaStream_t stream) {
  if (max_m_tiles <= 0 || N <= 0 || K <= 0) return;
  const CUtensorMap tmA = make_tensor_map_2d_b16(A, K, (uint64_t)max_m_tiles * BM, lda, BK, BM);
  const int total = max_m_tiles * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (total < grid) grid = total;
  if (w_mn) {
    // W[e] is [K, N] row-major: N contiguous -> MN-major B operand
    const CUtensorMap tmB = make_tensor_map_3d_b16(W, N, K, num_experts, N, (uint64_t)N * K, 64, BK, 1);
    static bool once = (configure(grouped_rows_kernel<1, false>), true);
    (void)once;
    grouped_rows_kernel<1, false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), tile_expert,
                                                                         max_m_tiles, num_experts, N, K, ldc, status, DispatchArgs{});
  } else {
    const CUtensorMap tmB = make_tensor_map_3d_b16(W, K, N, num_experts, K, (uint64_t)N * K, BK, BN, 1);
    static bool once = (configure(grouped_rows_kernel<0, false>), true);
    (void)once;
    grouped_rows_kernel<0, false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), tile_expert,
                                                                         max_m_tiles, num_experts, N, K, ldc, status, DispatchArgs{});
  }
  count_launch();
  check_cuda(cudaGetLastError(), "grouped_rows_gemm launch");
}

// The same product with the A rows gathered inside the kernel (see DispatchArgs): `src_ptrs[r]` is rank r's [tokens, K]
// bf16 token buffer (this GPU's own buffer or a peer mapping), `src_entry` names the (rank, token) of every row, `a_rows`
// receives the gathered rows, `ready` is an int32 buffer of max_m_tiles zeros.
void grouped_rows_dispatch_gemm(const void* const* src_ptrs, int num_ranks, const int* src_entry, int entries_per_rank, int k, void* a_rows,
                                int* ready, int copy_ctas, const void* W, void* C, long long ldc, const int* tile_expert, int max_m_tiles,
                                int num_experts, int N, int K, bool w_mn, int* status, cudaStream_t stream) {
  if (max_m_tiles <= 0 || N <= 0 || K <= 0) return;
  if (num_ranks < 1 || num_ranks > 16) throw std::runtime_error("grouped_rows_dispatch: between 1 and 16 source buffers");
  if ((K * 2) % 16 != 0 || K * 2 > 16384) throw std::runtime_error("grouped_rows_dispatch: row size must be a multiple of 16 bytes, at most 16 KB");
  const CUtensorMap tmA = make_tensor_map_2d_b16(a_rows, K, (uint64_t)max_m_tiles * BM, K, BK, BM);
  const int total = max_m_tiles * ((N + BN - 1) / BN);
  const int sms = sm_count();
  if (copy_ctas < 1) copy_ctas = 1;
  if (copy_ctas > sms / 2) copy_ctas = sms / 2;
  int grid = sms;  // every CTA must be resident: gather and GEMM CTAs wait on one another
  if (total + copy_ctas < grid) grid = total + copy_ctas;
  DispatchArgs da = {};
  for (int r = 0; r < num_ranks; ++r) da.src[r] = src_ptrs[r];
  da.src_entry = src_entry;
  da.a_rows = a_rows;
  da.ready = ready;
  da.entries_per_rank = entries_per_rank;
  da.k = k;
  da.copy_ctas = copy_ctas;
  da.epoch = 1;
  if (w_mn) {
    const CUtensorMap tmB = make_tensor_map_3d_b16(W, N, K, num_experts, N, (uint64_t)N * K, 64, BK, 1);
    static bool once = (configure(grouped_rows_kernel<1, true>), true);
    (void)once;
    grouped_rows_kernel<1, true><<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), tile_expert,
                                                                        max_m_tiles, num_experts, N, K, ldc, status, da);
  } else {
    const CUtensorMap tmB = make_tensor_map_3d_b16(W, K, N, num_experts, K, (uint64_t)N * K, BK, BN, 1);
    static bool once = (configure(grouped_rows_kernel<0, true>), true);
    (void)once;
    grouped_rows_kernel<0, true><<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), tile_expert,
                                                                        max_m_tiles, num_experts, N, K, ldc, status, da);
  }
  count_launch();
  check_cuda(cudaGetLastError(), "grouped_rows_dispatch_gemm launch");
}

// dY: [rows, Nw] bf16, X: [rows, Kw] bf16 (both contiguous grouped buffers), dW: [E, Nw, Kw] fp32.
void grouped_wgrad_gemm(const void* dY, const void* X, float* dW, const int* padded_offsets, long long total_rows,
                        int num_experts, int Nw, int Kw, bool accumulate, int* status, cudaStream_t stream) {
  if (total_rows <= 0) return;
  const CUtensorMap tmDY = make_tensor_map_2d_b16(dY, Nw, total_rows, Nw, 64, BK);
  const CUtensorMap tmX = make_tensor_map_2d_b16(X, Kw, total_rows, Kw, 64, BK);
  const int total = num_experts * ((Nw + BM - 1) / BM) * ((Kw + BN - 1) / BN);
  int grid = sm_count();
  if (total < grid) grid = total;
  if (accumulate) {
    static bool once = (configure(grouped_wgrad_kernel<true>), true);
    (void)once;
    grouped_wgrad_kernel<true><<<grid, THREADS, SMEM_BYTES, stream>>>(tmDY, tmX, dW, padded_offsets, num_experts, Nw, Kw, status);
  } else {
    static bool once = (configure(grouped_wgrad_kernel<false>), true);
    (void)once;
    grouped_wgrad_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmDY, tmX, dW, padded_offsets, num_experts, Nw, Kw, status);
  }
  count_launch();
  check_cuda(cudaGetLastError(), "grouped_wgrad_gemm launch");
}

}  // namespace b200

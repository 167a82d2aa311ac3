// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster compute one 256 x 256 output tile.
//
// Each CTA stages its own 128 rows of A and its own 128 of the 256 B rows per k-block (32 KB per stage instead of
// 48 KB for the single-CTA kernel, 6 stages) and keeps its 128 x 256 half of the accumulator in its own TMEM; the
// tensor cores of both SMs read both B halves, so every byte of B is fetched from L2 once per pair and the
// operand traffic per FLOP drops by a third. No multicast load is involved: every CTA loads only what it stores.
//
// Roles per CTA: warp 0 = TMA producer (both CTAs), warp 1 = MMA issuer (only in the even CTA of the pair, the
// "leader"), warps 2..5 = epilogue of the CTA's own accumulator half. Synchronisation across the pair:
//   full[s]      lives in the leader; the leader's producer arms it with the byte count of BOTH CTAs, both producers'
//                copies complete on it (cta_group::2 copies may signal the peer's barrier)
//   empty[s]     one per CTA; the leader's MMA thread commits to its own and to the peer's (two plain commits)
//   acc_full[b]  same pattern as empty
//   acc_empty[b] lives in the leader, 8 arrivals: the four epilogue warps of each CTA (the peer's arrive remotely)
// All mbarrier waits are bounded; cluster-wide barriers bracket the kernel so that neither CTA touches the other's
// shared memory before it is initialised or after it has exited.
//
// Epilogue: every epilogue warp owns 32 accumulator rows. It converts 128-byte row segments (64 bf16 / 32 fp32
// columns) into a swizzled 4 KB shared-memory box and hands the box to the TMA engine: a bulk tensor store, or a bulk
// tensor reduction (`.add`) for the accumulating variants, so that the read-modify-write of a weight-gradient tile
// happens in L2 and never travels to the SM. Two boxes per warp alternate, the store of one overlaps the conversion
// of the next. Outputs that a tensor map cannot describe (unaligned base / row stride) take the register -> global path.
//
// SwiGLU epilogue (forward of the gated MLP up-projection): the weight is [2I, K] with rows [0, I) = up and
// [I, 2I) = gate. The even CTA of a pair loads 128 up rows and the odd CTA the 128 gate rows of the same channels, so
// accumulator columns [0,128) and [128,256) of one tile hold up and gate of the same 128 channels; the epilogue
// writes both halves of the projection (backward needs them) and up * silu(gate), computed from the bf16-rounded
// values exactly as the stand-alone kernel does, without the projection making a round trip through HBM.
//
// SwiGLU-backward epilogue (data gradient of the gated MLP's down-projection): the accumulator is d(act) = dy W; the
// epilogue reads up and gate of the same rows and channels from the saved projection (plain 16-byte loads requested
// 32 columns ahead of the arithmetic) and writes d(up) = d(act) * silu(gate), d(gate) = d(act) * up * silu'(gate) and
// the recomputed act = up * silu(gate) (the weight gradient of the down-projection needs it), so d(act) never exists in
// memory. d(act) is rounded to bf16 first, which makes the three outputs bit-identical to GEMM + stand-alone kernel.
#include <cuda.h>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "../ops/ops.h"

namespace b200 {

namespace {

constexpr int BM = 128;       // rows per CTA (256 per pair)
constexpr int BN = 256;       // columns per pair
constexpr int BN_HALF = 128;  // B rows staged per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN_HALF * BK * 2;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int BOX_BYTES = 32 * 128;            // one epilogue box: 32 rows x 128 bytes
constexpr int STAGING_BYTES = 4 * 2 * BOX_BYTES;  // two boxes for each of the four epilogue warps
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + STAGING_BYTES + 1024 + 256;
constexpr int TRACE_WORDS = 8;

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ACC = 3, EPI_SWIGLU = 4, EPI_SWIGLU_BWD = 5 };

struct KernelOpts {
  int group;        // > 0: panels of `group` 256-row tiles, rows fastest; < 0: panels of -group 256-column tiles, columns fastest
  int tma_store;    // epilogue leaves through shared memory and bulk tensor stores / reductions
  int k_skew;       // k-block at which tile (i, j) starts its walk over K is (i + j) * k_skew mod k_blocks
  int swiglu_i;     // EPI_SWIGLU: intermediate size I (N == 2 I); EPI_SWIGLU_BWD: I == N
  const __nv_bfloat16* fc;  // EPI_SWIGLU_BWD: the saved projection [M, 2 I] = [up | gate]
  long long ldfc;   // its row stride in elements
  int split_k;      // >= 1; > 1 only with the bulk-reduction epilogues: each tile is computed as that many partial sums over K
  long long* trace; // TRACE builds: TRACE_WORDS cycle counters per CTA
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `local` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local), "r"(rank));
  return out;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void tmem_alloc_2sm(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Copy into this CTA's shared memory; completion bytes are credited to the barrier at `bar_cluster_addr`, which may
// belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* desc, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void umma_f16_ss_2sm(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on the barrier at a shared::cluster address once all MMAs issued so far by this thread have retired.
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ float silu_f(float x) { return silu_fast(x); }

struct TileCoord {
  int mi, ni;  // tile indices (256-row, 256-column units)
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles, int group) {
  if (group > 0) {
    const int per_group = group * n_tiles;
    const int g = tile / per_group;
    const int first = g * group;
    const int gsize = min(m_tiles - first, group);
    const int r = tile - g * per_group;
    return {first + r % gsize, r / gsize};
  }
  group = -group;
  const int per_group = group * m_tiles;
  const int g = tile / per_group;
  const int first = g * group;
  const int gsize = min(n_tiles - first, group);
  const int r = tile - g * per_group;
  return {r / gsize, first + r % gsize};
}

// Row `lane` of a swizzled 32 x 128-byte box: 16-byte chunk `c` of the row lands at chunk `c ^ (lane & 7)`.
__device__ __forceinline__ void box_write(uint8_t* box, int lane, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(box + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = v;
}

template <int A_MN, int B_MN, int EPI, bool TRACE>
__global__ void __launch_bounds__(THREADS, 1)
    gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmC2,
                         void* __restrict__ Cv, int M, int N, int K, long long ldc, float alpha, int* status, KernelOpts opts) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sStage = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + STAGING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = (N + BN - 1) / BN;
  const int k_blocks = (K + BK - 1) / BK;
  const int split = opts.split_k;
  const int total = m_tiles * n_tiles * split;  // work units: (tile, k range)
  long long* trace = TRACE ? opts.trace + (long long)blockIdx.x * TRACE_WORDS : nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything remote touches them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      long long waited = 0;
      for (int unit = pair; unit < total && ok; unit += num_pairs) {
        const TileCoord tc = tile_coord(unit / split, m_tiles, n_tiles, opts.group);
        const int kb_begin = (int)((long long)(unit % split) * k_blocks / split);
        const int kb_end = (int)((long long)(unit % split + 1) * k_blocks / split);
        const int m0 = tc.mi * (2 * BM) + (int)cta_rank * BM;
        const int n0 = EPI == EPI_SWIGLU ? tc.ni * BN_HALF + (int)cta_rank * opts.swiglu_i : tc.ni * BN + (int)cta_rank * BN_HALF;
        const int k_len = kb_end - kb_begin;
        int kk = kb_begin + (opts.k_skew && k_len > 0 ? (int)(((long long)(tc.mi + tc.ni) * opts.k_skew) % k_len) : 0);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          const long long t0 = TRACE ? clock64() : 0;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
            ok = false;
            break;
          }
          if (TRACE) waited += clock64() - t0;
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), &tmA, full_leader, m0 + j * 64, kk * BK);
          } else {
            tma_load_2d_pair(a_dst, &tmA, full_leader, kk * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_pair(b_dst + j * (BK * 128), &tmB, full_leader, n0 + j * 64, kk * BK);
          } else {
            tma_load_2d_pair(b_dst, &tmB, full_leader, kk * BK, n0);
          }
          if (++kk == kb_end) kk = kb_begin;
        }
      }
      if (TRACE) trace[0] = waited;
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = TRACE ? clock64() : 0;
      for (int unit = pair; unit < total && ok; unit += num_pairs, ++tcount) {
        const int kb_begin = (int)((long long)(unit % split) * k_blocks / split);
        const int kb_end = (int)((long long)(unit % split + 1) * k_blocks / split);
        const uint32_t buf = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        long long t0 = TRACE ? clock64() : 0;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutMma, abort_flag);
          break;
        }
        if (TRACE) wait_acc += clock64() - t0;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          t0 = TRACE ? clock64() : 0;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutMma, abort_flag);
            ok = false;
            break;
          }
          if (TRACE) wait_full += clock64() - t0;
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(a_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(b_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss_2sm(d_tmem, da, db, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
          }
          // release the stage in both CTAs
          const uint32_t e_local = smem_u32(&empty[s]);
          umma_commit_2sm(map_to_cta(e_local, 0));
          umma_commit_2sm(map_to_cta(e_local, 1));
        }
        if (ok) {
          const uint32_t f_local = smem_u32(&acc_full[buf]);
          umma_commit_2sm(map_to_cta(f_local, 0));
          umma_commit_2sm(map_to_cta(f_local, 1));
        }
      }
      if (TRACE) {
        trace[1] = wait_full;
        trace[2] = wait_acc;
        trace[3] = clock64() - t_begin;
        trace[6] = tcount;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue: this CTA's 128 x 256 half
    const int q = warp & 3;
    uint8_t* stage0 = sStage + q * (2 * BOX_BYTES);
    uint32_t tcount = 0, nstore = 0;
    long long wait_acc = 0, wait_store = 0;
    const long long t_begin = TRACE ? clock64() : 0;
    for (int unit = pair; unit < total; unit += num_pairs, ++tcount) {
      const TileCoord tc = tile_coord(unit / split, m_tiles, n_tiles, opts.group);
      const uint32_t buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      long long t0 = TRACE ? clock64() : 0;
      if (!mbar_wait(&acc_full[buf], aph, abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
        break;
      }
      if (TRACE) wait_acc += clock64() - t0;
      tc_fence_after_sync();
      const int row0 = tc.mi * (2 * BM) + (int)cta_rank * BM + q * 32;
      const int row = row0 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;

      if (EPI == EPI_SWIGLU) {
        // accumulator columns [0,128) = up, [128,256) = gate of channels [ni*128, ni*128 + 128)
        const int ch0 = tc.ni * BN_HALF;
        uint8_t* box_u = stage0;
        uint8_t* box_g = stage0 + BOX_BYTES;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          const int ch = ch0 + c * 64;
          if (ch >= opts.swiglu_i) break;
          uint32_t actp[32];
          if (TRACE) t0 = clock64();
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          if (TRACE) wait_store += clock64() - t0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t vu[32], vg[32];
            B200_TMEM_LD_32(vu, t_row + c * 64 + half * 32);
            B200_TMEM_LD_32(vg, t_row + BN_HALF + c * 64 + half * 32);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t pu[4], pg[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                pu[e] = pack_bf16x2(__uint_as_float(vu[8 * j + 2 * e]) * alpha, __uint_as_float(vu[8 * j + 2 * e + 1]) * alpha);
                pg[e] = pack_bf16x2(__uint_as_float(vg[8 * j + 2 * e]) * alpha, __uint_as_float(vg[8 * j + 2 * e + 1]) * alpha);
                const float2 u = unpack_bf16x2(pu[e]), g = unpack_bf16x2(pg[e]);
                actp[half * 16 + j * 4 + e] = pack_bf16x2(u.x * silu_f(g.x), u.y * silu_f(g.y));
              }
              box_write(box_u, lane, half * 4 + j, make_uint4(pu[0], pu[1], pu[2], pu[3]));
              box_write(box_g, lane, half * 4 + j, make_uint4(pg[0], pg[1], pg[2], pg[3]));
            }
          }
          if (c == 1 || ch + 64 >= opts.swiglu_i) {
            // last read of this accumulator: hand the TMEM buffer back before the stores drain
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < M) {
            tma_store_2d(&tmC, box_u, ch, row0);
            tma_store_2d(&tmC, box_g, opts.swiglu_i + ch, row0);
            tma_store_commit();
            tma_store_wait_read<0>();
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) box_write(box_u, lane, j, make_uint4(actp[4 * j], actp[4 * j + 1], actp[4 * j + 2], actp[4 * j + 3]));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < M) {
            tma_store_2d(&tmC2, box_u, ch, row0);
            tma_store_commit();
          }
        }
        continue;
      }

      if (EPI == EPI_SWIGLU_BWD) {
        const int I = opts.swiglu_i;
        uint8_t* box_a = stage0;
        uint8_t* box_b = stage0 + BOX_BYTES;
        const int tile_col0 = tc.ni * BN;
        const int halves = min(BN, I - tile_col0) / 32;  // 32-column halves of this tile (I % 64 == 0: an even number)
        // rows past M read the last row instead (their results never leave: the bulk stores clip at M)
        const __nv_bfloat16* fc_row = opts.fc + (long long)min(row, M - 1) * opts.ldfc + tile_col0;
        // up / gate of the NEXT 32 columns are requested before the current ones are worked on, so that their trip from
        // L2 or HBM is covered by about a thousand instructions of arithmetic
        uint4 un[4], gn[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          un[j] = __ldg(reinterpret_cast<const uint4*>(fc_row) + j);
          gn[j] = __ldg(reinterpret_cast<const uint4*>(fc_row + I) + j);
        }
#pragma unroll 1
        for (int c = 0; c < halves / 2; ++c) {
          const int col0 = tile_col0 + c * 64;
          uint32_t yp[32];
          if (TRACE) t0 = clock64();
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          if (TRACE) wait_store += clock64() - t0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int h = 2 * c + half;
            uint32_t v[32];
            B200_TMEM_LD_32(v, t_row + h * 32);
            uint4 u4[4], g4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              u4[j] = un[j];
              g4[j] = gn[j];
            }
            if (h + 1 < halves) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                un[j] = __ldg(reinterpret_cast<const uint4*>(fc_row + (h + 1) * 32) + j);
                gn[j] = __ldg(reinterpret_cast<const uint4*>(fc_row + I + (h + 1) * 32) + j);
              }
            }
            tmem_ld_wait();
            if (h + 1 == halves) {
              // last read of this accumulator: hand the TMEM buffer back before the arithmetic and the stores
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t uu[4] = {u4[j].x, u4[j].y, u4[j].z, u4[j].w}, gg[4] = {g4[j].x, g4[j].y, g4[j].z, g4[j].w};
              uint32_t du[4], dg[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 a = unpack_bf16x2(uu[e]), b = unpack_bf16x2(gg[e]);
                const float2 q = unpack_bf16x2(pack_bf16x2(__uint_as_float(v[8 * j + 2 * e]) * alpha, __uint_as_float(v[8 * j + 2 * e + 1]) * alpha));
                const float s0 = sigmoid_fast(b.x), s1 = sigmoid_fast(b.y);
                const float act0 = b.x * s0, act1 = b.y * s1;
                const float dact0 = s0 * (1.f + b.x * (1.f - s0)), dact1 = s1 * (1.f + b.y * (1.f - s1));
                du[e] = pack_bf16x2(q.x * act0, q.y * act1);
                dg[e] = pack_bf16x2(q.x * a.x * dact0, q.y * a.y * dact1);
                yp[half * 16 + j * 4 + e] = pack_bf16x2(a.x * act0, a.y * act1);
              }
              box_write(box_a, lane, half * 4 + j, make_uint4(du[0], du[1], du[2], du[3]));
              box_write(box_b, lane, half * 4 + j, make_uint4(dg[0], dg[1], dg[2], dg[3]));
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < M) {
            tma_store_2d(&tmC, box_a, col0, row0);
            tma_store_2d(&tmC, box_b, I + col0, row0);
            tma_store_commit();
            tma_store_wait_read<0>();
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) box_write(box_a, lane, j, make_uint4(yp[4 * j], yp[4 * j + 1], yp[4 * j + 2], yp[4 * j + 3]));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < M) {
            tma_store_2d(&tmC2, box_a, col0, row0);
            tma_store_commit();
          }
        }
        continue;
      }

      if (opts.tma_store) {
        constexpr bool kBf16 = EPI == EPI_BF16 || EPI == EPI_BF16_ACC;
        constexpr int kColsPerBox = kBf16 ? 64 : 32;
        constexpr int kBoxes = BN / kColsPerBox;
#pragma unroll 1
        for (int c = 0; c < kBoxes; ++c) {
          const int col0 = tc.ni * BN + c * kColsPerBox;
          if (col0 >= N) break;
          uint8_t* box = stage0 + (nstore & 1) * BOX_BYTES;
          if (TRACE) t0 = clock64();
          if (lane == 0) tma_store_wait_read<1>();  // the store that used this box two boxes ago has read it
          __syncwarp();
          if (TRACE) wait_store += clock64() - t0;
          if (kBf16) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t v[32];
              B200_TMEM_LD_32(v, t_row + c * 64 + half * 32);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                box_write(box, lane, half * 4 + j,
                          make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]) * alpha, __uint_as_float(v[8 * j + 1]) * alpha),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 2]) * alpha, __uint_as_float(v[8 * j + 3]) * alpha),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 4]) * alpha, __uint_as_float(v[8 * j + 5]) * alpha),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 6]) * alpha, __uint_as_float(v[8 * j + 7]) * alpha)));
              }
            }
          } else {
            uint32_t v[32];
            B200_TMEM_LD_32(v, t_row + c * 32);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              box_write(box, lane, j,
                        make_uint4(__float_as_uint(__uint_as_float(v[4 * j]) * alpha), __float_as_uint(__uint_as_float(v[4 * j + 1]) * alpha),
                                   __float_as_uint(__uint_as_float(v[4 * j + 2]) * alpha), __float_as_uint(__uint_as_float(v[4 * j + 3]) * alpha)));
            }
          }
          if (c == kBoxes - 1 || col0 + kColsPerBox >= N) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < M) {
            if (EPI == EPI_F32_ACC || EPI == EPI_BF16_ACC) tma_reduce_add_2d(&tmC, box, col0, row0);
            else tma_store_2d(&tmC, box, col0, row0);
            tma_store_commit();
          }
          ++nstore;
        }
        continue;
      }

      // register -> global path
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tc.ni * BN + c * 32;
        if (col0 >= N) break;
        uint32_t v[32];
        B200_TMEM_LD_32(v, t_row + c * 32);
        tmem_ld_wait();
        if (row < M) {
          if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + (long long)row * ldc + col0;
            if (col0 + 32 <= N && (ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(Cv) & 15) == 0) {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * j + e]) * alpha;
                if (EPI == EPI_BF16_ACC) {
                  const uint4 old = d4[j];
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                d4[j] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
              }
            } else {
              for (int e = 0; e < 32 && col0 + e < N; ++e) {
                float f = __uint_as_float(v[e]) * alpha;
                if (EPI == EPI_BF16_ACC) f += __bfloat162float(dst[e]);
                dst[e] = __float2bfloat16(f);
              }
            }
          } else {
            float* dst = reinterpret_cast<float*>(Cv) + (long long)row * ldc + col0;
            if (col0 + 32 <= N && (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(Cv) & 15) == 0) {
              float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 o = make_float4(__uint_as_float(v[4 * j]) * alpha, __uint_as_float(v[4 * j + 1]) * alpha,
                                       __uint_as_float(v[4 * j + 2]) * alpha, __uint_as_float(v[4 * j + 3]) * alpha);
                if (EPI == EPI_F32_ACC) {
                  const float4 old = d4[j];
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                d4[j] = o;
              }
            } else {
              for (int e = 0; e < 32 && col0 + e < N; ++e) {
                float f = __uint_as_float(v[e]) * alpha;
                if (EPI == EPI_F32_ACC) f += dst[e];
                dst[e] = f;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
    // every bulk store of this warp has left shared memory and reached global memory before the CTA exits
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
    if (TRACE && q == 2 && lane == 0) {
      trace[4] = wait_acc;
      trace[5] = clock64() - t_begin;
      trace[7] = wait_store;
    }
  }

  // Neither CTA may free its TMEM or exit while the other can still reach into it.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}

struct LaunchArgs {
  CUtensorMap tmA, tmB, tmC, tmC2;
  void* C;
  int M, N, K;
  long long ldc;
  float alpha;
  int* status;
  int max_ctas;
  KernelOpts opts;
  cudaStream_t stream;
};

template <int A_MN, int B_MN, int EPI, bool TRACE>
void launch_variant(const LaunchArgs& a) {
  auto kernel = gemm_bf16_2sm_kernel<A_MN, B_MN, EPI, TRACE>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "gemm 2sm smem attr");
    configured = true;
  }
  const int tiles = ((a.M + 2 * BM - 1) / (2 * BM)) * ((a.N + BN - 1) / BN) * a.opts.split_k;
  int pairs = sm_count() / 2;
  if (a.max_ctas > 0 && a.max_ctas / 2 < pairs) pairs = a.max_ctas / 2 > 0 ? a.max_ctas / 2 : 1;
  if (tiles < pairs) pairs = tiles;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, a.tmA, a.tmB, a.tmC, a.tmC2, a.C, a.M, a.N, a.K, a.ldc, a.alpha, a.status, a.opts),
             "gemm_bf16_2sm launch");
  count_launch();
}

template <int A_MN, int B_MN>
void launch_epi(int epi, const LaunchArgs& a) {
  const bool trace = a.opts.trace != nullptr;
  switch (epi) {
    case EPI_BF16:
      if (trace) launch_variant<A_MN, B_MN, EPI_BF16, true>(a);
      else launch_variant<A_MN, B_MN, EPI_BF16, false>(a);
      break;
    case EPI_F32: launch_variant<A_MN, B_MN, EPI_F32, false>(a); break;
    case EPI_F32_ACC:
      if (trace) launch_variant<A_MN, B_MN, EPI_F32_ACC, true>(a);
      else launch_variant<A_MN, B_MN, EPI_F32_ACC, false>(a);
      break;
    case EPI_BF16_ACC: launch_variant<A_MN, B_MN, EPI_BF16_ACC, false>(a); break;
    default: throw std::runtime_error("gemm_bf16_2sm: unknown epilogue");
  }
}

// Raster: the 74 pairs that run at a time should cover a patch of the output that is as square as possible in bytes
// of operands (its A rows and B rows are what L2 serves to all of them); a panel is `group` tiles tall and spans all
// columns, so consecutive pairs share A within a panel column and B across the panel's rows.
int default_group(int M, int N) {
  const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
  int g = 8;
  if (n_tiles < 9) g = 16;
  if (g > m_tiles) g = m_tiles;
  return g > 0 ? g : 1;
}

// Split of K for the accumulating epilogues (the partial sums meet in the bulk reduction, so the split costs nothing):
// taken when the tiles alone would leave the last wave of CTA pairs mostly idle.
int default_split(int M, int N, int K, int pairs) {
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const int k_blocks = (K + BK - 1) / BK;
  auto efficiency = [&](int split) {
    const int units = tiles * split;
    const int waves = (units + pairs - 1) / pairs;
    return (double)units / ((double)waves * pairs);
  };
  int best = 1;
  double best_eff = efficiency(1);
  for (int split = 2; split <= 4; ++split) {
    if (k_blocks / split < 16) break;
    const double e = efficiency(split);
    if (e > best_eff + 0.04) {
      best = split;
      best_eff = e;
    }
  }
  return best;
}

PairGemmTuning g_tuning;

}  // namespace

PairGemmTuning& pair_gemm_tuning() { return g_tuning; }

// Same contract as gemm_bf16 (see gemm_bf16.cu).
void gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                   bool a_mn, bool b_mn, int epi, float alpha, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  if ((lda & 7) || (ldb & 7)) throw std::runtime_error("gemm_bf16_2sm: leading dimensions of A and B must be multiples of 8");
  LaunchArgs a;
  a.tmA = a_mn ? make_tensor_map_2d_b16(A, M, K, lda, 64, BK) : make_tensor_map_2d_b16(A, K, M, lda, BK, BM);
  a.tmB = b_mn ? make_tensor_map_2d_b16(B, N, K, ldb, 64, BK) : make_tensor_map_2d_b16(B, K, N, ldb, BK, BN_HALF);
  const bool bf16_out = epi == EPI_BF16 || epi == EPI_BF16_ACC;
  const int esize = bf16_out ? 2 : 4;
  const bool c_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc * esize) % 16 == 0 && !g_tuning.direct_store;
  if (c_ok) a.tmC = bf16_out ? make_tensor_map_2d_b16(C, N, M, ldc, 64, 32) : make_tensor_map_2d_f32(C, N, M, ldc, 32, 32);
  else a.tmC = a.tmA;
  a.tmC2 = a.tmC;
  a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc; a.alpha = alpha; a.status = status; a.max_ctas = max_ctas; a.stream = stream;
  a.opts.group = g_tuning.group != 0 ? g_tuning.group : default_group(M, N);
  a.opts.tma_store = c_ok ? 1 : 0;
  a.opts.k_skew = g_tuning.k_skew;
  a.opts.swiglu_i = 0;
  a.opts.fc = nullptr;
  a.opts.ldfc = 0;
  a.opts.split_k = 1;
  if (c_ok && (epi == EPI_F32_ACC || epi == EPI_BF16_ACC) && max_ctas <= 0)
    a.opts.split_k = g_tuning.split_k > 0 ? g_tuning.split_k : default_split(M, N, K, sm_count() / 2);
  {
    const int k_blocks = (K + BK - 1) / BK;  // every partial sum covers at least four k-blocks
    if (a.opts.split_k > k_blocks / 4) a.opts.split_k = k_blocks / 4 > 0 ? k_blocks / 4 : 1;
  }
  a.opts.trace = g_tuning.trace;
  if (a_mn) {
    if (b_mn) launch_epi<1, 1>(epi, a);
    else launch_epi<1, 0>(epi, a);
  } else {
    if (b_mn) launch_epi<0, 1>(epi, a);
    else launch_epi<0, 0>(epi, a);
  }
}

// fc[M, 2I] = A[M, K] W[2I, K]^T (both halves stored) and act[M, I] = fc[:, :I] * silu(fc[:, I:]) in one kernel.
void gemm_bf16_swiglu(const void* A, const void* W, void* fc, void* act, int M, int I, int K, long long lda, long long ldw,
                      long long ldfc, long long ldact, int* status, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return;
  if ((lda & 7) || (ldw & 7) || (ldfc & 7) || (ldact & 7) || (I % BN_HALF) != 0 || M < 2 * BM)
    throw std::runtime_error("gemm_bf16_swiglu: needs I % 128 == 0, M >= 256 and leading dimensions that are multiples of 8");
  LaunchArgs a;
  a.tmA = make_tensor_map_2d_b16(A, K, M, lda, BK, BM);
  a.tmB = make_tensor_map_2d_b16(W, K, 2 * (long long)I, ldw, BK, BN_HALF);
  a.tmC = make_tensor_map_2d_b16(fc, 2 * (long long)I, M, ldfc, 64, 32);
  a.tmC2 = make_tensor_map_2d_b16(act, I, M, ldact, 64, 32);
  a.C = fc; a.M = M; a.N = 2 * I; a.K = K; a.ldc = ldfc; a.alpha = 1.f; a.status = status; a.max_ctas = 0; a.stream = stream;
  a.opts.group = g_tuning.group != 0 ? g_tuning.group : default_group(M, 2 * I);
  a.opts.tma_store = 1;
  a.opts.k_skew = g_tuning.k_skew;
  a.opts.swiglu_i = I;
  a.opts.fc = nullptr;
  a.opts.ldfc = 0;
  a.opts.split_k = 1;
  a.opts.trace = nullptr;
  launch_variant<0, 0, EPI_SWIGLU, false>(a);
}

// d(fc)[M, 2I] and act[M, I] from dy[M, K] . W[K, I] (W row-major [K, I], i.e. the down-projection weight [H, I]) and the saved
// projection fc[M, 2I] = [up | gate]:  d(up) = d(act) silu(gate), d(gate) = d(act) up silu'(gate), act = up silu(gate).
void gemm_bf16_swiglu_bwd(const void* dy, const void* W, const void* fc, void* dfc, void* act, int M, int I, int K, long long lddy,
                          long long ldw, long long ldfc, long long lddfc, long long ldact, int* status, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return;
  if ((lddy & 7) || (ldw & 7) || (ldfc & 7) || (lddfc & 7) || (ldact & 7) || (I % 64) != 0 || M < 2 * BM ||
      (reinterpret_cast<uintptr_t>(fc) & 15) != 0)
    throw std::runtime_error("gemm_bf16_swiglu_bwd: needs I % 64 == 0, M >= 256, 16-byte aligned fc and leading dimensions that are multiples of 8");
  LaunchArgs a;
  a.tmA = make_tensor_map_2d_b16(dy, K, M, lddy, BK, BM);
  a.tmB = make_tensor_map_2d_b16(W, I, K, ldw, 64, BK);  // MN-major: rows are k, columns are the intermediate channels
  a.tmC = make_tensor_map_2d_b16(dfc, 2 * (long long)I, M, lddfc, 64, 32);
  a.tmC2 = make_tensor_map_2d_b16(act, I, M, ldact, 64, 32);
  a.C = dfc; a.M = M; a.N = I; a.K = K; a.ldc = lddfc; a.alpha = 1.f; a.status = status; a.max_ctas = 0; a.stream = stream;
  a.opts.group = g_tuning.group != 0 ? g_tuning.group : default_group(M, I);
  a.opts.tma_store = 1;
  a.opts.k_skew = g_tuning.k_skew;
  a.opts.swiglu_i = I;
  a.opts.fc = reinterpret_cast<const __nv_bfloat16*>(fc);
  a.opts.ldfc = ldfc;
  a.opts.split_k = 1;
  a.opts.trace = g_tuning.trace;
  if (a.opts.trace != nullptr) launch_variant<0, 1, EPI_SWIGLU_BWD, true>(a);
  else launch_variant<0, 1, EPI_SWIGLU_BWD, false>(a);
}

}  // namespace b200

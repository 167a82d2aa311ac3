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
#include <cuda.h>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

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
constexpr int GROUP_M = 4;  // in units of 256-row tiles
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 + 256;

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ACC = 3 };

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

struct TileCoord {
  int m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(m_tiles - first_m, GROUP_M);
  const int r = tile - g * per_group;
  return {(first_m + r % gsize) * (2 * BM), (r / gsize) * BN};
}

template <int A_MN, int B_MN, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
    gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         void* __restrict__ Cv, int M, int N, int K, long long ldc, float alpha, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
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
  const int total = m_tiles * n_tiles;

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
      for (int tile = pair; tile < total && ok; tile += num_pairs) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles);
        const int m0 = tc.m0 + (int)cta_rank * BM;
        const int n0 = tc.n0 + (int)cta_rank * BN_HALF;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
            ok = false;
            break;
          }
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), &tmA, full_leader, m0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(a_dst, &tmA, full_leader, kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j) tma_load_2d_pair(b_dst + j * (BK * 128), &tmB, full_leader, n0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(b_dst, &tmB, full_leader, kb * BK, n0);
          }
        }
      }
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
      for (int tile = pair; tile < total && ok; tile += num_pairs, ++tcount) {
        const uint32_t buf = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutMma, abort_flag);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutMma, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_base = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(a_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(b_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss_2sm(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
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
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue: this CTA's 128 x 256 half
    const int q = warp & 3;
    uint32_t tcount = 0;
    for (int tile = pair; tile < total; tile += num_pairs, ++tcount) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles);
      const uint32_t buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], aph, abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
        break;
      }
      tc_fence_after_sync();
      const int row = tc.m0 + (int)cta_rank * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tc.n0 + c * 32;
        if (col0 >= N) break;
        uint32_t v[32];
        B200_TMEM_LD_32(v, t_row + c * 32);
        tmem_ld_wait();
        if (row < M) {
          if (EPI == EPI_BF16 || EPI == EPI_BF16_ACC) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + (long long)row * ldc + col0;
            if (col0 + 32 <= N && (ldc & 7) == 0) {
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
            if (col0 + 32 <= N && (ldc & 3) == 0) {
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

template <int A_MN, int B_MN, int EPI>
void launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int M, int N, int K, long long ldc, float alpha,
                    int* status, int max_ctas, cudaStream_t stream) {
  auto kernel = gemm_bf16_2sm_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "gemm 2sm smem attr");
    configured = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = sm_count() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < pairs) pairs = tiles;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  check_cuda(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, C, M, N, K, ldc, alpha, status), "gemm_bf16_2sm launch");
  count_launch();
}

template <int A_MN, int B_MN>
void launch_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int M, int N, int K, long long ldc,
                float alpha, int* status, int max_ctas, cudaStream_t stream) {
  switch (epi) {
    case EPI_BF16: launch_variant<A_MN, B_MN, EPI_BF16>(tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream); break;
    case EPI_F32: launch_variant<A_MN, B_MN, EPI_F32>(tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream); break;
    case EPI_F32_ACC: launch_variant<A_MN, B_MN, EPI_F32_ACC>(tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream); break;
    case EPI_BF16_ACC: launch_variant<A_MN, B_MN, EPI_BF16_ACC>(tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream); break;
    default: throw std::runtime_error("gemm_bf16_2sm: unknown epilogue");
  }
}

}  // namespace

// Same contract as gemm_bf16 (see gemm_bf16.cu).
void gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                   bool a_mn, bool b_mn, int epi, float alpha, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  if ((lda & 7) || (ldb & 7)) throw std::runtime_error("gemm_bf16_2sm: leading dimensions of A and B must be multiples of 8");
  const CUtensorMap tmA = a_mn ? make_tensor_map_2d_b16(A, M, K, lda, 64, BK) : make_tensor_map_2d_b16(A, K, M, lda, BK, BM);
  const CUtensorMap tmB = b_mn ? make_tensor_map_2d_b16(B, N, K, ldb, 64, BK) : make_tensor_map_2d_b16(B, K, N, ldb, BK, BN_HALF);
  if (a_mn) {
    if (b_mn) launch_epi<1, 1>(epi, tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream);
    else launch_epi<1, 0>(epi, tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream);
  } else {
    if (b_mn) launch_epi<0, 1>(epi, tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream);
    else launch_epi<0, 0>(epi, tmA, tmB, C, M, N, K, ldc, alpha, status, max_ctas, stream);
  }
}

}  // namespace b200

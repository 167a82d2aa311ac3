// Tensor-parallel GEMMs fused with their collective, one kernel each, over NVLink peer memory.
//
//   all-gather + GEMM   Y[T, N] = gather_r(X_r)[T, K] . W^T        X_r: [T / tp, K] rows of rank r (symmetric memory)
//   GEMM + reduce-scatter   Y_r[T / tp, N] = sum over ranks of (X[T, K] . W^T)[rows of r]
//
// Both are the persistent tcgen05 GEMM of gemm/gemm_bf16.cu (128 x 256 x 64 tiles, 4-stage TMA ring, two TMEM
// accumulators, warp 0 = TMA, warp 1 = MMA, warps 2-5 = epilogue) with the transfer folded in:
//
// * all-gather: the first `copy_ctas` CTAs do no math. One thread of each drives TMA bulk copies (untiled
//   cp.async.bulk, no multicast) peer -> shared memory ring -> this GPU's staging buffer, 128 rows at a time, and
//   publishes `ready[m_tile] = epoch` with a release store when a row block has landed. The GEMM CTAs walk the row
//   blocks starting with this rank's own rows (already in place), so the first T / tp rows of math hide the transfer;
//   before the first TMA load of a remote row block the producer thread waits (bounded) for its flag. Every remote
//   byte crosses NVLink exactly once and is then read from local memory / L2 by all the column tiles that need it.
// * reduce-scatter: the epilogue stores each bf16 fragment straight into the owner rank's memory (16-byte peer
//   stores), into the slot reserved there for this source rank: slots[source][T / tp, N]. Row blocks owned by other
//   ranks are computed first and this rank's own last, so the remote stores drain while local tiles still compute.
//   After a peer barrier every rank sums its `tp` slots in fp32 (`sum_slots_bf16`): no atomics, every partial result
//   crosses NVLink once as bf16, and the sum is in rank order (reproducible).
//
// B (the weight) is K-major [N, K] (forward) or MN-major [K, N] (data gradients). A is row-major [T, K].
// Shapes: T a multiple of 128 * tp; K, N multiples of 8.
#include <stdexcept>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "peer.h"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int TMEM_COLS = 512;
constexpr int RING_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 256;

constexpr int PIECE_BYTES = 16 * 1024;  // one bulk copy
constexpr int HALF = 4;                 // pieces per batch; two batches (one ring) in flight
static_assert(2 * HALF * PIECE_BYTES <= RING_BYTES, "copy ring must fit in the GEMM ring's shared memory");
constexpr uint32_t kFlagSpinLimit = 1u << 24;  // x ~100 ns sleep: a couple of seconds

enum : int { MODE_AG = 1, MODE_RS = 2 };

struct TileCoord {
  int mi, m0, n0;  // processing index of the row block, first row, first column
};

// Row blocks are visited rank by rank: all-gather starts with this rank's rows, reduce-scatter ends with them.
__device__ __forceinline__ int actual_m_tile(int mi, int tiles_per_rank, int rank, int world, int mode) {
  const int step = mi / tiles_per_rank;
  const int owner = (rank + step + (mode == MODE_RS ? 1 : 0)) % world;
  return owner * tiles_per_rank + (mi - step * tiles_per_rank);
}

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles, int tiles_per_rank, int rank, int world, int mode) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(m_tiles - first_m, GROUP_M);
  const int r = tile - g * per_group;
  const int mi = first_m + r % gsize;
  return {mi, actual_m_tile(mi, tiles_per_rank, rank, world, mode) * BM, (r / gsize) * BN};
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct FusedArgs {
  PeerPtrs peers;     // AG: X_r of every rank (bf16 [T / tp, K]); RS: slot buffers of every rank (bf16 [tp][T / tp, N])
  void* staging;      // AG: local [T, K] bf16 gather target (this rank's own rows already in place)
  int* ready;         // AG: one flag per row block
  int epoch;          // AG: value that marks a flag as set for this launch
  int rank, world, copy_ctas;
};

template <int B_MN, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
    tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv, int M, int N,
                   int K, long long ldc, FusedArgs fa, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint64_t* copy_bar = bars + 2 * STAGES + 4;  // 2 * HALF barriers of the copy ring
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + 2 * HALF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = M / BM;
  const int n_tiles = (N + BN - 1) / BN;
  const int k_blocks = (K + BK - 1) / BK;
  const int total = m_tiles * n_tiles;
  const int tiles_per_rank = m_tiles / fa.world;
  const int copy_ctas = MODE == MODE_AG ? fa.copy_ctas : 0;

  // ------------------------------------------------------------------------------------------------ gather CTAs
  if (MODE == MODE_AG && (int)blockIdx.x < copy_ctas) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < 2 * HALF; ++s) mbar_init(&copy_bar[s], 1);
      *abort_flag = 0;
      fence_barrier_init();
      const long long unit_bytes = (long long)BM * K * 2;  // one row block, contiguous on both sides
      const int pieces = (int)((unit_bytes + PIECE_BYTES - 1) / PIECE_BYTES);
      const int batches = (pieces + HALF - 1) / HALF;
      uint32_t uses = 0;                  // batches so far: selects the half of the ring
      uint32_t slot_uses[2 * HALF] = {};  // completed loads per slot: parity of its barrier
      bool ok = true;
      // remote row blocks in the order the GEMM CTAs consume them, dealt round-robin to the gather CTAs
      for (int mi = tiles_per_rank + blockIdx.x; mi < m_tiles && ok; mi += copy_ctas) {
        const int m_tile = actual_m_tile(mi, tiles_per_rank, fa.rank, fa.world, MODE_AG);
        const int owner = m_tile / tiles_per_rank;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(fa.peers.p[owner]) + (long long)(m_tile - owner * tiles_per_rank) * unit_bytes;
        uint8_t* dst = reinterpret_cast<uint8_t*>(fa.staging) + (long long)m_tile * unit_bytes;
        auto issue_loads = [&](int batch, uint32_t half) {
          for (int j = 0; j < HALF; ++j) {
            const int p = batch * HALF + j;
            if (p >= pieces) break;
            const long long off = (long long)p * PIECE_BYTES;
            const uint32_t bytes = (uint32_t)min((long long)PIECE_BYTES, unit_bytes - off);
            uint64_t* bar = &copy_bar[half * HALF + j];
            mbar_arrive_expect_tx(bar, bytes);
            bulk_load(smem + (half * HALF + j) * PIECE_BYTES, src + off, bytes, bar);
          }
        };
        issue_loads(0, uses & 1);
        for (int b = 0; b < batches && ok; ++b, ++uses) {
          const uint32_t half = uses & 1;
          if (b + 1 < batches) {
            tma_store_wait_read<0>();  // the other half's previous stores have left shared memory
            issue_loads(b + 1, half ^ 1);
          }
          for (int j = 0; j < HALF; ++j) {
            const int p = b * HALF + j;
            if (p >= pieces) break;
            if (!mbar_wait(&copy_bar[half * HALF + j], slot_uses[half * HALF + j]++ & 1, abort_flag)) {
              raise_status(status, kStatusWaitTimeoutPeer, abort_flag);
              ok = false;
              break;
            }
            const long long off = (long long)p * PIECE_BYTES;
            const uint32_t bytes = (uint32_t)min((long long)PIECE_BYTES, unit_bytes - off);
            bulk_store(dst + off, smem + (half * HALF + j) * PIECE_BYTES, bytes);
          }
          tma_store_commit();
        }
        tma_store_wait<0>();  // the row block is in this GPU's memory
        fence_proxy_async_all();
        __threadfence();
        if (ok) st_release_gpu(&fa.ready[m_tile], fa.epoch);
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // bounded grace for copies still in flight
        tma_store_wait<0>();
      }
    }
    return;
  }

  // ------------------------------------------------------------------------------------------------ GEMM CTAs
  const int cta = (int)blockIdx.x - copy_ctas;
  const int ctas = (int)gridDim.x - copy_ctas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      int last_checked = -1;
      for (int tile = cta; tile < total && ok; tile += ctas) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, tiles_per_rank, fa.rank, fa.world, MODE);
        if (MODE == MODE_AG && tc.mi >= tiles_per_rank && tc.mi != last_checked) {
          // rows of another rank: wait until the gather CTAs have landed this row block
          const int* flag = &fa.ready[tc.m0 / BM];
          uint32_t spins = 0;
          while (ld_acquire_gpu(flag) != fa.epoch) {
            if (++spins > kFlagSpinLimit || *abort_flag) {
              raise_status(status, kStatusWaitTimeoutPeer, abort_flag);
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();  // the staged rows were written by other SMs; the loads below are TMA reads
          last_checked = tc.mi;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          tma_load_2d(sA + s * A_STAGE_BYTES, &tmA, &full[s], kb * BK, tc.m0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, &full[s], tc.n0 + j * 64, kb * BK);
          } else {
            tma_load_2d(b_dst, &tmB, &full[s], kb * BK, tc.n0);
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, B_MN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = cta; tile < total && ok; tile += ctas, ++tcount) {
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
            const uint64_t da = umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(b_base + k * 16 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    uint32_t tcount = 0;
    const int rows_per_rank = tiles_per_rank * BM;
    for (int tile = cta; tile < total; tile += ctas, ++tcount) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, tiles_per_rank, fa.rank, fa.world, MODE);
      const uint32_t buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], aph, abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
        break;
      }
      tc_fence_after_sync();
      const int row = tc.m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tc.n0 + c * 32;
        if (col0 >= N) break;
        uint32_t v[32];
        B200_TMEM_LD_32(v, t_row + c * 32);
        tmem_ld_wait();
        {
          __nv_bfloat16* dst;
          if (MODE == MODE_RS) {
            // slot of this source rank in the owner's buffer: [world][rows_per_rank][ldc]
            const int owner = tc.m0 / rows_per_rank;
            dst = reinterpret_cast<__nv_bfloat16*>(fa.peers.p[owner]) +
                  ((long long)fa.rank * rows_per_rank + (row - owner * rows_per_rank)) * ldc + col0;
          } else {
            dst = reinterpret_cast<__nv_bfloat16*>(Cv) + (long long)row * ldc + col0;
          }
          if (col0 + 32 <= N) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
              d4[j] = o;
            }
          } else {
            for (int e = 0; e < 32 && col0 + e < N; ++e) dst[e] = __float2bfloat16(__uint_as_float(v[e]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[i] = sum over s of slots[s][i] (bf16 in, fp32 sum in slot order, bf16 out); i in units of 8 elements.
__global__ void sum_slots_kernel(const uint4* __restrict__ slots, uint4* __restrict__ out, long long nv, int world) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) {
      const uint4 v = slots[(long long)s * nv + i];
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      acc[0] += a.x, acc[1] += a.y, acc[2] += b.x, acc[3] += b.y, acc[4] += c.x, acc[5] += c.y, acc[6] += d.x, acc[7] += d.y;
    }
    out[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

template <int B_MN, int MODE>
void launch(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, int M, int N, int K, long long ldc, const FusedArgs& fa, int* status,
            cudaStream_t stream) {
  auto kernel = tp_gemm_kernel<B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "tp_gemm smem attr");
    configured = true;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  int grid = sm_count();  // at most one CTA per SM: the gather CTAs and the GEMM CTAs that wait for them are co-resident
  const int copy = MODE == MODE_AG ? fa.copy_ctas : 0;
  if (tiles + copy < grid) grid = tiles + copy;
  kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, C, M, N, K, ldc, fa, status);
  count_launch();
  check_cuda(cudaGetLastError(), "tp_gemm launch");
}

void check_shapes(int M, int N, int K, int world, const char* what) {
  if (world < 1 || world > kMaxPeers) throw std::runtime_error(std::string(what) + ": bad group size");
  if (M <= 0 || M % (BM * world) != 0) throw std::runtime_error(std::string(what) + ": rows must be a positive multiple of 128 x group size");
  if (N <= 0 || K <= 0 || N % 8 || K % 8) throw std::runtime_error(std::string(what) + ": N and K must be positive multiples of 8");
}

}  // namespace

// Y[M, N] (bf16, row stride ldc) = gather(X)[M, K] . W^T. `staging` ([M, K] bf16, contiguous) holds this rank's rows at
// [rank * M / world, ...) already; the other rows are fetched from `x_ptrs[r]` ([M / world, K] contiguous on rank r).
void ag_gemm_bf16(const PeerPtrs& x_ptrs, void* staging, int* ready, int epoch, const void* W, void* Y, int M, int N, int K, long long ldw,
                  long long ldc, bool w_mn, int rank, int copy_ctas, int* status, cudaStream_t stream) {
  const int world = x_ptrs.n;
  check_shapes(M, N, K, world, "ag_gemm");
  if (ldw % 8 || ldc % 8) throw std::runtime_error("ag_gemm: leading dimensions must be multiples of 8");
  if (world == 1) copy_ctas = 0;
  if (copy_ctas < 0 || copy_ctas > sm_count() / 2) throw std::runtime_error("ag_gemm: bad number of gather CTAs");
  if (world > 1 && copy_ctas == 0) throw std::runtime_error("ag_gemm: at least one gather CTA is needed");
  const CUtensorMap tmA = make_tensor_map_2d_b16(staging, K, M, K, BK, BM);
  const CUtensorMap tmB = w_mn ? make_tensor_map_2d_b16(W, N, K, ldw, 64, BK) : make_tensor_map_2d_b16(W, K, N, ldw, BK, BN);
  FusedArgs fa{x_ptrs, staging, ready, epoch, rank, world, copy_ctas};
  if (w_mn) launch<1, MODE_AG>(tmA, tmB, Y, M, N, K, ldc, fa, status, stream);
  else launch<0, MODE_AG>(tmA, tmB, Y, M, N, K, ldc, fa, status, stream);
}

// slots_r[rank][M / world, N] (bf16, row stride ldc) = (X[M, K] . W^T)[rows of r] for every r; rank r then sums its slots.
void gemm_rs_bf16(const void* X, const void* W, const PeerPtrs& out_ptrs, int M, int N, int K, long long ldx, long long ldw, long long ldc,
                  bool w_mn, int rank, int* status, cudaStream_t stream) {
  const int world = out_ptrs.n;
  check_shapes(M, N, K, world, "gemm_rs");
  if (ldx % 8 || ldw % 8 || ldc % 8) throw std::runtime_error("gemm_rs: leading dimensions must be multiples of 8");
  const CUtensorMap tmA = make_tensor_map_2d_b16(X, K, M, ldx, BK, BM);
  const CUtensorMap tmB = w_mn ? make_tensor_map_2d_b16(W, N, K, ldw, 64, BK) : make_tensor_map_2d_b16(W, K, N, ldw, BK, BN);
  FusedArgs fa{out_ptrs, nullptr, nullptr, 0, rank, world, 0};
  if (w_mn) launch<1, MODE_RS>(tmA, tmB, nullptr, M, N, K, ldc, fa, status, stream);
  else launch<0, MODE_RS>(tmA, tmB, nullptr, M, N, K, ldc, fa, status, stream);
}

void sum_slots_bf16(const void* slots, void* out, long long n, int world, cudaStream_t stream) {
  if (n == 0) return;
  if (n % 8) throw std::runtime_error("sum_slots: length must be a multiple of 8");
  const long long nv = n / 8;
  long long blocks = (nv + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  sum_slots_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(slots), reinterpret_cast<uint4*>(out), nv, world);
  count_launch();
  check_cuda(cudaGetLastError(), "sum_slots launch");
}

}  // namespace b200

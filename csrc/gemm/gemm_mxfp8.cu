// MXFP8 GEMM for sm_100a: tcgen05.mma kind::mxf8f6f4 with block scaling (OCP microscaling: e4m3 / e5m2 payload, one
// UE8M0 power-of-two scale per 32 elements along the contraction dimension), fp32 accumulation in tensor memory.
//
//   C[M,N] = alpha * sum_kb 2^(sa[m,kb]-127) * 2^(sb[n,kb]-127) * sum_{k in block kb} A(m,k) * B(n,k)
//
// Structure of gemm_fp8.cu (128 x 256 tiles, k-block = 128 bytes = four scale blocks, 4-stage TMA ring, warp 0 = TMA,
// warp 1 = MMA, warps 2-5 = epilogue) plus the scale path: per stage the producer also fetches the stage's scale
// factors (512 bytes for the 128 rows of A, 2 x 512 for the 256 rows of B; plain bulk copies on the same barrier), the MMA
// thread moves them from shared to tensor memory with tcgen05.cp (32x128b.warpx4) and issues four MMAs of K = 32 whose
// scale-factor ids 0..3 select the stage's four scale blocks. Tensor memory holds ONE 256-column accumulator next to
// four rotating 12-column scale slots (two accumulators plus scales do not fit into 512 columns), so the epilogue
// of a tile is not hidden behind the next tile's MMAs; with K in the thousands that costs a few percent.
//
// Scale factors arrive in the layout the tensor core reads (and the quantisation kernel writes): tiles of
// 128 rows x 4 scale blocks = 512 bytes, byte (r % 32) * 16 + ((r / 32) % 4) * 4 + (kb % 4) of tile
// (r / 128) * (K / 128) + kb / 4. Measured on a B200: the MMA takes the scale of accumulator row m from TMEM lane m,
// column base + m / 32, byte = scale id; for column n of B from lane n % 32, column base + n / 32, byte = scale id,
// which is exactly what the warpx4 copy of such a tile produces.
//
// Both operands may be K-major or MN-major (8-bit payloads allow both), so the forward, data-gradient and
// weight-gradient products of a linear layer read row-major tensors; what differs per product is along which dimension
// the 32-element blocks of the quantisation run.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes = elements
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int B_STAGE_BYTES = BN * BK;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int TMEM_COLS = 512;
constexpr int SF_TILE_BYTES = 512;               // 128 rows x 4 scale blocks
constexpr int SF_STAGE_BYTES = 3 * SF_TILE_BYTES;  // A tile + two B tiles
constexpr int SF_SLOTS = 4;                      // rotating scale slots in tensor memory
constexpr int SF_SLOT_COLS = 12;                 // 4 columns for A + 8 for B
constexpr int SF_TMEM_COL = BN;                  // scale slots sit behind the accumulator
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES + SF_STAGE_BYTES) + 1024 /*alignment slack*/ + 256 /*barriers*/;

// D[tmem] (+)= (A[smem] * B[smem]) with per-32-element block scales read from tensor memory.
__device__ __forceinline__ void umma_mxf8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tmem_sfa,
                                             uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}

// 32 rows x 16 bytes from shared memory into 4 TMEM columns, replicated into the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t tmem_dst, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}

// Descriptor of an unswizzled shared-memory matrix of 16-byte rows: 8-row groups `sbo_bytes` apart.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;
  return d;
}

// Untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), completing on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Instruction descriptor of the block-scaled kind: formats 0 = e4m3, 1 = e5m2; scales are UE8M0.
__host__ __device__ constexpr uint32_t idesc_mxf8(int m, int n, int a_fmt, int b_fmt, int a_mn, int b_mn) {
  return (uint32_t(a_fmt) << 7) | (uint32_t(b_fmt) << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) | (uint32_t(n >> 3) << 17) |
         (1u << 23) | (uint32_t(m >> 4) << 24);
}
constexpr uint32_t kSfIdShiftA = 29, kSfIdShiftB = 4;

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_BF16_ACC = 3 };

struct TileCoord {
  int m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(m_tiles - first_m, GROUP_M);
  const int r = tile - g * per_group;
  return {(first_m + r % gsize) * BM, (r / gsize) * BN};
}

template <int A_MN, int B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, void* __restrict__ Cv, int M, int N, int K,
                      long long ldc, float alpha, uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sSF = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + STAGES * SF_STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM;
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
      mbar_init(&acc_empty[b], 4);  // only buffer 0 is used: one accumulator
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES + SF_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          uint8_t* sf_dst = sSF + s * SF_STAGE_BYTES;
          const long long kt = kb, k_tiles = k_blocks;  // one 512-byte scale tile per 128 rows and k-block
          bulk_load(sf_dst, sfa + ((long long)(tc.m0 / 128) * k_tiles + kt) * SF_TILE_BYTES, SF_TILE_BYTES, &full[s]);
          bulk_load(sf_dst + SF_TILE_BYTES, sfb + ((long long)(tc.n0 / 128) * k_tiles + kt) * SF_TILE_BYTES, SF_TILE_BYTES, &full[s]);
          bulk_load(sf_dst + 2 * SF_TILE_BYTES, sfb + ((long long)(tc.n0 / 128 + 1) * k_tiles + kt) * SF_TILE_BYTES, SF_TILE_BYTES, &full[s]);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 128; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmA, &full[s], tc.m0 + j * 128, kb * BK);
          } else {
            tma_load_2d(a_dst, &tmA, &full[s], kb * BK, tc.m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, &full[s], tc.n0 + j * 128, kb * BK);
          } else {
            tma_load_2d(b_dst, &tmB, &full[s], kb * BK, tc.n0);
          }
        }
      }
      if (!ok) {
        // Unwind: give copies that are still in flight a bounded amount of time to land.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++tcount) {
        const uint32_t buf = 0;
        const uint32_t aph = tcount & 1;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutMma, abort_flag);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base;
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
          // this stage's scales: shared memory -> a free scale slot of tensor memory (ordered before the MMAs below)
          const uint32_t sf_smem = smem_u32(sSF + s * SF_STAGE_BYTES);
          const uint32_t sf_tmem = tmem_base + SF_TMEM_COL + (it % SF_SLOTS) * SF_SLOT_COLS;
          tmem_cp_32x128b_warpx4(sf_tmem, smem_desc_plain(sf_smem, 128, 128));
          tmem_cp_32x128b_warpx4(sf_tmem + 4, smem_desc_plain(sf_smem + SF_TILE_BYTES, 128, 128));
          tmem_cp_32x128b_warpx4(sf_tmem + 8, smem_desc_plain(sf_smem + 2 * SF_TILE_BYTES, 128, 128));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(a_base + k * 32 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(b_base + k * 32 * 128, BK * 128, 1024)
                                     : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_mxf8_ss(d_tmem, da, db, idesc | (uint32_t(k) << kSfIdShiftA) | (uint32_t(k) << kSfIdShiftB), sf_tmem, sf_tmem + 4,
                         (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, 128 TMEM lanes)
    const int q = warp & 3;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++tcount) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles);
      const uint32_t buf = 0;
      const uint32_t aph = tcount & 1;
      if (!mbar_wait(&acc_full[buf], aph, abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
        break;
      }
      tc_fence_after_sync();
      const int row = tc.m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tc.n0 + c * 32;
        if (col0 >= N) break;  // uniform across the warp
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
                  const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
                               o3 = unpack_bf16x2(old.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                d4[j] = o;
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
                float4 o;
                o.x = __uint_as_float(v[4 * j + 0]) * alpha;
                o.y = __uint_as_float(v[4 * j + 1]) * alpha;
                o.z = __uint_as_float(v[4 * j + 2]) * alpha;
                o.w = __uint_as_float(v[4 * j + 3]) * alpha;
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

template <int A_MN, int B_MN, int EPI>
void launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const uint8_t* sfa, const uint8_t* sfb, void* C, int M, int N, int K,
                    long long ldc, float alpha, uint32_t idesc, int* status, cudaStream_t stream) {
  auto kernel = gemm_mxfp8_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "gemm_mxfp8 smem attr");
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  kernel<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, sfa, sfb, C, M, N, K, ldc, alpha, idesc, status);
  count_launch();
  check_cuda(cudaGetLastError(), "gemm_mxfp8 launch");
}

template <int A_MN, int B_MN>
void launch_epi(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const uint8_t* sfa, const uint8_t* sfb, void* C, int M, int N,
                int K, long long ldc, float alpha, uint32_t idesc, int* status, cudaStream_t stream) {
  switch (epi) {
    case EPI_BF16: launch_variant<A_MN, B_MN, EPI_BF16>(tmA, tmB, sfa, sfb, C, M, N, K, ldc, alpha, idesc, status, stream); break;
    case EPI_F32: launch_variant<A_MN, B_MN, EPI_F32>(tmA, tmB, sfa, sfb, C, M, N, K, ldc, alpha, idesc, status, stream); break;
    case EPI_F32_ACC: launch_variant<A_MN, B_MN, EPI_F32_ACC>(tmA, tmB, sfa, sfb, C, M, N, K, ldc, alpha, idesc, status, stream); break;
    case EPI_BF16_ACC: launch_variant<A_MN, B_MN, EPI_BF16_ACC>(tmA, tmB, sfa, sfb, C, M, N, K, ldc, alpha, idesc, status, stream); break;
    default: throw std::runtime_error("gemm_mxfp8: unknown epilogue");
  }
}

}  // namespace

long long mx_scale_bytes(long long rows, long long k) {
  // scale tiles cover 128 rows x 128 contraction elements; the row tiles are padded to an even count so that a 256-column
  // tile of B always finds two of them
  const long long row_tiles = ((rows + 127) / 128 + 1) / 2 * 2;
  return row_tiles * (k / 128) * SF_TILE_BYTES;
}

// A: K-major -> [M, K] bytes with row stride lda; MN-major -> [K, M] with row stride lda. Same for B with N. K % 128 == 0.
// sfa / sfb: UE8M0 scale codes of A (M rows) and B (N rows) in 512-byte tiles (see the top of this file), sized by
// mx_scale_bytes. a_fmt / b_fmt: 0 = e4m3, 1 = e5m2. epi: 0 = bf16 store, 1 = fp32 store, 2 = fp32 accumulate, 3 = bf16 accumulate.
void gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long long lda,
                long long ldb, long long ldc, bool a_mn, bool b_mn, int a_fmt, int b_fmt, int epi, float alpha, int* status,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  if (K % BK) throw std::runtime_error("gemm_mxfp8: the contraction size must be a multiple of 128");
  if ((lda & 15) || (ldb & 15)) throw std::runtime_error("gemm_mxfp8: leading dimensions of A and B must be multiples of 16");
  if ((reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    throw std::runtime_error("gemm_mxfp8: scale buffers must be 16-byte aligned");
  const CUtensorMap tmA = a_mn ? make_tensor_map_2d_u8(A, M, K, lda, 128, BK) : make_tensor_map_2d_u8(A, K, M, lda, BK, BM);
  const CUtensorMap tmB = b_mn ? make_tensor_map_2d_u8(B, N, K, ldb, 128, BK) : make_tensor_map_2d_u8(B, K, N, ldb, BK, BN);
  const uint32_t idesc = idesc_mxf8(BM, BN, a_fmt, b_fmt, a_mn ? 1 : 0, b_mn ? 1 : 0);
  auto a8 = reinterpret_cast<const uint8_t*>(sfa);
  auto b8 = reinterpret_cast<const uint8_t*>(sfb);
  if (a_mn) {
    if (b_mn) launch_epi<1, 1>(epi, tmA, tmB, a8, b8, C, M, N, K, ldc, alpha, idesc, status, stream);
    else launch_epi<1, 0>(epi, tmA, tmB, a8, b8, C, M, N, K, ldc, alpha, idesc, status, stream);
  } else {
    if (b_mn) launch_epi<0, 1>(epi, tmA, tmB, a8, b8, C, M, N, K, ldc, alpha, idesc, status, stream);
    else launch_epi<0, 0>(epi, tmA, tmB, a8, b8, C, M, N, K, ldc, alpha, idesc, status, stream);
  }
}

}  // namespace b200

// Causal softmax attention backward over packed variable-length sequences (sm_100a).
//
// One CTA owns 128 keys of one document and one key/value head. K and V stay resident in shared memory;
// the CTA walks the query heads of the group and, for each, the query tiles that can see these keys:
//   S^T  = K Q^T,  dP^T = V dO^T                      (tcgen05, fp32 in TMEM)
//   P^T  = exp2(S^T * scale*log2e - lse*log2e)         (256 arithmetic threads: row = key, two warps share a row and split its columns)
//   dS^T = P^T o (dP^T - delta) * scale
//   dV  += P^T dO,  dK += dS^T Q,  dQ_tile = dS K       (tcgen05; dQ is added to an fp32 buffer by bulk tensor reductions)
// P^T never visits shared memory: it is written as bf16 over the S^T columns of tensor memory it was computed from and
// the dV product reads it there (A operand from TMEM). dS^T is written once to shared memory and used twice through two
// descriptors (K-major A operand of dK, MN-major A operand of dQ).
//
// The slowest single thing in a step is the bulk reduction that adds the 64 KB dQ tile into the fp32 accumulator (the
// TMA engine needs about 3000 clocks to read the tile), so four warps of their own move dQ from tensor memory to staging
// boxes and issue the reductions (the instruction blocks while the engine's queue is full, which would stall the
// arithmetic warps). The staging holds half a tile: the drain warps write the first 64 columns, keep the other 64 in
// registers (which frees the tensor-memory columns at once) and write them when the first reduction has read the boxes.
// Q is double-buffered, so S(i+1) is issued as soon as dV(i) has consumed P(i). Order of a step i:
//   MMA thread       dV(i) S(i+1) | dQ(i) dK(i) | dP(i+1) (once dQ(i) has left the columns of dP(i))
//   arithmetic warps P(i) from S(i) | dS(i) from dP(i)
//   drain warps      dQ(i): first half to the boxes, reduce, second half to the boxes, reduce
// dO(i+1) is loaded as soon as dV(i) has retired, Q(i+2) as soon as dK(i) has.
// Two small kernels bracket it: delta = rowsum(dO o O) before, fp32 dQ -> bf16 into the fused gradient after.
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/tensor_map.h"
#include "attention.h"

namespace b200 {

namespace {

constexpr int BT = 128;  // tile edge for both queries and keys
constexpr int SOFTMAX_WARPS = 8;   // two warps per TMEM lane quarter, each taking half of the columns
constexpr int PARTS = SOFTMAX_WARPS / 4;   // column parts of a 128-wide tile
constexpr int PART_COLS = BT / PARTS;      // 64
constexpr int PART_CHUNKS = PART_COLS / 32;
constexpr int DRAIN_WARPS = 4;             // one per TMEM lane quarter: dQ from tensor memory to the fp32 accumulator
constexpr int SOFTMAX_THREADS = SOFTMAX_WARPS * 32;
constexpr int BWD_THREADS = 64 + SOFTMAX_THREADS + DRAIN_WARPS * 32;  // producer, MMA issuer, arithmetic warps, dQ drain warps

template <int D>
struct BwdSmem {
  static constexpr int TILE_D = BT * D * 2;    // a [128 x D] bf16 tile
  static constexpr int TILE_S = BT * BT * 2;   // a [128 x 128] bf16 tile
  static constexpr int BOX = BT * 128;         // one dQ staging box: 128 rows x 32 fp32
  static constexpr int PHASE_BOXES = D / 64;   // boxes per half of the dQ tile
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_D;
  static constexpr int OFF_Q = OFF_V + TILE_D;          // two buffers
  static constexpr int OFF_DO = OFF_Q + 2 * TILE_D;
  static constexpr int OFF_DS = OFF_DO + TILE_D;        // dS^T
  static constexpr int OFF_STAGE = OFF_DS + TILE_S;     // dQ staging: half a tile
  static constexpr int OFF_ROW = OFF_STAGE + PHASE_BOXES * BOX;  // [2 buffers][lse 128 | delta 128] floats
  static constexpr int OFF_BAR = OFF_ROW + 2 * 2 * BT * 4;
  static constexpr int TOTAL = OFF_BAR + 256;
  static_assert(TOTAL <= 232448, "attention backward: shared-memory layout exceeds the 227 KB limit");
};

enum {
  B_KV = 0, B_Q_FULL = 1 /* two */, B_Q_EMPTY = 3 /* two */, B_DO_FULL = 5, B_DO_EMPTY = 6, B_S_FULL = 7, B_DP_FULL = 8,
  B_P_READY = 9, B_DS_READY = 10, B_DQ_FULL = 11, B_DQ_DRAINED = 12, B_ROWS = 13, B_COUNT = 14
};

template <int D, bool TRACE>
__global__ void __launch_bounds__(BWD_THREADS, 1)  // 14 warps: four on two of the schedulers, hence at most 128 registers
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dq, const float* __restrict__ lse, const float* __restrict__ delta,
                    __nv_bfloat16* __restrict__ dqkv, long long dqkv_stride, const int* __restrict__ cu_seqlens,
                    int num_docs, int T, int groups, int qpg, float scale, float scale_log2, int causal, int* status,
                    long long* trace_out) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using L = BwdSmem<D>;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sDO = smem + L::OFF_DO;
  uint8_t* sDS = smem + L::OFF_DS;
  uint8_t* sStage = smem + L::OFF_STAGE;
  float* s_rows = reinterpret_cast<float*>(smem + L::OFF_ROW);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grp = blockIdx.x;  // key/value head (fastest grid index: the long key tiles of every head are scheduled first)
  const int k_col = (grp * (qpg + 2) + qpg) * D;
  const int v_col = k_col + D;
  // optional cycle counters of the first CTA (the longest one): where its arithmetic threads and its MMA thread wait
  const bool tracing = TRACE && trace_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0;

  if ((smem_u32(smem) & 1023u) != 0) {
    // the swizzled tiles need a 1024-byte aligned base and the layout has no room for rounding up
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, kStatusBadArgument);
    return;
  }

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
    for (int b = 0; b < B_COUNT; ++b) mbar_init(&bars[b], (b == B_P_READY || b == B_DS_READY || b == B_ROWS) ? SOFTMAX_THREADS : (b == B_DQ_DRAINED ? DRAIN_WARPS * 32 : 1));
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
  const uint32_t tmem_S = tmem_base;             // 128 columns; bf16 P^T is written over the first half of every column part
  const uint32_t tmem_dP = tmem_base + BT;       // 128 columns; dQ (D columns) takes them once dP^T has been read
  const uint32_t tmem_dV = tmem_base + 2 * BT;   // D columns
  const uint32_t tmem_dK = tmem_base + 2 * BT + D;  // D columns

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
        const int q_col = (grp * (qpg + 2) + qh) * D;
        const int do_col = (grp * qpg + qh) * D;
        const int row = doc_start + qt * BT;
        const int b = it & 1;
        // Q(it) goes into the buffer that dK(it - 2) has finished with
        if (!mbar_wait(&bars[B_Q_EMPTY + b], ((it >> 1) & 1) ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
          break;
        }
        mbar_arrive_expect_tx(&bars[B_Q_FULL + b], L::TILE_D);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)
          tma_load_2d(sQ + b * L::TILE_D + kb * (BT * 128), &tm_qkv, &bars[B_Q_FULL + b], q_col + kb * 64, row);
        // dO(it) replaces dO(it - 1) once dV(it - 1) has retired
        if (!mbar_wait(&bars[B_DO_EMPTY], (it & 1) ^ 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutProducer, abort_flag);
          break;
        }
        mbar_arrive_expect_tx(&bars[B_DO_FULL], L::TILE_D);
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb) tma_load_2d(sDO + kb * (BT * 128), &tm_do, &bars[B_DO_FULL], do_col + kb * 64, row);
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
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base0 = smem_u32(sQ), do_base = smem_u32(sDO);
      const uint32_t ds_base = smem_u32(sDS);
      auto issue_s = [&](uint32_t q_base) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_S, umma_smem_desc_sw128(k_base + off, 16, 1024), umma_smem_desc_sw128(q_base + off, 16, 1024),
                      idesc_st, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_S_FULL]);
      };
      auto issue_dp = [&]() {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BT * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_dP, umma_smem_desc_sw128(v_base + off, 16, 1024), umma_smem_desc_sw128(do_base + off, 16, 1024),
                      idesc_st, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_DP_FULL]);
      };
      bool ok = mbar_wait(&bars[B_KV], 0, abort_flag) && mbar_wait(&bars[B_Q_FULL + 0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_s(q_base0);
        ok = mbar_wait(&bars[B_DO_FULL], 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        issue_dp();
      }
      long long tw[5] = {0, 0, 0, 0, 0}, t0 = 0;
      const long long t_begin = tracing ? clock64() : 0;
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        const uint32_t acc = it > 0 ? 1u : 0u;
        if (tracing) t0 = clock64();
        if (!mbar_wait(&bars[B_P_READY], ph, abort_flag)) { ok = false; break; }
        if (tracing) tw[0] += clock64() - t0;
        tc_fence_after_sync();
        // dV += P^T dO: 16 queries per step; the bf16 P^T of column part p sits in the first half of S columns [p*PART_COLS, +PART_COLS)
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t a_col = (k * 16 / PART_COLS) * PART_COLS + (k * 16 % PART_COLS) / 2;
          const uint32_t b_off = k * 16 * 128;  // MN-major B: 16 query rows per step
          umma_f16_ts(tmem_dV, tmem_S + a_col, umma_smem_desc_sw128(do_base + b_off, BT * 128, 1024), idesc_kv, (acc | (k != 0)) ? 1u : 0u);
        }
        umma_commit(&bars[B_DO_EMPTY]);
        if (it + 1 < n_iter) {
          const int nb = (it + 1) & 1;
          if (tracing) t0 = clock64();
          if (!mbar_wait(&bars[B_Q_FULL + nb], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          if (tracing) tw[1] += clock64() - t0;
          tc_fence_after_sync();
          issue_s(q_base0 + nb * L::TILE_D);  // overwrites P(it): dV(it) was issued before it
        }
        if (tracing) t0 = clock64();
        if (!mbar_wait(&bars[B_DS_READY], ph, abort_flag)) { ok = false; break; }
        if (tracing) tw[2] += clock64() - t0;
        tc_fence_after_sync();
        const uint32_t q_base = q_base0 + (it & 1) * L::TILE_D;
        // dQ first: the next dP, and with it the next dS, waits for dQ to leave its columns; dK is in nobody's way
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t off = k * 16 * 128;  // 16 key rows per step for both operands
          umma_f16_ss(tmem_dP, umma_smem_desc_sw128(ds_base + off, BT * 128, 1024),
                      umma_smem_desc_sw128(k_base + off, BT * 128, 1024), idesc_dq, k != 0 ? 1u : 0u);
        }
        umma_commit(&bars[B_DQ_FULL]);
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t a_off = (k / 4) * (BT * 128) + (k % 4) * 32;  // K-major A: 16 query columns per step
          const uint32_t b_off = k * 16 * 128;
          umma_f16_ss(tmem_dK, umma_smem_desc_sw128(ds_base + a_off, 16, 1024),
                      umma_smem_desc_sw128(q_base + b_off, BT * 128, 1024), idesc_kv, (acc | (k != 0)) ? 1u : 0u);
        }
        umma_commit(&bars[B_Q_EMPTY + (it & 1)]);
        if (it + 1 < n_iter) {
          if (tracing) t0 = clock64();
          if (!mbar_wait(&bars[B_DQ_DRAINED], ph, abort_flag)) { ok = false; break; }
          if (tracing) { tw[3] += clock64() - t0; t0 = clock64(); }
          if (!mbar_wait(&bars[B_DO_FULL], (it + 1) & 1, abort_flag)) { ok = false; break; }
          if (tracing) tw[4] += clock64() - t0;
          tc_fence_after_sync();
          issue_dp();
        }
      }
      if (tracing) {
        for (int i = 0; i < 5; ++i) trace_out[9 + i] = tw[i];
        trace_out[14] = clock64() - t_begin;
        trace_out[15] = n_iter;
      }
      if (!ok) raise_status(status, kStatusWaitTimeoutMma, abort_flag);
    }
    __syncwarp();
  } else if (warp >= 2 + SOFTMAX_WARPS) {
    // ---------------------------------------------------------------- dQ drain: TMEM -> fp32 staging -> bulk add into the accumulator
    // Each warp owns the 32 query rows of its TMEM lane quarter in every staging box and issues the reductions of its
    // own [32 x 32] pieces, so nothing here synchronises with another warp; the issue may block while the engine's
    // queue is full, which is why the arithmetic warps do not do this themselves.
    const int q4 = warp & 3;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    uint8_t* const my_rows = sStage + q4 * 32 * 128;  // rows [q4*32, +32) of box 0; box c is c * BOX further
    constexpr int PB = L::PHASE_BOXES;
    int qh = 0, qt = first_q_tile;
    for (int it = 0; it < n_iter; ++it) {
      const int head = grp * qpg + qh;
      const int row0 = doc_start + qt * BT + q4 * 32;
      const bool issue = lane == 0 && row0 < T;
      if (!mbar_wait(&bars[B_DQ_FULL], it & 1, abort_flag)) {
        raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
        break;
      }
      tc_fence_after_sync();
      if (lane == 0) tma_store_wait_read<0>();  // this warp's reductions of the previous step have read its pieces
      __syncwarp();
      // 128-byte-swizzled rows of 32 fp32: full lines at L2 instead of scattered 16-byte atomics. Query rows past the
      // document are exact zeros (their P is 0).
      auto to_boxes = [&](const uint32_t (&o)[PB][32]) {
#pragma unroll
        for (int c = 0; c < PB; ++c) {
          uint8_t* row = my_rows + c * L::BOX + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(row + ((ch ^ (lane & 7)) * 16)) = make_uint4(o[c][4 * ch], o[c][4 * ch + 1], o[c][4 * ch + 2], o[c][4 * ch + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
      };
      auto reduce = [&](int first_col) {
        if (issue) {
#pragma unroll
          for (int c = 0; c < PB; ++c) tma_reduce_add_2d(&tm_dq, my_rows + c * L::BOX, head * D + first_col + c * 32, row0);
          tma_store_commit();
        }
      };
      {
        uint32_t o[PB][32];
#pragma unroll
        for (int c = 0; c < PB; ++c) B200_TMEM_LD_32(o[c], tmem_dP + lane_addr + c * 32);
        tmem_ld_wait();
        to_boxes(o);
      }
      {
        uint32_t o[PB][32];  // the second half waits in registers: the tensor-memory columns are free from here on
#pragma unroll
        for (int c = 0; c < PB; ++c) B200_TMEM_LD_32(o[c], tmem_dP + lane_addr + (PB + c) * 32);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(&bars[B_DQ_DRAINED]);
        reduce(0);  // may block while the engine's queue is full: only after the columns have been handed back
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        to_boxes(o);
        reduce(PB * 32);
      }
      if (++qt == n_q_tiles) {
        qt = first_q_tile;
        ++qh;
      }
    }
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- P / dS producers, dQ drain, final dK / dV
    const int q4 = warp & 3;            // TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;   // which part of the columns (of S^T / dP^T, dQ, dK, dV) this warp takes
    const int st = threadIdx.x - 64;    // 0 .. SOFTMAX_THREADS - 1
    const int r = q4 * 32 + lane;  // key row inside the tile (S^T, dV, dK) / query row inside the tile (dQ)
    const int kv_local = kv0 + r;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    const bool kv_valid = kv_local < doc_len;
    const float2 scale_log2_2 = make_float2(scale_log2, scale_log2), scale_2 = make_float2(scale, scale);
    constexpr int OUT_CHUNKS = D / 32;  // 32-column chunks of dQ / dK / dV, dealt to the parts round-robin
    bool ok = true;

    // Per-query statistics of a step for buffer (step & 1): thread st < 128 fetches lse, st < 256 delta. Kept negated
    // (and delta pre-multiplied by the softmax scale) so that each element below is one fused multiply-add. The fetch is
    // issued a phase before its value is stored, so that nobody waits for the trip to global memory at the barrier.
    auto fetch_row = [&](int head, int q0) -> float {  // the raw value: nothing here waits for the load
      if (st >= 2 * BT) return 0.f;
      const int ql = min(q0 + (st & (BT - 1)), doc_len - 1);
      return __ldg((st < BT ? lse : delta) + (long long)head * T + doc_start + ql);
    };
    auto stage_rows = [&](int buf, int q0, float raw) {
      if (st >= 2 * BT) return;
      float value = st < BT ? raw * -1.4426950408889634f : raw * -scale;
      if (q0 + (st & (BT - 1)) >= doc_len) value = st < BT ? -INFINITY : 0.f;
      s_rows[buf * (2 * BT) + st] = value;
    };

    // (head, query tile) of the current step, advanced without divisions
    int qh = 0, qt = first_q_tile;
    // The statistics of step i are published through the mbarrier B_ROWS (completion i): written by all arithmetic
    // threads, step 0 here and step i + 1 at the start of dS(i), when every thread is known to have finished dS(i - 1),
    // the last reader of that buffer (dP(i) is issued only after dS(i - 1) of all threads has been consumed by dQ(i - 1)).
    if (n_iter > 0) stage_rows(0, qt * BT, fetch_row(grp * qpg, qt * BT));
    mbar_arrive(&bars[B_ROWS]);
    const bool tr = tracing && st == 0;
    long long tw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t0 = 0;
    const long long t_begin = tr ? clock64() : 0;

    bool got = true;  // false once one of this thread's waits gave up
    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = qt * BT;
      int next_qh = qh, next_qt = qt + 1;
      if (next_qt == n_q_tiles) {
        next_qt = first_q_tile;
        ++next_qh;
      }
      uint32_t pp[PART_CHUNKS * 16];  // P^T of this step, this thread's query columns as bf16 pairs (kept from P to dS)
      const float next_row = it + 1 < n_iter ? fetch_row(grp * qpg + next_qh, next_qt * BT) : 0.f;
      {
        // ------------------------------------------------ P(it) from S(it)
        const float* w_lse = s_rows + (it & 1) * (2 * BT) + part * PART_COLS;
        // Only the diagonal tile and the last key tile of a document mask anything: every other tile takes the short path.
        const bool masked = !kv_valid || (causal && (q0 < kv0 + BT - 1));
        const int first_visible = kv_valid ? (causal ? kv_local - q0 : 0) : BT;  // query columns below this see nothing of this key
        if (tr) t0 = clock64();
        if (!mbar_wait(&bars[B_S_FULL], it & 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
          got = false;
        }
        if (got && !mbar_wait(&bars[B_ROWS], it & 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
          got = false;
        }
        if (tr) { tw[0] += clock64() - t0; t0 = clock64(); }
        tc_fence_after_sync();
#pragma unroll
        for (int cc = 0; cc < PART_CHUNKS; ++cc) {
          const int col0 = part * PART_COLS + cc * 32;  // first query column of this chunk
          uint32_t sv[32];
          B200_TMEM_LD_32(sv, tmem_S + lane_addr + col0);
          tmem_ld_wait();
          const float4* nl4 = reinterpret_cast<const float4*>(w_lse + cc * 32);
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float4 nl = nl4[e / 4];
            // packed fp32 pairs: t = s * scale*log2e - lse*log2e
            const float2 t0v = __ffma2_rn(make_float2(__uint_as_float(sv[e]), __uint_as_float(sv[e + 1])), scale_log2_2, make_float2(nl.x, nl.y));
            const float2 t1v = __ffma2_rn(make_float2(__uint_as_float(sv[e + 2]), __uint_as_float(sv[e + 3])), scale_log2_2, make_float2(nl.z, nl.w));
            float2 p0 = make_float2(fast_exp2(t0v.x), fast_exp2(t0v.y));
            float2 p1 = make_float2(fast_exp2(t1v.x), fast_exp2(t1v.y));
            if (masked) {
              const int col = col0 + e;  // query column inside the tile
              if (col < first_visible) p0.x = 0.f;
              if (col + 1 < first_visible) p0.y = 0.f;
              if (col + 2 < first_visible) p1.x = 0.f;
              if (col + 3 < first_visible) p1.y = 0.f;
            }
            pp[cc * 16 + e / 2] = pack_bf16x2(p0.x, p0.y);
            pp[cc * 16 + e / 2 + 1] = pack_bf16x2(p1.x, p1.y);
          }
          // over columns this thread has already read: the stores fill the first half of the part's columns
          B200_TMEM_ST_16(tmem_S + lane_addr + part * PART_COLS + cc * 16, pp + cc * 16);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&bars[B_P_READY]);
        if (tr) { tw[1] += clock64() - t0; t0 = clock64(); }
      }
      {
        // ------------------------------------------------ dS(it) from dP(it) and the P kept in registers
        const float* w_delta = s_rows + (it & 1) * (2 * BT) + BT + part * PART_COLS;
        if (!mbar_wait(&bars[B_DP_FULL], it & 1, abort_flag)) {
          raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
          got = false;
        }
        if (tr) { tw[5] += clock64() - t0; t0 = clock64(); }
        tc_fence_after_sync();
        if (it + 1 < n_iter) {
          stage_rows((it + 1) & 1, next_qt * BT, next_row);
          mbar_arrive(&bars[B_ROWS]);
        }
#pragma unroll
        for (int cc = 0; cc < PART_CHUNKS; ++cc) {
          const int c = (part * PART_COLS) / 32 + cc;  // 32-column chunk of the tile
          uint32_t dpv[32];
          B200_TMEM_LD_32(dpv, tmem_dP + lane_addr + c * 32);
          tmem_ld_wait();
          uint32_t dd[16];
          const float4* nd4 = reinterpret_cast<const float4*>(w_delta + cc * 32);
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float4 nd = nd4[e / 4];
            // g = dP * scale - delta * scale
            const float2 g0 = __ffma2_rn(make_float2(__uint_as_float(dpv[e]), __uint_as_float(dpv[e + 1])), scale_2, make_float2(nd.x, nd.y));
            const float2 g1 = __ffma2_rn(make_float2(__uint_as_float(dpv[e + 2]), __uint_as_float(dpv[e + 3])), scale_2, make_float2(nd.z, nd.w));
            const float2 d0 = __fmul2_rn(unpack_bf16x2(pp[cc * 16 + e / 2]), g0), d1 = __fmul2_rn(unpack_bf16x2(pp[cc * 16 + e / 2 + 1]), g1);
            dd[e / 2] = pack_bf16x2(d0.x, d0.y);
            dd[e / 2 + 1] = pack_bf16x2(d1.x, d1.y);
          }
          // 32 columns = half of a 64-column K block: four 16-byte chunks of this thread's row
          uint8_t* drow = sDS + (c >> 1) * (BT * 128) + r * 128;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const int chunk = ((c & 1) * 4 + ch) ^ (r & 7);
            *reinterpret_cast<uint4*>(drow + chunk * 16) = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[B_DS_READY]);
        if (tr) { tw[7] += clock64() - t0; t0 = clock64(); }
      }
      if (!got) break;  // this thread's wait gave up and raised the flag: the other threads' waits end on it
      qh = next_qh;
      qt = next_qt;
    }
    if (tr) {
      for (int i = 0; i < 8; ++i) trace_out[i] = tw[i];
      trace_out[8] = clock64() - t_begin;
    }
    // dK / dV are complete when the last dK has been committed (the MMAs retire in order)
    if (ok && got && !mbar_wait(&bars[B_Q_EMPTY + ((n_iter - 1) & 1)], ((n_iter - 1) >> 1) & 1, abort_flag)) got = false;
    ok = ok && got;
    if (!ok) {
      raise_status(status, kStatusWaitTimeoutEpilogue, abort_flag);
    } else {
      // dK and dV of this key tile (all MMAs retired: dQ of the last step was committed after them)
      tc_fence_after_sync();
      __nv_bfloat16* krow = dqkv + (long long)(doc_start + kv_local) * dqkv_stride + k_col;
      __nv_bfloat16* vrow = krow + D;
#pragma unroll
      for (int c = part; c < OUT_CHUNKS; c += PARTS) {
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
                float scale, bool causal, int* status, long long* trace, cudaStream_t stream) {
  auto kernel = trace != nullptr ? attn_bwd_kernel<D, true> : attn_bwd_kernel<D, false>;
  static bool configured[2] = {false, false};
  if (!configured[trace != nullptr]) {
    check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::TOTAL), "attn_bwd smem attr");
    configured[trace != nullptr] = true;
  }
  const int tiles_upper = (T + BT - 1) / BT + num_docs;
  dim3 grid(groups, tiles_upper);
  kernel<<<grid, BWD_THREADS, BwdSmem<D>::TOTAL, stream>>>(tm_qkv, tm_do, tm_dq, lse, delta,
                                                           reinterpret_cast<__nv_bfloat16*>(dqkv), dqkv_stride, cu_seqlens,
                                                           num_docs, T, groups, qpg, scale, scale * 1.4426950408889634f,
                                                           causal ? 1 : 0, status, trace);
  check_cuda(cudaGetLastError(), "attn_bwd launch");
}

long long* g_trace = nullptr;

}  // namespace

// 16 cycle counters of the first CTA of every following backward launch are written to `words` (nullptr: off).
void attn_bwd_set_trace(long long* words) { g_trace = words; }

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
  const CUtensorMap tm_dq = make_tensor_map_2d_f32(dq_accum, (long long)hq * head_dim, T, (long long)hq * head_dim, 32, 32);
  if (head_dim == 128) launch_bwd<128>(tm_qkv, tm_do, tm_dq, lse, delta, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, causal, status, g_trace, stream);
  else if (head_dim == 64) launch_bwd<64>(tm_qkv, tm_do, tm_dq, lse, delta, dqkv, dqkv_stride, cu_seqlens, num_docs, T, groups, qpg, scale, causal, status, g_trace, stream);
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

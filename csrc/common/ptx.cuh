// Blackwell (sm_100a) device primitives used by every kernel in this tree:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// (TMEM allocation, UMMA issue, commit, TMEM loads/stores) and bounded waits.
//
// Every wait on an mbarrier is bounded: after `kSpinLimit` polls the waiter
// records a status word and returns false so that the kernel can unwind
// (drain its own copies, free TMEM, return) instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Status codes written to the per-launch status word (0 = ok).
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeoutProducer = 1,
  kStatusWaitTimeoutMma = 2,
  kStatusWaitTimeoutEpilogue = 3,
  kStatusWaitTimeoutPeer = 4,
  kStatusBadArgument = 5,
};

// Poll budget of a bounded wait. mbarrier.try_wait itself blocks for a
// hardware-defined slice of time, so this is on the order of seconds.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false when the budget ran out or when another role of
// the CTA already raised `*abort_flag` (a word in shared memory).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void raise_status(int* status, int code, volatile int* abort_flag) {
  *abort_flag = 1;
  if (status != nullptr) atomicCAS(status, 0, code);
}

// 2^x on the special-function unit: one instruction, no range fix-ups (denormal results flush to zero).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 1 / x on the special-function unit (one instruction, about 1 ulp).
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies). Loads complete on an mbarrier of this CTA.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* desc, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* desc, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* desc, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

// Element-wise add of a shared-memory tile into global memory (element type taken from the tensor map).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* desc, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

// Barrier `id` (1..15) over `nthreads` threads of the CTA that also returns the OR of `pred` over them: every
// participant learns whether any of them gave up a bounded wait, so that all of them leave a loop together.
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %3, 0;\n"
      "bar.red.or.pred q, %1, %2, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}"
      : "=r"(r)
      : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory + UMMA
// ----------------------------------------------------------------------------
// Allocate `ncols` (power of two, 32..512) TMEM columns; the base address is
// written to `*smem_result`. Must be executed by one whole warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on `bar` once all tcgen05.mma issued so far by this thread retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; bf16/fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; 8-bit float inputs (e4m3 / e5m2), fp32 accumulate.
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor of kind::f16 with bf16 operands and fp32 accumulator.
// a_mn / b_mn: 0 = operand is K-major in shared memory, 1 = MN-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int a_mn, int b_mn) {
  return (1u << 4)                      // accumulator format: f32
         | (1u << 7)                    // A format: bf16
         | (1u << 10)                   // B format: bf16
         | (uint32_t(a_mn) << 15)       // A major
         | (uint32_t(b_mn) << 16)       // B major
         | (uint32_t(n >> 3) << 17)     // N / 8
         | (uint32_t(m >> 4) << 24);    // M / 16
}

// Instruction descriptor of kind::f8f6f4 with fp32 accumulator. a_fmt / b_fmt: 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t umma_idesc_f8(int m, int n, int a_fmt, int b_fmt, int a_mn, int b_mn) {
  return (1u << 4) | (uint32_t(a_fmt) << 7) | (uint32_t(b_fmt) << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) |
         (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//  K-major : rows of 64 bf16 (128 B); 8-row groups `sbo_bytes` apart (1024 for a dense tile).
//  MN-major: K-rows of 64 bf16 along MN (128 B); 8-K-row groups `sbo_bytes` apart,
//            64-wide MN blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;  // descriptor version of this architecture
  d |= uint64_t(2) << 61;  // 128-byte swizzle
  return d;
}

// TMEM address = (lane << 16) | column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

#define B200_TMEM_LD_32(ARR, ADDR)                                                                                  \
  asm volatile(                                                                                                     \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                     \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                     \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                     \
      : "=r"((ARR)[0]), "=r"((ARR)[1]), "=r"((ARR)[2]), "=r"((ARR)[3]), "=r"((ARR)[4]), "=r"((ARR)[5]),             \
        "=r"((ARR)[6]), "=r"((ARR)[7]), "=r"((ARR)[8]), "=r"((ARR)[9]), "=r"((ARR)[10]), "=r"((ARR)[11]),           \
        "=r"((ARR)[12]), "=r"((ARR)[13]), "=r"((ARR)[14]), "=r"((ARR)[15]), "=r"((ARR)[16]), "=r"((ARR)[17]),       \
        "=r"((ARR)[18]), "=r"((ARR)[19]), "=r"((ARR)[20]), "=r"((ARR)[21]), "=r"((ARR)[22]), "=r"((ARR)[23]),       \
        "=r"((ARR)[24]), "=r"((ARR)[25]), "=r"((ARR)[26]), "=r"((ARR)[27]), "=r"((ARR)[28]), "=r"((ARR)[29]),       \
        "=r"((ARR)[30]), "=r"((ARR)[31])                                                                            \
      : "r"(ADDR)                                                                                                   \
      : "memory")

#define B200_TMEM_ST_32(ADDR, ARR)                                                                                  \
  asm volatile(                                                                                                     \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                               \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                                    \
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                            \
      :                                                                                                             \
      : "r"(ADDR), "r"((ARR)[0]), "r"((ARR)[1]), "r"((ARR)[2]), "r"((ARR)[3]), "r"((ARR)[4]), "r"((ARR)[5]),        \
        "r"((ARR)[6]), "r"((ARR)[7]), "r"((ARR)[8]), "r"((ARR)[9]), "r"((ARR)[10]), "r"((ARR)[11]), "r"((ARR)[12]), \
        "r"((ARR)[13]), "r"((ARR)[14]), "r"((ARR)[15]), "r"((ARR)[16]), "r"((ARR)[17]), "r"((ARR)[18]),             \
        "r"((ARR)[19]), "r"((ARR)[20]), "r"((ARR)[21]), "r"((ARR)[22]), "r"((ARR)[23]), "r"((ARR)[24]),             \
        "r"((ARR)[25]), "r"((ARR)[26]), "r"((ARR)[27]), "r"((ARR)[28]), "r"((ARR)[29]), "r"((ARR)[30]),             \
        "r"((ARR)[31])                                                                                              \
      : "memory")

#define B200_TMEM_ST_16(ADDR, ARR)                                                                                  \
  asm volatile(                                                                                                     \
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                               \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                                    \
      :                                                                                                             \
      : "r"(ADDR), "r"((ARR)[0]), "r"((ARR)[1]), "r"((ARR)[2]), "r"((ARR)[3]), "r"((ARR)[4]), "r"((ARR)[5]),        \
        "r"((ARR)[6]), "r"((ARR)[7]), "r"((ARR)[8]), "r"((ARR)[9]), "r"((ARR)[10]), "r"((ARR)[11]), "r"((ARR)[12]), \
        "r"((ARR)[13]), "r"((ARR)[14]), "r"((ARR)[15])                                                              \
      : "memory")

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}

// sigmoid and SiLU with the approximate exponential and reciprocal (two MUFU operations and two FMA-pipe operations per
// value instead of an IEEE division); every kernel that evaluates SwiGLU uses these, so that a fused epilogue and the
// stand-alone kernel produce the same bits.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float silu_fast(float x) { return x * sigmoid_fast(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace b200

// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the triangle-attention
// kernels use: mbarrier, TMA tiled loads, tcgen05 tensor-memory allocation, MMA, load/store.
// Every wait is bounded: a wait that runs out of time records a status and returns false,
// and the kernel then tears down (frees its tensor memory) and exits.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace oops_ta {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival per warp: every lane has finished its part (the caller has run the fences it needs), lane 0 arrives.
// Barriers that warps arrive on are initialised with the number of warps, not threads.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
constexpr uint32_t kSuspendHintNs = 20000;  // 20 us per probe; the bounded wait below re-probes until its own limit
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  // The suspend-time hint lets the hardware park the warp until the phase completes (or the hint expires)
  // instead of returning at once, so a waiting warp does not burn issue slots of the warps that compute.
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
      : "memory");
  return done != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any thread of the CTA has given up, the
// others stop waiting too.  Returns false if the wait was abandoned.
constexpr uint64_t kWaitLimitNs = 250000000ull;  // 0.25 s

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t start = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x7) == 0) {
      if (*abort_flag != 0) return false;
      if (globaltimer_ns() - start > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Non-blocking probe of a phase.  Several probes issued back to back overlap their trips to the barrier words; a
// waiter that finds every phase complete (the steady state of a pipeline whose consumer is the slow side) pays one
// round trip for all of them instead of one each.  `mbar_wait_probed` falls back to the bounded wait.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_probed(bool complete, uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return complete ? true : mbar_wait(bar, parity, abort_flag);
}

// The bounded wait run by every lane of a warp; the lanes leave converged with one warp-uniform answer.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok) != 0;
}

// 16-byte chunk `c` of a 128-byte row in a 128-byte-swizzled tile.  The hardware stores chunk c of row r at chunk
// c ^ (r & 7); `row_x` is the (128-byte aligned) row address plus the thread's own term ((r & 7) ^ c0) << 4, so that
// the chunk c0 + c (c < 8, c0 a multiple of the unrolled range) costs one XOR with an immediate.
__device__ __forceinline__ const uint8_t* swizzled_chunk(const uint8_t* row_x, int c) {
  return reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(row_x) ^ uintptr_t(c << 4));
}

// ---- loads that stay where they are written ---------------------------------------------------------
// A prefetch of next step's operand only hides latency if the load issues before this step's work.  The compiler
// may sink an ordinary load to its first use (it does when registers are tight); a volatile asm load keeps its
// place among the other volatile statements (barrier waits, tensor-memory loads).
__device__ __forceinline__ float ldg_f32_here(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_u8_here(const uint8_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Four f32 added to global memory without a return value (performed at the L2; nothing to wait for).
__device__ __forceinline__ void red_add_f4(float4* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// Four words from global memory past the L1 (data another thread of the CTA has written or added to).
__device__ __forceinline__ float4 ldcg_f4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// Four words from shared memory, requested where the statement stands; the result is not waited for until it is used.
__device__ __forceinline__ uint4 lds_v4_here(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
  return v;
}

// Four words from global memory when `take` is set, zeros otherwise; like the loads above it keeps its place and its
// result is not touched before the caller uses it.
__device__ __forceinline__ uint4 ldg_v4_here_if(const void* p, bool take) {
  uint4 v;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.u32 p, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\t"
      "mov.u32 %1, 0;\n\t"
      "mov.u32 %2, 0;\n\t"
      "mov.u32 %3, 0;\n\t"
      "@p ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n\t"
      "}\n"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "r"(uint32_t(take)));
  return v;
}

// ---- proxies and fences ------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- TMA: tiled 5-D load global -> shared, completion on an mbarrier ---------------------------
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------------------
// One warp allocates `cols` (a power of two >= 32) columns; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by one thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]; issued by one thread.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same products issued by a CONVERGED warp: every lane runs the surrounding code, `elect.sync` picks the one lane
// that executes the instruction.  The operand descriptors are then warp-uniform values the compiler keeps in uniform
// registers, where code under `if (lane == 0)` computes them per thread and moves every operand across (six moves per
// product): measured on a B200, a step of 28 products issues in 43 instead of 59 clocks per product.
__device__ __forceinline__ void mma_ss_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_warp(uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(bar)
      : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory operand descriptor (sm_100 format): start address, leading/stride byte offsets
// (all in 16-byte units), descriptor version 1, swizzle mode in bits 61-63.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle) {
  return uint64_t((addr & 0x3ffff) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) |
         (uint64_t(1) << 46) | (swizzle << 61);
}

// Instruction descriptor for kind::f16: f32 accumulate, A/B format (0 = f16, 1 = bf16), majors
// (0 = K-major, 1 = MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t ab_format, uint32_t a_major, uint32_t b_major, uint32_t m,
                                                  uint32_t n) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_major << 15) | (b_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// 32 lanes x 32 columns of 32-bit words: thread i of the warp receives lane (base + i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
      "%25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16-column variants of the above.
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 8-column load.
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(addr)
               : "memory");
}
// 4-column load.
__device__ __forceinline__ void tmem_ld4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(addr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The registers a tensor-memory load fills are plain asm outputs: nothing ties their readers to the wait above, and
// the compiler may schedule arithmetic on them before it.  Passing them through an empty volatile statement placed
// after the wait (volatile statements keep their order) makes every later reader depend on it; it emits no code.
template <int N>
__device__ __forceinline__ void tmem_loaded(uint32_t (&r)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(r[i]));
}

// ---- math ---------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Packed pairs of f32 (Blackwell executes fma/add/mul on a pair as one instruction).  The compiler's own
// float2 intrinsics are used so that register pairs are allocated without extra moves.
typedef float2 f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  lo = v.x;
  hi = v.y;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { return __fmul2_rn(a, b); }

// fma with the result clamped to [0, 1] (a NaN or -inf input gives 0).
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
  float d;
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^(128 u + kExp2PolyLow) for a pair of u in [0, 1], computed on the FMA pipe instead of the special-function unit
// (which serves 16 `ex2` per clock per SM and is the first pipe to saturate at head size 32).  The caller obtains u
// from its exponent x with one saturating multiply-add, u = sat((x - low) / 128), which also clamps x to
// [low, low + 128].  w = 128 u is split by the round-to-nearest of a large-constant add into an integer n and a
// remainder f in [-1/2, 1/2]; 2^f is a degree-3 polynomial (relative error 7.5e-5, below the 16-bit rounding the
// result gets before its MMA); n + low goes into the exponent field with one shift-add per element.
constexpr int kExp2PolyLow = -120;  // results span 2^-120 .. 2^8: exponents above the running maximum by the lazy-rescale slack fit
__device__ __forceinline__ f32x2 ex2_poly_unit(f32x2 u) {
  constexpr float magic = 12582912.f + float(kExp2PolyLow);  // 1.5 * 2^23 + low: the sum's low mantissa bits hold n + low
  const f32x2 scale128 = pack2(128.f, 128.f), magic2 = pack2(magic, magic);
  const f32x2 r = fma2(u, scale128, magic2);
  const f32x2 minus_n = fma2(r, pack2(-1.f, -1.f), magic2);
  const f32x2 f = fma2(u, scale128, minus_n);
  f32x2 poly = fma2(f, pack2(0.0551716685f, 0.0551716685f), pack2(0.2426111251f, 0.2426111251f));
  poly = fma2(poly, f, pack2(0.6932609677f, 0.6932609677f));
  poly = fma2(poly, f, pack2(0.9999280572f, 0.9999280572f));
  float r_lo, r_hi, p_lo, p_hi;
  unpack2(r, r_lo, r_hi);
  unpack2(poly, p_lo, p_hi);
  return pack2(__int_as_float(__float_as_int(p_lo) + (__float_as_int(r_lo) << 23)),
               __int_as_float(__float_as_int(p_hi) + (__float_as_int(r_hi) << 23)));
}

template <typename T>
struct Half2;
template <>
struct Half2<__nv_bfloat16> {
  static constexpr uint32_t kFormat = 1;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  __device__ static __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
  __device__ static __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
  __device__ static __forceinline__ f32x2 widen(uint32_t v) { return pack2(lo(v), hi(v)); }
};
template <>
struct Half2<__half> {
  static constexpr uint32_t kFormat = 0;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  __device__ static __forceinline__ float lo(uint32_t v) {
    return __half2float(__ushort_as_half((unsigned short)(v & 0xffffu)));
  }
  __device__ static __forceinline__ float hi(uint32_t v) { return __half2float(__ushort_as_half((unsigned short)(v >> 16))); }
  __device__ static __forceinline__ f32x2 widen(uint32_t v) { return pack2(lo(v), hi(v)); }
};

}  // namespace ptx
}  // namespace oops_ta

// Thin inline-PTX layer for the Blackwell (sm_100a) features the kernels use: mbarrier with
// transaction counts, TMA (cp.async.bulk[.tensor]), tensor memory (tcgen05.alloc/ld/st) and
// tcgen05.mma with shared-memory or tensor-memory operands.  Every wait is bounded.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace xqt_b200 {
namespace sm100 {

constexpr uint32_t kSpinLimit = 1u << 22;  // try_wait attempts before a wait gives up (each returns within about a microsecond)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// try_wait WITHOUT a suspend-time hint.  With a hint (tens of microseconds) the wait is compiled into a
// test / nanosleep back-off loop whose wake-up lags the barrier by up to a microsecond; in producer/consumer
// rings whose stages last a few hundred nanoseconds that lag set the pace (measured: the fused W4A16 GEMM
// 198 -> 171 us, its K-split form 132 -> 96 us from this change alone).
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test.  try_wait may suspend the thread for a while when the phase is not complete (measured: about 800
// cycles per unsuccessful call); a look-ahead poll that expects "not yet" as a normal answer must use this form.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// false when the attempt limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Two barriers at once.  A try_wait takes about 150 cycles to return its predicate even when the
// phase has already completed, but independent ones pipeline: polling both in one go costs one
// round trip instead of two.
__device__ __forceinline__ bool mbar_try_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
      "and.pred p, p, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar_a), "r"(parity_a), "r"(bar_b), "r"(parity_b)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait2(bar_a, parity_a, bar_b, parity_b)) return true;
  return false;
}

// ---------------------------------------------------------------- programmatic dependent launch
// No-ops when the kernel was launched without the programmatic-serialization attribute.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// 2-D tiled load, coordinates (c0 = innermost element index, c1 = row); c0 * element size must be a
// multiple of 16 bytes
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// ask for `bytes` (a multiple of 16, from a 16-byte aligned address) to be brought into L2; no
// destination, no completion to wait for
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
  return r;
}
// Cluster-wide barrier in its split form.  Every thread of every CTA of the cluster takes part in
// each phase; the hardware schedules the CTAs of a cluster together, so the wait cannot outlast them.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// address of this CTA's shared-memory location `saddr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t caddr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(caddr), "f"(v) : "memory");
}

// ---------------------------------------------------------------- wide loads
// 32 bytes per thread from global memory that is read once: no L1 allocation, first in line for
// L2 eviction.  The address must be 32-byte aligned.
__device__ __forceinline__ void ldg256_stream(uint32_t (&r)[8], const void* p) {
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p));
}
__device__ __forceinline__ void ldg128_stream(uint32_t (&r)[4], const void* p) {
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "l"(p));
}
__device__ __forceinline__ uint32_t ldg32_stream(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];\n" : "=r"(r) : "l"(p));
  return r;
}
__device__ __forceinline__ void ldg64_stream(uint32_t (&r)[2], const void* p) {
  asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "l"(p));
}

// ---------------------------------------------------------------- tensor memory
// allocate `cols` (power of two >= 32) columns; the base address is written to *slot (shared)
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// wait::ld tied to the registers of the preceding tcgen05.ld, so that no use of them can be
// scheduled ahead of the wait
__device__ __forceinline__ void tmem_wait_ld_dep(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// this warp's 32 lanes x 32 consecutive 32-bit columns -> 32 registers (thread = lane = row)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 32 columns in the accumulator-fragment distribution (shape 16x256b, four times along the columns):
// lane t of the warp holds rows t/4 and t/4 + 8 (relative to the lane in taddr) and, of every 8-column group j, the
// columns 2*(t%4) and 2*(t%4)+1: r[4j+0..1] = row t/4, r[4j+2..3] = row t/4 + 8
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 registers -> this warp's 32 lanes x 32 columns
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 4 registers -> this warp's 32 lanes x 4 columns
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory operand, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
// (what a TMA box of 128 bytes x R rows with CU_TENSOR_MAP_SWIZZLE_128B writes).  The tile must be
// 1024-byte aligned; advancing along K inside the 128-byte row adds the byte offset to the start.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                          // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtU8 = 0, kFmtS8 = 1, kAccF32 = 1, kAccS32 = 2 };

// instruction descriptor: dense, K-major A and B, no negation
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t acc_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
  return (acc_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
template <bool I8>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// D[tmem] (+)= A[smem] * B[smem] with 8-bit floating operands (kind::f8f6f4; formats in the descriptor:
// E4M3 = 0, E5M2 = 1), fp32 accumulators; issued by ONE thread
enum : uint32_t { kFmtE4M3 = 0, kFmtE5M2 = 1 };
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// a pair of fp32 values in one 64-bit register (shuffled as one value in the W4A4 store epilogue)
__device__ __forceinline__ unsigned long long f32x2_pack(float lo, float hi) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void f32x2_unpack(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
// packed fp32 arithmetic: one instruction for two lanes of a register pair (round to nearest, as the scalar forms)
__device__ __forceinline__ unsigned long long f32x2_mul(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ unsigned long long f32x2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long f32x2_add(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// One K block of four SS MMA steps (descriptors a0..a3 / b0..b3), its commit to `done_bar`, and --
// issued first, consumed last -- one poll of `next_bar` (a non-blocking test_wait: try_wait would suspend the issuer
// when the next stage has not landed yet): the 150-cycle round trip of the poll runs while the MMAs are being issued.  Returns whether `next_bar` had completed `next_parity`.
// `first_accumulate` is the accumulate flag of the first step; the other three always accumulate.
template <bool I8>
__device__ __forceinline__ bool umma_ss_x4_commit_poll(uint32_t d_tmem, uint64_t a0, uint64_t b0, uint32_t idesc,
                                                        uint32_t first_accumulate, uint32_t done_bar, uint32_t next_bar,
                                                        uint32_t next_parity) {
  uint32_t ok;
  if (I8) {
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t.reg .b64 a, b;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%6], %7;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%1], %2, %3, %8, p;\n\t"
        "add.u64 a, %2, 2;\n\tadd.u64 b, %3, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%1], a, b, %8, t;\n\t"
        "add.u64 a, %2, 4;\n\tadd.u64 b, %3, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%1], a, b, %8, t;\n\t"
        "add.u64 a, %2, 6;\n\tadd.u64 b, %3, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%1], a, b, %8, t;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}\n"
        : "=r"(ok)
        : "r"(d_tmem), "l"(a0), "l"(b0), "r"(first_accumulate), "r"(done_bar), "r"(next_bar), "r"(next_parity), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, q, t;\n\t.reg .b64 a, b;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%6], %7;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %8, p;\n\t"
        "add.u64 a, %2, 2;\n\tadd.u64 b, %3, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %8, t;\n\t"
        "add.u64 a, %2, 4;\n\tadd.u64 b, %3, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %8, t;\n\t"
        "add.u64 a, %2, 6;\n\tadd.u64 b, %3, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %8, t;\n\t"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}\n"
        : "=r"(ok)
        : "r"(d_tmem), "l"(a0), "l"(b0), "r"(first_accumulate), "r"(done_bar), "r"(next_bar), "r"(next_parity), "r"(idesc)
        : "memory");
  }
  return ok != 0;
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

}  // namespace sm100
}  // namespace xqt_b200

// W4A16 decode (M <= 16) with the inner product on tcgen05: the Blackwell-native form of the
// persistent stream-K decode kernel.
//
// Roles inside the one CTA per SM (19 warps, 608 threads):
//   warps 0-15   four dequantisation warpgroups.  Thread (warp % 4, lane) owns output channel
//                32*(warp%4)+lane of the 128-channel tile -- the same index as its tensor-memory
//                lane.  A unit is 64 K of the 128 channels; warpgroup w takes unit w of every 256-K
//                stage.  Per unit a thread reads its 32 packed bytes from the shared-memory stage,
//                turns the nibbles into exact bf16/fp16 integers (code - zero point: shift, lop3 and
//                one packed subtraction per pair), stores them to tensor memory as the A operand
//                (one tcgen05.st of 32 columns), and two units later drains the 16 fp32 results of
//                that unit and folds them into its 16 running sums with the group scale:
//                y[m] += s * sum_k x[m,k] (q[k] - z).
//   warp 16      producer: per stage one bulk copy of the weights (16 KiB), one of the scales and
//                zero points, one tiled TMA load of the activations [16 x 256] into the
//                128-byte-swizzled layout tcgen05 reads (rows >= M arrive as zeros).
//   warps 17-18  MMA issuers, one per pair of warpgroups: M=128 x N=16 x K=16 tcgen05.mma steps
//                with A from tensor memory and B (activations) from shared memory, committed to
//                mbarriers.
// Measured on B200, and what the structure follows from: one tcgen05.mma costs its issuing thread
// about 44 cycles whatever its shape up to N=64 (27 when two threads issue), so a stage of 16 steps
// needs two issuers; an mbarrier try_wait returns its predicate after about 150 cycles even when
// the phase is complete, but independent polls pipeline, so every wait is one poll of everything
// the step needs and only lane 0 of a warp polls; the loop is instruction-bound (about 340
// warp-instructions per unit), hence four warpgroups and no divisions or generic loads inside it.
// The kernel is launched with programmatic stream serialization: it lets the next kernel of the
// stream start its set-up and weight prefetch early, and itself touches data of the previous
// kernel (activations, scratch, outputs) only after griddepcontrol.wait.
// The dequantised weight is an exact small integer, the scale is applied in fp32 to the fp32 group
// sum, so the result equals the contract reference (xqt/kernels/ops/gemm/reference.py:263-271,527)
// up to fp32 summation order.  Zero points must be integers in [0, 119] (true of every RTN / AWQ
// checkpoint); other weights are served by the mma.sync decode kernel.
// Stream-K partition, partial-sum scratch, ticket-elected finisher and bounded waits are those of
// w4a16_decode.cu.
#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

namespace dtc {
constexpr int kTileRows = 128;
constexpr int kStageK = 256;
constexpr int kUnitK = 64;                                 // K per unit: 32 tensor-memory columns, four MMA steps
constexpr int kUnitsPerStage = kStageK / kUnitK;           // 4
constexpr int kWG = 4;                                     // dequantisation warpgroups
constexpr int kUnitsPerWg = kUnitsPerStage / kWG;          // units of a stage per warpgroup
constexpr int kDequantThreads = kWG * 128;
constexpr int kMmaWarps = 2;                               // each issues for kWG / kMmaWarps warpgroups
constexpr int kProducerWarp = kWG * 4;
constexpr int kFirstMmaWarp = kProducerWarp + 1;
constexpr int kThreads = (kWG * 4 + 1 + kMmaWarps) * 32;
constexpr int kWBytes = 128 * kStageK / 2;   // 16 KiB
constexpr int kXBytes = 16 * kStageK * 2;    // 8 KiB: four 64-K atoms of [16 rows x 128 B]
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 216 * 1024;
constexpr int kPartialFloats = 16 * kTileRows;
constexpr int kRedFloats = (kWG - 1) * kPartialFloats;
constexpr int kMaxTiles = 8192;
constexpr int kMaxGrid = 256;
constexpr uint32_t kTmemCols = 512;
enum Status : unsigned int { kTimeout = 32 };
constexpr int kNB = 2;   // tensor-memory buffers (A operand + result) per warpgroup
constexpr int kColsPerWg = kNB * (kUnitK / 2 + 16);
static_assert(kWG * kColsPerWg <= (int)kTmemCols, "tensor memory budget");
static_assert(kWG == 2 * kMmaWarps && kUnitsPerWg == 1, "each MMA issuer serves a pair of warpgroups, one unit each per stage");
__host__ __device__ constexpr uint32_t a_col(int wg, int buf) { return wg * kColsPerWg + buf * (kUnitK / 2); }
__host__ __device__ constexpr uint32_t d_col(int wg, int buf) { return wg * kColsPerWg + kNB * (kUnitK / 2) + buf * 16; }
}  // namespace dtc

struct DecodeTcParams {
  const uint8_t* wt;   // [tiles][K/128][4 chunks][128 channels][16 B]
  const uint8_t* sz;   // [tiles][K/128][128/g][128][2] param dtype
  const float* bias;
  const void* residual;
  void* out;
  int m, n, k;
  int out_f32;         // 1: output is fp32 [M,N] (partial sums of a K-sharded layer), else T
  int tiles, spt;
  long long total;
  int nstages, stage_bytes, sz_stage_bytes;
  float* partials;
  unsigned int* tickets;
  unsigned int* status;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void dq_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(dtc::kDequantThreads) : "memory"); }

template <typename T>
struct TcTraits;
template <>
struct TcTraits<__half> {
  using h2 = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;
  static constexpr float kBase = 1024.f;
  static constexpr uint32_t kFmt = kFmtF16;
  static __device__ __forceinline__ uint32_t pair(float v) {
    __half2 h = __float2half2_rn(v);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct TcTraits<__nv_bfloat16> {
  using h2 = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;
  static constexpr float kBase = 128.f;
  static constexpr uint32_t kFmt = kFmtBF16;
  static __device__ __forceinline__ uint32_t pair(float v) {
    __nv_bfloat162 h = __float2bfloat162_rn(v);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

// nibbles i (low half) and i (high half) of `word` as the exact 16-bit integers code - zero
template <typename T>
__device__ __forceinline__ uint32_t dq_col(uint32_t word, int i, uint32_t off2, uint32_t magic) {
  using Tr = TcTraits<T>;
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(word >> (4 * i)), "n"(0x000f000f), "r"(magic));
  typename Tr::h2 v = __hsub2(*reinterpret_cast<typename Tr::h2*>(&r), *reinterpret_cast<const typename Tr::h2*>(&off2));
  return *reinterpret_cast<uint32_t*>(&v);
}

// shared-memory loads by 32-bit shared address (the stage pointers are computed, so generic loads
// would be emitted otherwise)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
// (scale, zero point) pair of one channel and group
template <typename P>
__device__ __forceinline__ void load_scale_zero(uint32_t addr, float& sc, float& zp);
template <>
__device__ __forceinline__ void load_scale_zero<__nv_bfloat16>(uint32_t addr, float& sc, float& zp) {
  const uint32_t v = lds32(addr);
  sc = __uint_as_float(v << 16);
  zp = __uint_as_float(v & 0xffff0000u);
}
template <>
__device__ __forceinline__ void load_scale_zero<__half>(uint32_t addr, float& sc, float& zp) {
  const uint32_t v = lds32(addr);
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
  sc = f.x;
  zp = f.y;
}
template <>
__device__ __forceinline__ void load_scale_zero<float>(uint32_t addr, float& sc, float& zp) {
  sc = __uint_as_float(lds32(addr));
  zp = __uint_as_float(lds32(addr + 4));
}

// a / b for non-negative operands; `small` (uniform) says both fit 32 bits, which avoids the long
// software routine of the 64-bit division
__device__ __forceinline__ long long div_nn(long long a, long long b, bool small) {
  return small ? (long long)((uint32_t)a / (uint32_t)b) : a / b;
}
__device__ __forceinline__ int cta_of_stage(long long x, long long total, int grid, bool small) {
  return (int)div_nn((x + 1) * grid - 1, total, small);
}

// GK: quantisation group size (128 or 64)
template <typename T, typename P, bool SIGNED, int GK>
__global__ void __launch_bounds__(dtc::kThreads, 1)
w4a16_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const DecodeTcParams p) {
  using namespace dtc;
  using Tr = TcTraits<T>;
  constexpr uint32_t kIdesc = umma_idesc(kAccF32, Tr::kFmt, Tr::kFmt, 128, 16);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + kWG * kNB + kMmaWarps * kNB];
  __shared__ uint32_t s_tmem_base;
  __shared__ unsigned int s_flag;
  __shared__ volatile unsigned int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const bool small = p.total * (long long)(grid + 1) < 0x7fffffffLL;
  const long long s_begin = div_nn((long long)cta * p.total, grid, small), s_end = div_nn((long long)(cta + 1) * p.total, grid, small);
  const int ns = p.nstages;
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(stages + (size_t)ns * p.stage_bytes);   // [kWG-1][16][128] fp32
  auto full_bar = [&](int s) { return smem_addr(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_addr(&bars[kMaxStages + s]); };
  auto aready_bar = [&](int wg, int b) { return smem_addr(&bars[2 * kMaxStages + wg * kNB + b]); };
  // results ready: one barrier per MMA issuer (pair of warpgroups) and buffer
  auto dready_bar = [&](int wg, int b) { return smem_addr(&bars[2 * kMaxStages + kWG * kNB + (wg >> 1) * kNB + b]); };

  // Producer state (used by one thread): running (tile, stage-in-tile, ring slot, ring phase) so that
  // the loop has no divisions.
  const uint32_t tx = kWBytes + kXBytes + p.sz_stage_bytes;
  const long long units_per_tile = p.k / 128;
  long long pr_tile = 0;
  int pr_ks = 0, pr_slot = 0;
  uint32_t pr_phase = 0;
  // weights and scales of the next stage (they never depend on an earlier kernel) ...
  auto issue_weights = [&]() {
    unsigned char* st = stages + (size_t)pr_slot * p.stage_bytes;
    const long long unit = pr_tile * units_per_tile + (long long)pr_ks * 2;   // first (tile, 128-K block)
    mbar_expect_tx(full_bar(pr_slot), tx);
    bulk_g2s(smem_addr(st + kXBytes), p.wt + unit * 8192, kWBytes, full_bar(pr_slot));
    bulk_g2s(smem_addr(st + kXBytes + kWBytes), p.sz + unit * (p.sz_stage_bytes / 2), p.sz_stage_bytes, full_bar(pr_slot));
  };
  // ... and its activations, which may be the output of the kernel before this one
  auto issue_acts = [&](int slot, int ks) {
    tma_load_3d(smem_addr(stages + (size_t)slot * p.stage_bytes), &tm_x, 0, 0, ks * 4, full_bar(slot));
  };
  auto advance = [&]() {
    if (++pr_ks == p.spt) { pr_ks = 0; ++pr_tile; }
    if (++pr_slot == ns) { pr_slot = 0; pr_phase ^= 1; }
  };
  uint32_t pr_it = 0;

  if (tid == kProducerWarp * 32) {
    // The same thread initialises the barriers and at once requests the first stage, so that the
    // first weights are on their way while the other warps are still setting up.
    s_abort = 0u;
    for (int i = 0; i < ns; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), kMmaWarps);   // one tcgen05.commit per MMA issuer
    }
    for (int wg = 0; wg < kWG; ++wg)
      for (int b = 0; b < kNB; ++b) {
        mbar_init(aready_bar(wg, b), 4);                      // one arrival per warp of the warpgroup
        if ((wg & 1) == 0) mbar_init(dready_bar(wg, b), 1);   // tcgen05.commit
      }
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
    pr_tile = div_nn(s_begin, p.spt, small);
    pr_ks = (int)(s_begin - pr_tile * p.spt);
    if (s_begin < s_end) {   // the first weights go out before the CTA-wide barrier, the rest right after it
      issue_weights();
    }
  }
  if (warp == kFirstMmaWarp) {
    tmem_alloc(smem_addr(&s_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  // Programmatic dependent launch: the next kernel of the stream may start its own set-up and
  // weight prefetch as soon as every CTA here has passed this point; everything of this kernel
  // that reads or writes data of the previous one comes after the dependency wait (the producer
  // thread waits later, after it has requested its first weights).
  grid_launch_dependents();
  if (tid != kProducerWarp * 32) grid_dependency_wait();

  // Waits: the first poll is the fast path; the abort flag is consulted only when a wait has to spin,
  // so that after one timeout the remaining waits of the CTA fall through quickly.
  auto guarded_wait = [&](uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return;
    if (s_abort == 0u && !mbar_wait(bar, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };
  auto guarded_wait2 = [&](uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b) {
    if (mbar_try_wait2(bar_a, parity_a, bar_b, parity_b)) return;
    if (s_abort == 0u && !mbar_wait2(bar_a, parity_a, bar_b, parity_b)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      // Fill the ring with weights first: under programmatic dependent launch this kernel may have
      // started while the one before it (which may produce the activations) is still running.
      const int ks0 = pr_ks;
      long long s = s_begin;
      for (; s < s_end && pr_it < (uint32_t)ns; ++s, ++pr_it) {
        if (pr_it != 0) issue_weights();   // stage 0 went out before the barrier
        advance();
      }
      grid_dependency_wait();
      for (int j = 0, ks = ks0; j < (int)pr_it; ++j) {
        issue_acts(j, ks);
        if (++ks == p.spt) ks = 0;
      }
      for (; s < s_end; ++s, ++pr_it) {
        guarded_wait(empty_bar(pr_slot), pr_phase ^ 1);
        issue_weights();
        issue_acts(pr_slot, pr_ks);
        advance();
      }
    }
  } else if (warp >= kFirstMmaWarp) {
    // ------------------------------------------------------------------ MMA issuers
    if (elect_one()) {
      const int wg0 = (warp - kFirstMmaWarp) * 2;   // the pair of warpgroups served
      uint32_t it = 0;
      int slot = 0;
      // No wait on the stage's own barrier: a warpgroup signals its unit only after it has seen the
      // stage complete, and the activations arrive under the same barrier as the weights.
      for (long long s = s_begin; s < s_end; ++s, ++it) {
        const uint32_t xbase = smem_addr(stages + (size_t)slot * p.stage_bytes);
        const int buf = it & (kNB - 1);
        const uint32_t bphase = (it / kNB) & 1;
        guarded_wait2(aready_bar(wg0, buf), bphase, aready_bar(wg0 + 1, buf), bphase);
        tc_fence_after();
        // The instruction rate, not the arithmetic, bounds these M=128 x N=16 x K=16 steps (each
        // moves 4 KiB of A operand); the two units are interleaved only to keep the order fixed.
#pragma unroll
        for (int kk = 0; kk < kUnitK / 16; ++kk) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int wg = wg0 + j;                     // 64-K unit of the stage == its swizzle atom
            const uint64_t bdesc = umma_desc_sw128(xbase + wg * 2048 + kk * 32);
            umma_ts_f16(tmem_base + d_col(wg, buf), tmem_base + a_col(wg, buf) + kk * 8, bdesc, kIdesc, kk != 0 ? 1u : 0u);
          }
        }
        umma_commit(dready_bar(wg0, buf));
        umma_commit(empty_bar(slot));   // this issuer's reads of the stage (activations) are done; the weights
                                        // were consumed by the threads before they signalled the units ready
        if (++slot == ns) slot = 0;
      }
    }
  } else {
    // ------------------------------------------------------------------ dequantisation warpgroups
    const int wg = warp >> 2, quarter = warp & 3;
    const int ch = quarter * 32 + lane;                 // channel inside the tile == tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    // Units of this warpgroup alternate between two tensor-memory buffers.  Up to two units are
    // outstanding (stored, their MMAs possibly still running); the older one is folded into acc at
    // the start of the next unit, a whole unit after it was handed to the MMA issuer.
    uint32_t iw = 0;             // units issued
    uint32_t drained = 0;        // units folded into acc
    float s_even = 0.f, s_odd = 0.f;   // scales of the outstanding units, by buffer

    // fold unit `drained` into acc; `waited` says its barrier has already been observed
    auto drain = [&](bool waited) {
      const uint32_t j = drained;
      const int b = j & (kNB - 1);
      if (!waited) guarded_wait(dready_bar(wg, b), (j / kNB) & 1);
      tc_fence_after();
      uint32_t r[16];
      tmem_ld_32x16(tmem_base + lane_addr + d_col(wg, b), r);
      tmem_wait_ld_dep(r);
      const float sc = b == 0 ? s_even : s_odd;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(sc, __uint_as_float(r[i]), acc[i]);
      ++drained;
    };

    const uint32_t stages_s = smem_addr(stages);
    // the magic exponent pattern lives in a register the compiler cannot re-create per use
    uint32_t magic;
    asm volatile("mov.b32 %0, %1;\n" : "=r"(magic) : "n"(Tr::kMagic));
    long long tile = div_nn(s_begin, p.spt, small);
    int ks = (int)(s_begin - tile * p.spt);
    int slot = 0;
    uint32_t phase = 0, it = 0;
    // the (at most two) tiles this CTA shares with other CTAs: who contributes, and in which of its
    // two partial-sum slots the first contributor keeps this tile
    struct Edge { long long tile; int c_first, c_last, first_seg; };
    auto make_edge = [&](long long t) {
      Edge e;
      e.tile = t;
      const long long t_first = t * p.spt;
      e.c_first = cta_of_stage(t_first, p.total, grid, small);
      e.c_last = cta_of_stage(t_first + p.spt - 1, p.total, grid, small);
      e.first_seg = (div_nn((long long)e.c_first * p.total, grid, small) == t_first) ? 0 : 1;
      return e;
    };
    const Edge edge_a = make_edge(tile), edge_b = make_edge(div_nn(s_end - 1, p.spt, small));
    for (long long s = s_begin; s < s_end; ++s, ++it) {
      const uint32_t st_s = stages_s + (uint32_t)slot * (uint32_t)p.stage_bytes;
      // one poll for both things this unit needs: the stage, and (two units later) the results of
      // the unit whose tensor-memory buffers it will reuse
      // Lane 0 polls for its warp (512 threads polling the same barriers queue up behind one another),
      // the warp barrier hands the observation to the other lanes.
      const bool due = iw - drained >= (uint32_t)kNB;
      if (lane == 0) {
        if (due) guarded_wait2(full_bar(slot), phase, dready_bar(wg, drained & (kNB - 1)), (drained / kNB) & 1);
        else guarded_wait(full_bar(slot), phase);
      }
      __syncwarp();
      if (++slot == ns) { slot = 0; phase ^= 1; }
#pragma unroll
      for (int uu = 0; uu < kUnitsPerWg; ++uu) {
        if (due) drain(true);                            // frees the buffers the new unit will use
        const int u = uu * kWG + wg;                     // 64-K unit of the stage handled by this warpgroup
        const int kb = u >> 1;                           // its 128-K block
        const int sub = GK == 64 ? (u & 1) : 0;          // its group inside the block
        // scale and zero point of (channel, group)
        float sc, zp;
        load_scale_zero<P>(st_s + kXBytes + kWBytes + (uint32_t)(((kb * (128 / GK) + sub) * kTileRows + ch) * 2 * sizeof(P)), sc, zp);
        const uint32_t off2 = Tr::pair(Tr::kBase + zp + (SIGNED ? 8.f : 0.f));
        // packed weights: [kblock][chunk][channel][16 B]; a chunk is 32 K, a unit two chunks
        const uint32_t wsrc = st_s + kXBytes + (uint32_t)(((kb * 4 + (u & 1) * 2) * kTileRows + ch) * 16);
        const uint4 v0 = lds128(wsrc);
        const uint4 v1 = lds128(wsrc + kTileRows * 16);
        const uint32_t words[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const int buf = iw & (kNB - 1);
        uint32_t cols[32];
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          const uint32_t word = SIGNED ? (words[w] ^ 0x88888888u) : words[w];
#pragma unroll
          for (int i = 0; i < 4; ++i) cols[w * 4 + i] = dq_col<T>(word, i, off2, magic);
        }
        tmem_st_32x32(tmem_base + lane_addr + a_col(wg, buf), cols);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(aready_bar(wg, buf));
        if (buf == 0) s_even = sc; else s_odd = sc;
        ++iw;
      }
      const bool tile_end = (ks == p.spt - 1);
      const long long cur_tile = tile;
      if (++ks == p.spt) { ks = 0; ++tile; }
      if (!tile_end && s != s_end - 1) continue;

      // ---------------------------------------------------------------- end of this CTA's run in `tile`
      while (drained < iw) drain(false);
      // combine the warpgroups' sums (fixed order)
      if (wg != 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) red[((wg - 1) * 16 + i) * kTileRows + ch] = acc[i];
      }
      dq_sync();
      if (wg == 0) {
#pragma unroll
        for (int g = 0; g < kWG - 1; ++g) {
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] += red[(g * 16 + i) * kTileRows + ch];
        }
      }
      const bool at_a = cur_tile == edge_a.tile, at_b = cur_tile == edge_b.tile;
      const int c_first = at_a ? edge_a.c_first : (at_b ? edge_b.c_first : cta);
      const int c_last = at_a ? edge_a.c_last : (at_b ? edge_b.c_last : cta);
      const int first_seg = at_a ? edge_a.first_seg : edge_b.first_seg;
      bool finish = true;
      if (c_first != c_last) {
        const int seg = at_a ? 0 : 1;
        float* mine = p.partials + ((size_t)cta * 2 + seg) * kPartialFloats;
        if (wg == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < p.m) mine[i * kTileRows + ch] = acc[i];
        }
        dq_sync();
        if (tid == 0) {
          __threadfence();   // cumulative: publishes the partial sums the barrier has ordered before it
          s_flag = atomicAdd(&p.tickets[cur_tile], 1u);
        }
        dq_sync();
        finish = (s_flag == (unsigned int)(c_last - c_first));
        if (finish) {
          __threadfence();
          // the warpgroups add interleaved contributors (always in the same order), then combine
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = 0.f;
          // two contributors per batch: all their loads are in flight before the first add
          for (int c0 = c_first + wg; c0 <= c_last; c0 += 2 * kWG) {
            float v[2][16];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const int c = c0 + kWG * b;
              const int cseg = c == c_first ? first_seg : 0;   // later contributors begin inside the tile
              const float* src = p.partials + ((size_t)c * 2 + cseg) * kPartialFloats;
#pragma unroll
              for (int i = 0; i < 16; ++i) v[b][i] = (c <= c_last && i < p.m) ? __ldcg(src + i * kTileRows + ch) : 0.f;
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] += v[b][i];
            }
          }
          if (wg != 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) red[((wg - 1) * 16 + i) * kTileRows + ch] = acc[i];
          }
          dq_sync();
          if (wg == 0) {
#pragma unroll
            for (int g = 0; g < kWG - 1; ++g) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] += red[(g * 16 + i) * kTileRows + ch];
            }
          }
          if (tid == 0) p.tickets[cur_tile] = 0u;
        }
      }
      if (finish && wg == 0) {
        const long long chn = cur_tile * kTileRows + ch;
        if (chn < p.n) {
          T* out = reinterpret_cast<T*>(p.out);
          const T* res = reinterpret_cast<const T*>(p.residual);
          const float b = p.bias != nullptr ? p.bias[chn] : 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (i < p.m) {
              float v = acc[i] + b;
              const size_t o = (size_t)i * p.n + chn;
              if (res != nullptr) v += to_float<T>(res[o]);
              if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = v;
              else out[o] = from_float<T>(v);
            }
          }
        }
      }
      // `red` is reused at the next tile end: nobody may overwrite it before warpgroup 0 has read it
      dq_sync();
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kFirstMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// --------------------------------------------------------------------------------------- host side

int make_tile_map_x3d(CUtensorMap* map, const void* base, int is_bf16, int m, int k);  // below

static int dtc_sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  return v;
}

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// activations [M, K] 16-bit row-major seen as [K/64 atoms][M rows][64 elements]; box = 4 atoms x 16 rows
int make_tile_map_x3d(CUtensorMap* map, const void* base, int is_bf16, int m, int k) {
  static EncodeTiledFn3 fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (int)cudaErrorNotSupported;
    fn = reinterpret_cast<EncodeTiledFn3>(sym);
  }
  cuuint64_t dims[3] = {64, (cuuint64_t)m, (cuuint64_t)(k / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)k * 2, 128};
  cuuint32_t box[3] = {64, 16, 4};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

size_t w4a16_decode_tc_workspace_bytes() {
  using namespace dtc;
  return 256 + (size_t)kMaxTiles * sizeof(unsigned int) + (size_t)kMaxGrid * 2 * kPartialFloats * sizeof(float);
}

bool w4a16_decode_tc_supported(int m, int n, int k, int group_size) {
  using namespace dtc;
  return m >= 1 && m <= 16 && n >= 1 && k >= kStageK && k % kStageK == 0 && (group_size == 64 || group_size == 128) &&
         ceil_div(n, kTileRows) <= kMaxTiles;
}

// XQT_B200_PDL=0 in the environment launches the kernel without the programmatic-dependency
// attribute (the in-kernel dependency instructions are then no-ops).
static bool dependent_launch_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* v = getenv("XQT_B200_PDL");
    state = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return state == 1;
}

template <typename T, typename P>
static int dtc_launch(const CUtensorMap& tm, const DecodeTcParams& p, int group_size, bool is_signed, int grid,
                      size_t smem_bytes, cudaStream_t stream) {
#define XQT_DTC(SG, GKV)                                                                                     \
  do {                                                                                                       \
    auto kern = w4a16_decode_tc_kernel<T, P, SG, GKV>;                                                       \
    XQT_SMEM_OPT_IN(kern, dtc::kSmemBudget);                                                                 \
    cudaLaunchConfig_t cfg = {};                                                                             \
    cfg.gridDim = dim3((unsigned)grid);                                                                      \
    cfg.blockDim = dim3(dtc::kThreads);                                                                      \
    cfg.dynamicSmemBytes = smem_bytes;                                                                       \
    cfg.stream = stream;                                                                                     \
    cudaLaunchAttribute attr[1];                                                                             \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                         \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                                  \
    cfg.attrs = attr;                                                                                        \
    cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;                                                       \
    XQT_CUDA(cudaLaunchKernelEx(&cfg, kern, tm, p));                                                         \
  } while (0)
  if (group_size == 128) {
    if (is_signed) XQT_DTC(true, 128); else XQT_DTC(false, 128);
  } else {
    if (is_signed) XQT_DTC(true, 64); else XQT_DTC(false, 64);
  }
#undef XQT_DTC
  return launch_status();
}

int w4a16_decode_tc_launch(const void* x, const void* wt, const void* sz, const float* bias, const void* residual,
                           void* out, int m, int n, int k, int group_size, int nibble_signed, int act_dtype,
                           int param_dtype, int out_f32, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  using namespace dtc;
  XQT_REQUIRE(w4a16_decode_tc_supported(m, n, k, group_size));
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= w4a16_decode_tc_workspace_bytes());
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)wt & 15) == 0 && ((uintptr_t)sz & 15) == 0);
  CUtensorMap tm;
  {
    const int rc = make_tile_map_x3d(&tm, x, act_dtype == XQT_B200_BF16, m, k);
    if (rc != 0) return rc;
  }
  const int psize = param_dtype == XQT_B200_FP32 ? 4 : 2;
  DecodeTcParams p;
  p.wt = (const uint8_t*)wt; p.sz = (const uint8_t*)sz; p.bias = bias; p.residual = residual; p.out = out;
  p.m = m; p.n = n; p.k = k; p.out_f32 = out_f32;
  XQT_REQUIRE(!out_f32 || residual == nullptr);
  p.tiles = ceil_div(n, kTileRows);
  p.spt = k / kStageK;
  p.total = (long long)p.tiles * p.spt;
  p.sz_stage_bytes = 2 * (128 / group_size) * kTileRows * 2 * psize;
  p.stage_bytes = (kXBytes + kWBytes + p.sz_stage_bytes + 1023) / 1024 * 1024;
  int ns = (kSmemBudget - 1024 - kRedFloats * 4) / p.stage_bytes;
  p.nstages = ns > kMaxStages ? kMaxStages : ns;
  XQT_REQUIRE(p.nstages >= 2);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<unsigned int*>(ws);
  p.tickets = reinterpret_cast<unsigned int*>(ws + 256);
  p.partials = reinterpret_cast<float*>(ws + 256 + (size_t)kMaxTiles * sizeof(unsigned int));
  long long grid = dtc_sm_count();
  if (grid > kMaxGrid) grid = kMaxGrid;
  if (grid > p.total) grid = p.total;
  const size_t smem_bytes = (size_t)p.nstages * p.stage_bytes + kRedFloats * 4 + 1024;
  const bool sg = nibble_signed != 0;
  if (act_dtype == XQT_B200_BF16) {
    if (param_dtype == XQT_B200_BF16) return dtc_launch<__nv_bfloat16, __nv_bfloat16>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
    if (param_dtype == XQT_B200_FP16) return dtc_launch<__nv_bfloat16, __half>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
    return dtc_launch<__nv_bfloat16, float>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
  }
  if (param_dtype == XQT_B200_BF16) return dtc_launch<__half, __nv_bfloat16>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
  if (param_dtype == XQT_B200_FP16) return dtc_launch<__half, __half>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
  return dtc_launch<__half, float>(tm, p, group_size, sg, (int)grid, smem_bytes, stream);
}

}  // namespace xqt_b200

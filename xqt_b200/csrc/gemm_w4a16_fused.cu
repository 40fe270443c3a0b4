// Fused W4A16 GEMM for 17 <= M <= 512 tokens on tcgen05:
//   Y[M,N] = X[M,K] * dequant(W)[N,K]^T, weights read straight from the canonical xqt_int4_nk_v1 bytes and
// dequantised in registers on their way to the tensor core -- no N*K*2 scratch, no second pass.
//
// A CTA tile is 128 output channels x up to 256 tokens (MT = 1 or 2 blocks of 128 rows that share ONE
// dequantised weight tile): for M <= 256 every packed weight is read and converted exactly once per call; a
// larger M is cut into 256-token chunks.  Per 64-K stage
//   * TMA brings the activation blocks [MT x 128 x 64] fp16 (128-byte swizzle) and, through a deeper ring
//     of its own, the packed weights of the stage (128 rows x 32 bytes, plain layout);
//   * eight dequantisation warps turn the nibbles into fp16 values (code - zero) * scale -- the zero point
//     folded into the exact magic-number subtraction, one rounding in the multiply -- and store them in the
//     128-byte-swizzled K-major layout tcgen05 reads.  They work as four groups of two warps, group g on the
//     stages it = g (mod 4), a thread on two weight rows: converting a stage is a chain of waits (two barrier
//     tests of ~200 cycles, the scale loads, the proxy fence) that one warp cannot overlap with itself, so four
//     stages are in conversion at any time;
//   * one thread issues 4 x MT MMAs (K = 16, kind::f16, fp32 accumulators in tensor memory, 128 columns per
//     token block, the tile's accumulators double-buffered so the epilogue overlaps the next tile).
// Warps (480 threads): 0 activation producer, 1 MMA issuer, 2-5 epilogue, 6-13 dequantisation, 14 packed-weight
// producer.  What the pipeline's rate depended on, measured with cycle stamps (down projection 4096 x 14336 at M = 64:
// 76 -> 43 us; gate/up 28672 x 4096: 133 -> 63 us): the packed-weight ring needs a producer of its own (one thread
// feeding both rings in order tied weights to the activation ring's waits); the conversion waits for the stage to be
// FREE, not for its activations; look-ahead polls use mbarrier.test_wait (try_wait on an incomplete phase suspends
// the thread for ~800 cycles) and the MMA issuer polls after issuing; parameter prefetches keep raw bits (converting
// them at once waits for the load); ring slots and phases are kept incrementally (`it % stages` is a division).
// Few channel tiles (a down projection: N = 4096 is 32 tiles for 148 SMs) are split over K: every split
// stores its fp32 partial tile, takes a ticket, and the CTA that draws the last ticket adds the partials in
// split order (bit-reproducible) and runs the epilogue -- nobody waits for anybody.
//
// Precision: as the two-pass form -- fp16 operands (bf16 activations are converted once per call; range
// violations set a status bit), weights rounded once to fp16, fp32 accumulation.  Envelope: group size 64 or
// 128, K a multiple of 64, N a multiple of 8, integer zero points (or none).  Reference arithmetic:
// xqt/kernels/ops/gemm/reference.py:263-271,527; it replaces the reference's fused HMMA kernels
// (csrc/quantization/w4a16_fused_kernel.cu) on this range of M.
#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows);
int make_byte_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows);

namespace w4f {
constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kFirstEpiWarp = 2, kEpiWarps = 4, kFirstDqWarp = 6, kDqWarps = 8;
constexpr int kDqGroups = 4, kDqGroupWarps = kDqWarps / kDqGroups;   // stage it is converted by warp group it % kDqGroups
constexpr int kRawWarp = kFirstDqWarp + kDqWarps;          // producer of the packed-weight ring (a warp of its own)
constexpr int kThreads = (kRawWarp + 1) * 32;              // 480
constexpr int kMaxStages = 6, kMaxRaw = 8;
constexpr int kABlockBytes = kBM * 128, kBBytes = kBN * 128;
constexpr int kRawBytes = kBN * (kBK / 2);                  // 4 KiB of packed nibbles per stage
constexpr int kSmemBudget = 226 * 1024;
enum Status : unsigned int { kTimeout = 48 };
constexpr int kBarFull = 0, kBarReady = kBarFull + kMaxStages, kBarEmpty = kBarReady + kMaxStages;
constexpr int kBarRawFull = kBarEmpty + kMaxStages, kBarRawEmpty = kBarRawFull + kMaxRaw;
constexpr int kBarTileFull = kBarRawEmpty + kMaxRaw, kBarTileEmpty = kBarTileFull + 2, kBarCount = kBarTileEmpty + 2;
}  // namespace w4f

struct W4FusedParams {
  int m, n, k, group_size, groups;
  int mchunks, ntiles, splits, kb_per_split, kblocks, stages, raw_bufs;
  int param_dtype, nibble_signed, out_f32;
  const void* scales;
  const void* zeros;
  const float* bias;
  const void* residual;
  void* out;
  float* partials;          // [tiles][splits][MT*128][128] fp32 (splits > 1)
  unsigned int* tickets;    // [tiles], zero between calls
  unsigned int* status;
};

template <typename OutT>
__device__ __forceinline__ void w4f_store8(OutT* dst, const float (&v)[8]);
template <>
__device__ __forceinline__ void w4f_store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void w4f_store8<__half>(__half* dst, const float (&v)[8]) {
  uint4 o;
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <typename T>
__device__ __forceinline__ void w4f_load8(const T* src, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = to_float<T>(e[i]);
}

// 8 nibbles of `word` (k0..k7, canonical order) -> fp16 (code - zero) * scale as 4 registers in K order
__device__ __forceinline__ uint4 w4f_dequant_word(uint32_t word, __half2 off2, __half2 scale2) {
  uint32_t d[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(word >> (4 * i)), "n"(0x000f000f), "n"(0x64006400));
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&r), off2), scale2);   // (k_i, k_{i+4})
    d[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  uint4 o;
  o.x = __byte_perm(d[0], d[1], 0x5410);   // (k0, k1)
  o.y = __byte_perm(d[2], d[3], 0x5410);   // (k2, k3)
  o.z = __byte_perm(d[0], d[1], 0x7632);   // (k4, k5)
  o.w = __byte_perm(d[2], d[3], 0x7632);   // (k6, k7)
  return o;
}

// tile -> (token chunk, channel tile, K split); the splits of one output tile are adjacent CTAs
struct W4FTile {
  int mc, nt, sp, kb0, kbn, out_tile;
};
__device__ __forceinline__ W4FTile w4f_tile(const W4FusedParams& p, int tile) {
  W4FTile t;
  t.sp = tile % p.splits;
  t.out_tile = tile / p.splits;
  t.mc = t.out_tile % p.mchunks;
  t.nt = t.out_tile / p.mchunks;
  t.kb0 = t.sp * p.kb_per_split;
  const int left = p.kblocks - t.kb0;
  t.kbn = left < p.kb_per_split ? left : p.kb_per_split;
  return t;
}

// Position in a ring of `n` slots that is walked in fixed steps: slot index and phase parity kept incrementally (a
// runtime `it % n` / `it / n` pair per stage is two integer divisions on every role's critical path).
struct W4FRing {
  uint32_t slot, phase, n;
  __device__ __forceinline__ W4FRing(uint32_t start, uint32_t slots) : slot(start % slots), phase((start / slots) & 1u), n(slots) {}
  __device__ __forceinline__ void advance(uint32_t step) {
    slot += step;
    while (slot >= n) { slot -= n; phase ^= 1u; }
  }
};

template <int MT, typename T>
__global__ void __launch_bounds__(w4f::kThreads, 1)
gemm_w4a16_fused_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                        const __grid_constant__ W4FusedParams p) {
  using namespace w4f;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[kBarCount];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;
  __shared__ unsigned int s_ticket;

  constexpr int kABytes = MT * kABlockBytes, kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTileCols = MT * kBN;              // accumulator columns of one tile
  constexpr uint32_t kTmemCols = 2 * kTileCols;         // double-buffered: 256 or 512
  constexpr uint32_t kIdesc = umma_idesc(kAccF32, kFmtF16, kFmtF16, kBM, kBN);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ns = p.stages, nr = p.raw_bufs;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  unsigned char* raw_base = tiles + (size_t)ns * kStageBytes;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };

  if (threadIdx.x == 0) {
    s_abort = 0u;
    for (int s = 0; s < ns; ++s) {
      mbar_init(bar(kBarFull + s), 1);
      mbar_init(bar(kBarReady + s), kDqGroupWarps);
      mbar_init(bar(kBarEmpty + s), 1);
    }
    for (int r = 0; r < nr; ++r) {
      mbar_init(bar(kBarRawFull + r), 1);
      mbar_init(bar(kBarRawEmpty + r), kDqGroupWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(kBarTileFull + b), 1);
      mbar_init(bar(kBarTileEmpty + b), kEpiWarps);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_addr(&s_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = p.mchunks * p.ntiles * p.splits;

  // Every wait is bounded: when one runs out the CTA stops waiting anywhere, reports and drains out.
  auto guarded_wait = [&](uint32_t b, uint32_t parity) {
    if (s_abort == 0u && !mbar_wait(b, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };
  auto guarded_wait2 = [&](uint32_t b0, uint32_t parity0, uint32_t b1, uint32_t parity1) {
    if (s_abort == 0u && !mbar_wait2(b0, parity0, b1, parity1)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer of the activation blocks
    if (elect_one()) {
      W4FRing st_ring(0, ns);
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const W4FTile t = w4f_tile(p, tile);
        for (int kb = 0; kb < t.kbn; ++kb, st_ring.advance(1)) {
          const int s = st_ring.slot;
          guarded_wait(bar(kBarEmpty + s), st_ring.phase ^ 1);
          unsigned char* st = tiles + (size_t)s * kStageBytes;
          mbar_expect_tx(bar(kBarFull + s), kABytes);
#pragma unroll
          for (int mb = 0; mb < MT; ++mb)      // a block past the last token row is filled with zeros
            tma_load_2d(smem_addr(st + mb * kABlockBytes), &tm_a, (t.kb0 + kb) * kBK, (t.mc * MT + mb) * kBM, bar(kBarFull + s));
        }
      }
    }
  } else if (warp == kRawWarp) {
    // ---------------------------------------------------------------- TMA producer of the packed weights
    // A warp of its own: the weight ring runs as far ahead of the conversion as it has slots, whatever the activation
    // ring is waiting for (one thread feeding both rings in order tied the weights of step j to the stage of step j - 2).
    if (elect_one()) {
      const uint32_t raw_addr = smem_addr(raw_base);
      W4FRing raw_ring(0, nr);
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const W4FTile t = w4f_tile(p, tile);
        for (int kb = 0; kb < t.kbn; ++kb, raw_ring.advance(1)) {
          const int r = raw_ring.slot;
          guarded_wait(bar(kBarRawEmpty + r), raw_ring.phase ^ 1);
          mbar_expect_tx(bar(kBarRawFull + r), kRawBytes);
          tma_load_2d(raw_addr + (uint32_t)r * kRawBytes, &tm_w, (t.kb0 + kb) * (kBK / 2), t.nt * kBN, bar(kBarRawFull + r));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t local = 0;
      W4FRing cur(0, ns), nxt(1, ns);
      bool ready = false;          // the current stage's barrier has already been seen complete
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const W4FTile t = w4f_tile(p, tile);
        const int buf = local & 1;
        guarded_wait(bar(kBarTileEmpty + buf), ((local >> 1) & 1) ^ 1);
        tc_fence_after();
        for (int kb = 0; kb < t.kbn; ++kb, cur.advance(1), nxt.advance(1)) {
          const int s = cur.slot;
          // both operands of the stage: the weights dequantised (Ready) and the activation blocks landed (Full); the
          // dequantisation warps do not wait for the activations, only for the stage to be free
          if (!ready) guarded_wait2(bar(kBarReady + s), cur.phase, bar(kBarFull + s), cur.phase);
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t bdesc = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int mb = 0; mb < MT; ++mb) {
            const uint64_t adesc = umma_desc_sw128(a_addr + mb * kABlockBytes);
            const uint32_t d_tmem = tmem_base + buf * kTileCols + mb * kBN;
#pragma unroll
            for (int q = 0; q < 4; ++q) umma_ss<false>(d_tmem, adesc + 2 * q, bdesc + 2 * q, kIdesc, (kb != 0 || q != 0) ? 1u : 0u);
          }
          umma_commit(bar(kBarEmpty + s));
          // the next stage's barriers, tested without blocking after this stage's MMAs are on their way
          ready = mbar_test_wait(bar(kBarReady + nxt.slot), nxt.phase) && mbar_test_wait(bar(kBarFull + nxt.slot), nxt.phase);
        }
        umma_commit(bar(kBarTileFull + buf));
      }
    }
  } else if (warp < kFirstDqWarp) {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;
    const int et = threadIdx.x - kFirstEpiWarp * 32;      // 0..127
    T* out = reinterpret_cast<T*>(p.out);
    const T* res = reinterpret_cast<const T*>(p.residual);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const W4FTile t = w4f_tile(p, tile);
      const int buf = local & 1;
      const int n0 = t.nt * kBN;
      guarded_wait(bar(kBarTileFull + buf), (local >> 1) & 1);
      tc_fence_after();
      float* part = p.partials + ((size_t)t.out_tile * p.splits + t.sp) * (MT * kBM * kBN);
      // finished values of one row segment: bias, residual, rounding, store
      auto finish8 = [&](int row, int col, float (&v)[8]) {
        if (p.bias != nullptr) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += __ldg(p.bias + col + e);
        }
        if (res != nullptr) {
          float rv[8];
          w4f_load8<T>(res + (size_t)row * p.n + col, rv);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += rv[e];
        }
        if (p.out_f32) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)row * p.n + col);
          dst[0] = make_float4(v[0], v[1], v[2], v[3]);
          dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
          w4f_store8<T>(out + (size_t)row * p.n + col, v);
        }
      };
#pragma unroll 1
      for (int mb = 0; mb < MT; ++mb) {
        const int row_in_tile = mb * kBM + quarter * 32 + lane;
        const int row = t.mc * (MT * kBM) + row_in_tile;
        const uint32_t taddr = tmem_base + buf * kTileCols + mb * kBN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_wait_ld();
          if (p.splits > 1) {
            float4* dst = reinterpret_cast<float4*>(part + (size_t)row_in_tile * kBN + c * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          } else if (row < p.m) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + c * 32 + j * 8;
              if (col < p.n) {   // N is a multiple of 8
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
                finish8(row, col, v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarTileEmpty + buf));      // the accumulators are free for the tile after next
      if (p.splits > 1) {
        // ticket: the CTA whose partial tile is stored last adds all of them, in split order
        __threadfence();
        asm volatile("bar.sync 1, %0;\n" ::"n"(kEpiWarps * 32) : "memory");
        if (et == 0) s_ticket = atomicAdd(p.tickets + t.out_tile, 1u);
        asm volatile("bar.sync 1, %0;\n" ::"n"(kEpiWarps * 32) : "memory");
        if (s_ticket == (unsigned int)(p.splits - 1)) {
          __threadfence();
          if (et == 0) p.tickets[t.out_tile] = 0u;               // ready for the next call
          const float* base = p.partials + (size_t)t.out_tile * p.splits * (MT * kBM * kBN);
          // thread et adds 8-column segments: 16 segments per row, MT*128 rows
#pragma unroll 1
          for (int seg = et; seg < MT * kBM * (kBN / 8); seg += kEpiWarps * 32) {
            const int row_in_tile = seg / (kBN / 8), c8 = seg % (kBN / 8);
            const int row = t.mc * (MT * kBM) + row_in_tile, col = n0 + c8 * 8;
            if (row < p.m && col < p.n) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = 0.f;
              for (int sp = 0; sp < p.splits; ++sp) {
                const float4* src = reinterpret_cast<const float4*>(base + (size_t)sp * (MT * kBM * kBN) + (size_t)row_in_tile * kBN + c8 * 8);
                const float4 a = __ldcg(src), b = __ldcg(src + 1);
                v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
              }
              finish8(row, col, v);
            }
          }
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(kEpiWarps * 32) : "memory");   // s_ticket is rewritten by the next tile
      }
    }
  } else {
    // ---------------------------------------------------------------- dequantisation warps
    const int dt = threadIdx.x - kFirstDqWarp * 32;      // 0..255
    const int grp = dt >> 6, row_a = dt & 63;            // group of two warps; the thread's rows are row_a and row_a + 64
    const float zbase = 1024.f + (p.nibble_signed ? 8.f : 0.f);
    // This group converts the steps it = grp, grp + 4, grp + 8, ... of the CTA's run of steps (tiles back to back):
    // ring cursors for its current step and the one after, advanced by kDqGroups; no division in the loop.
    uint32_t it_base = 0;                                // index of the current tile's first step
    W4FRing st_cur(grp, ns), st_nxt(grp + kDqGroups, ns), raw_cur(grp, nr), raw_nxt(grp + kDqGroups, nr);
    const int gshift = p.group_size == 2 * kBK ? 1 : 0;  // quantisation group = one or two 64-K steps
    bool ahead_raw = false, ahead_full = false;          // this group's next stage was already seen ready
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const W4FTile t = w4f_tile(p, tile);
      size_t prow[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        int row = t.nt * kBN + row_a + 64 * rr;
        row = row < p.n ? row : p.n - 1;
        prow[rr] = (size_t)row * p.groups;
      }
      // scale and zero point of this group's next stage, requested one of its stages (four K blocks) ahead: they come
      // from L2 or DRAM, and a stage converted by this group has no other load to hide them behind
      // (as raw bits: converting them here would make the prefetch wait for its own loads, an L2 round trip per stage)
      uint32_t nsc[2] = {0u, 0u}, nzp[2] = {0u, 0u};
      bool have_next = false;
      auto fetch_params = [&](int kb, uint32_t (&sc)[2], uint32_t (&zp)[2]) {
        const int g = (t.kb0 + kb) >> gshift;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          sc[rr] = load_param_bits(p.scales, p.param_dtype, prow[rr] + g);
          zp[rr] = p.zeros != nullptr ? load_param_bits(p.zeros, p.param_dtype, prow[rr] + g) : 0u;
        }
      };
      // the tile's first step of this group: the smallest kb with (it_base + kb) % kDqGroups == grp
      for (int kb = (grp - (int)(it_base % kDqGroups)) & (kDqGroups - 1); kb < t.kbn; kb += kDqGroups,
               st_cur.advance(kDqGroups), st_nxt.advance(kDqGroups), raw_cur.advance(kDqGroups), raw_nxt.advance(kDqGroups)) {
        const int s = st_cur.slot, r = raw_cur.slot;
        uint32_t scb[2], zpb[2];
        if (have_next) {
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) { scb[rr] = nsc[rr]; zpb[rr] = nzp[rr]; }
        } else {
          fetch_params(kb, scb, zpb);
        }
        have_next = kb + kDqGroups < t.kbn;
        if (have_next) fetch_params(kb + kDqGroups, nsc, nzp);
        __half2 off2[2], scale2[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const float zp = p.zeros != nullptr ? param_from_bits(zpb[rr], p.param_dtype) : 0.f;
          off2[rr] = __float2half2_rn(zbase + zp);
          scale2[rr] = __float2half2_rn(param_from_bits(scb[rr], p.param_dtype));
        }
        if (!ahead_raw) guarded_wait(bar(kBarRawFull + r), raw_cur.phase);
        uint4 raw[2][2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const uint4* src = reinterpret_cast<const uint4*>(raw_base + (size_t)r * kRawBytes + (row_a + 64 * rr) * (kBK / 2));
          raw[rr][0] = src[0];
          raw[rr][1] = src[1];
        }
        // The stage's weight half is free once the MMAs of its previous use have completed (Empty).  Waiting for the
        // activation blocks instead (Full) put a TMA round trip, issued only after Empty, on every stage's critical path.
        if (!ahead_full) guarded_wait(bar(kBarEmpty + s), st_cur.phase ^ 1);
        unsigned char* bt = tiles + (size_t)s * kStageBytes + kABytes;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int row_in_tile = row_a + 64 * rr;
          unsigned char* brow = bt + row_in_tile * 128;
          const uint32_t words[8] = {raw[rr][0].x, raw[rr][0].y, raw[rr][0].z, raw[rr][0].w, raw[rr][1].x, raw[rr][1].y, raw[rr][1].z, raw[rr][1].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {                  // 16-byte chunk j of the 128-byte row, K order
            const uint32_t word = p.nibble_signed ? (words[j] ^ 0x88888888u) : words[j];   // two's complement -> code + 8
            *reinterpret_cast<uint4*>(brow + ((j ^ (row_in_tile & 7)) << 4)) = w4f_dequant_word(word, off2[rr], scale2[rr]);
          }
        }
        fence_proxy_async();     // make the generic-proxy stores visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(kBarReady + s));
          mbar_arrive(bar(kBarRawEmpty + r));            // the packed bytes were consumed by the conversion above
        }
        // this group's next stage: its two barriers are tested now, after this stage's work (a blocking wait costs ~200
        // cycles even when the phase is complete; the later the test, the likelier "yes"); non-blocking: "not yet" is
        // a normal answer
        ahead_raw = mbar_test_wait(bar(kBarRawFull + raw_nxt.slot), raw_nxt.phase);
        ahead_full = mbar_test_wait(bar(kBarEmpty + st_nxt.slot), st_nxt.phase ^ 1);
      }
      it_base += (uint32_t)t.kbn;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ----------------------------------------------------------------------------------------- host

bool w4a16_gemm_fused_supported(int m, int n, int k, int padded_k, int group_size) {
  return m >= 1 && n % 8 == 0 && k == padded_k && k % 64 == 0 && (group_size == 64 || group_size == 128);
}

// Measured on B200 (bf16, group 128), fused against two-pass: N = 4096, K = 14336 (32 channel tiles, split over K):
// 45 / 47 / 52 / 70 / 109 us against 122 / 122 / 122 / 125 / 128 us at M = 32 / 64 / 128 / 256 / 512; N = 28672, K = 4096
// (224 tiles): 71 / 72 / 74 / 89 / 159 us against 110 / 110 / 111 / 129 / 172 us.  So up to 512 tokens (two 256-token
// chunks, the weights converted once per chunk); beyond that the two-pass form, whose conversion cost does not grow
// with M, is ahead.
// Small layers (the shards of a tensor-parallel block) change the balance for two chunks: at M = 512 a 3584 x 4096 layer
// takes 61 us fused against 45 us two-pass, a 7168 x 4096 layer 47 against 53; below 24 M weights two chunks stay two-pass.
bool w4a16_gemm_fused_preferred(int m, int n, int k, int padded_k, int group_size) {
  if (!w4a16_gemm_fused_supported(m, n, k, padded_k, group_size) || m <= 16 || m > 4 * w4f::kBM) return false;
  return m <= 2 * w4f::kBM || (long long)n * k >= 24ll * 1024 * 1024;
}

struct W4FusedPlan {
  int mt, mchunks, ntiles, splits, kb_per_split;
};
static W4FusedPlan w4f_plan(int m, int n, int k, int sms) {
  W4FusedPlan pl;
  pl.mt = m > w4f::kBM ? 2 : 1;
  pl.mchunks = ceil_div(m, pl.mt * w4f::kBM);
  pl.ntiles = ceil_div(n, w4f::kBN);
  const int tiles = pl.mchunks * pl.ntiles, kblocks = k / w4f::kBK;
  // split K while the tiles leave more than half of the SMs idle; a split keeps at least 16 K blocks
  int splits = 1;
  while (tiles * splits * 2 <= sms && kblocks / (splits * 2) >= 16 && splits < 8) splits *= 2;
  pl.splits = splits;
  pl.kb_per_split = ceil_div(kblocks, splits);
  pl.splits = ceil_div(kblocks, pl.kb_per_split);
  return pl;
}

// [0,256) status | tickets (one per output tile, 4 KiB) | fp16 copy of bf16 activations | fp32 partial tiles of a K split
static size_t w4f_align(size_t v) { return (v + 255) & ~(size_t)255; }
constexpr size_t kW4FTicketBytes = 16384;
size_t w4a16_gemm_fused_workspace_bytes(int m, int n, int k) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const W4FusedPlan pl = w4f_plan(m, n, k, sms);
  size_t bytes = 256 + kW4FTicketBytes + w4f_align((size_t)m * k * 2);
  if (pl.splits > 1) bytes += (size_t)pl.mchunks * pl.ntiles * pl.splits * pl.mt * w4f::kBM * w4f::kBN * sizeof(float);
  return bytes;
}

int bf16_to_f16_launch(const void* src, void* dst, size_t elements, unsigned int* status, cudaStream_t stream);

template <int MT, typename T>
static int launch_w4f(const void* x, const void* qw, W4FusedParams p, cudaStream_t stream, int sms) {
  using namespace w4f;
  CUtensorMap tm_a, tm_w;
  XQT_CUDA((cudaError_t)make_tile_map(&tm_a, x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.m, p.k, kBM));
  XQT_CUDA((cudaError_t)make_byte_map(&tm_w, qw, p.n, p.k / 2, kBK / 2, kBN));
  constexpr int stage_bytes = MT * kABlockBytes + kBBytes;
  p.raw_bufs = kMaxRaw;
  int stages = (kSmemBudget - 1024 - p.raw_bufs * kRawBytes) / stage_bytes;
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  const size_t smem_bytes = (size_t)p.stages * stage_bytes + (size_t)p.raw_bufs * kRawBytes + 1024;
  auto kern = gemm_w4a16_fused_kernel<MT, T>;
  XQT_SMEM_OPT_IN(kern, kSmemBudget);
  int grid = sms;
  const int tiles = p.mchunks * p.ntiles * p.splits;
  if (grid > tiles) grid = tiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, tm_w, p);
  return launch_status();
}

int w4a16_gemm_fused_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                            const void* residual, void* out, int m, int n, int k, int group_size, int nibble_signed,
                            int act_dtype, int param_dtype, int out_f32, void* workspace, size_t workspace_bytes,
                            cudaStream_t stream) {
  XQT_REQUIRE(w4a16_gemm_fused_supported(m, n, k, k, group_size));
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= w4a16_gemm_fused_workspace_bytes(m, n, k) && ((uintptr_t)workspace & 255) == 0);
  XQT_REQUIRE(((uintptr_t)out & 15) == 0 && ((uintptr_t)qw & 15) == 0 && ((uintptr_t)x & 15) == 0);
  XQT_REQUIRE(!out_f32 || residual == nullptr);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const W4FusedPlan pl = w4f_plan(m, n, k, sms);
  unsigned char* base = reinterpret_cast<unsigned char*>(workspace);
  unsigned int* status = reinterpret_cast<unsigned int*>(base);
  unsigned int* tickets = reinterpret_cast<unsigned int*>(base + 256);
  unsigned char* x16 = base + 256 + kW4FTicketBytes;
  float* partials = reinterpret_cast<float*>(x16 + w4f_align((size_t)m * k * 2));
  XQT_REQUIRE((size_t)pl.mchunks * pl.ntiles * sizeof(unsigned int) <= kW4FTicketBytes);
  if (act_dtype == XQT_B200_BF16) {
    XQT_CUDA((cudaError_t)bf16_to_f16_launch(x, x16, (size_t)m * k, status, stream));
    x = x16;
  }
  W4FusedParams p{};
  p.m = m; p.n = n; p.k = k; p.group_size = group_size; p.groups = k / group_size;
  p.mchunks = pl.mchunks; p.ntiles = pl.ntiles; p.splits = pl.splits; p.kb_per_split = pl.kb_per_split; p.kblocks = k / w4f::kBK;
  p.param_dtype = param_dtype; p.nibble_signed = nibble_signed; p.out_f32 = out_f32;
  p.scales = scales; p.zeros = zeros; p.bias = bias; p.residual = residual; p.out = out;
  p.partials = partials; p.tickets = tickets; p.status = status;
  if (act_dtype == XQT_B200_BF16)
    return pl.mt == 2 ? launch_w4f<2, __nv_bfloat16>(x, qw, p, stream, sms) : launch_w4f<1, __nv_bfloat16>(x, qw, p, stream, sms);
  return pl.mt == 2 ? launch_w4f<2, __half>(x, qw, p, stream, sms) : launch_w4f<1, __half>(x, qw, p, stream, sms);
}

}  // namespace xqt_b200

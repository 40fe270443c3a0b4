// W4A4 SVDQuant / ConvRot GEMM on tcgen05:
//   Y[m,n] = sum_g a_s[m,g] w_s[n,g] * ( sum_{k in g} a_q[m,k] w_q[n,k] )  +  sum_r la[m,r] up[n,r]  + bias[n]
// with 64-K groups g, int4 codes on both sides, fp32 scales and an fp32 accumulation across groups.
//
// Operands.  Blackwell has no int4 MMA.  Both operands go to the tensor core as FP8 E4M3 bytes of the form
// sign << 7 | magnitude: for magnitudes 0..15 that byte IS the E4M3 number magnitude * 2^-9 (subnormals and
// the first binade are linear), so an int4 code becomes an exact FP8 value without a table.  The activation
// codes arrive in that form from the rotate+quantise prologue.  The packed two's-complement weight nibbles
// are widened to the same bytes by a streaming pre-pass (w44_expand_kernel, N*K bytes of scratch that stay
// in L2) -- each weight is converted once per call, not once per 128-row tile of activations, and both
// operands of the GEMM then come in by TMA.  Every product is an integer times 2^-18, a 64-K slab sums to
// at most 2^12 of them, so the fp32 accumulation of tcgen05.mma kind::f8f6f4 is exact and equals the
// reference's int32 group sum (jit/include/nunchaku/gemm_base.cuh:367-446); 2^18 is folded into the weight
// scale on the host.
//
// Per-group scales.  A 128-K stage is two slabs; each slab is two MMAs (K = 32) into its own 128 columns of
// tensor memory, and a stage's two slabs are handed to the drain warps together (two 256-column buffers:
// a barrier test costs about 200 cycles, so there is one hand-over per stage and warp, not per slab).
// Sixteen drain warps fold the slabs into fp32 register accumulators with a_s*w_s -- the per-slab scaling
// the reference does in half precision (gemm_w4a4.cuh:833-930), here in fp32: one multiply and one fused
// multiply-add per element (the packed f32x2 forms measured no faster).  That drain is CUDA-core work,
// M*N*K/64 scaled adds (two fp32 pipe operations each): 256 cycles per 128x128 slab at 128 lanes per SM
// and clock, against about 210 for the slab's MMAs; exact per-group scales bound the kernel near 0.8 of
// the tensor rate.
//
// Rank-R branch (reference: lora.cuh:110-243 "LoRA up").  la * up^T is one more slab per tile, computed by
// the tensor core from bf16 hi/lo splits of both factors (hi x hi + lo x hi + hi x lo, fp32 sums; the
// dropped lo x lo term is 2^-18 relative): six K = 16 steps over two 128-row operand images.
//
// Warp roles (576 threads): warp 0 TMA producer (both operand tiles and the two scale rows of both sides per
// stage, the two rank-R operand images per tile), warp 1 MMA issuer, warps 2-17 drain (tensor-memory lane quarter =
// warp % 4, 32-column quarter = (warp - 2) / 4).  A drain warp reads a slab in the accumulator-fragment
// distribution (tcgen05.ld shape 16x256b): lane t holds rows t/4 + {0, 8, 16, 24} and, of each 8-column
// group, columns 2*(t%4), 2*(t%4)+1.  A thread then needs 4 activation scales and 8 weight scales per slab,
// all from shared memory (activation scales read from global memory came back from L2 once per slab and
// were the longest stall of the drain: 539 -> 485 us for the forward of the 4096 x 12288 x 3072 layer);
// in the one-row-per-thread shape it would need 32 weight scales, every lane the same ones, and those
// broadcast loads alone (128 bytes of register write-back per lane and slab) take more shared-memory pipe
// time than the slab's MMAs.
#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows);

namespace w4a4 {
constexpr int kBM = 128, kBN = 128, kStageK = 128, kRank = 32;
constexpr int kDrainWarps = 16, kFirstDrainWarp = 2;
constexpr int kThreads = (kFirstDrainWarp + kDrainWarps) * 32;      // 576
constexpr int kMaxStages = 5;
constexpr int kPairBufs = 2;                                        // tensor-memory buffers of two slabs (256 columns)
constexpr int kABytes = kBM * 128, kBBytes = kBN * 128, kStageBytes = kABytes + kBBytes;
constexpr int kUpBytes = kBN * kRank * 4, kLaBytes = kBM * kRank * 4;
constexpr int kSmemBudget = 226 * 1024;
enum Status : unsigned int { kTimeout = 64 };
// barrier slots
constexpr int kBarFull = 0, kBarEmpty = kBarFull + kMaxStages;
constexpr int kBarPairFull = kBarEmpty + kMaxStages, kBarPairEmpty = kBarPairFull + kPairBufs;
constexpr int kBarEpiFull = kBarPairEmpty + kPairBufs, kBarEpiEmpty = kBarEpiFull + 1, kBarCount = kBarEpiEmpty + 1;
// Scales travel with their stage: a ring of (stages + 2) slots of [w_scale: 2 groups x 128 | a_scale: 2 groups x 128]
// fp32, filled by two bulk copies on the stage's full barrier.  A slot is rewritten for stage i only after the MMAs of
// stage i - stages have completed; those were issued after the drain warps had released the pair buffer of two
// hand-overs earlier, i.e. after they had read the scales of stage i - stages - 2: no barrier of its own.
constexpr int kScaleSlotBytes = 2 * 2 * 128 * 4;                    // 2048
constexpr int kScaleSlotsExtra = 2;
}  // namespace w4a4

struct W4A4Params {
  int m, n, k, groups;
  int mtiles, ntiles, kstages, stages;
  int aux_tile_bytes;          // groups * 512 + kUpBytes
  const float* a_scale_t;      // [mtiles][groups][128]: the activation scales, tile-major (rows past M are zero)
  const uint8_t* aux;          // per n-tile: w_scale * 2^18 as [groups][128] fp32, then the up factors as a 128-row operand image
  const uint8_t* la_tiles;     // per m-tile: the low-rank activations as a 128-row operand image (see w44_la_image_kernel)
  const float* bias;
  void* out;
  unsigned int* status;
};

__device__ __forceinline__ uint32_t w44_pack2(__nv_bfloat16*, float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t w44_pack2(__half*, float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float w44_lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned long long w44_lds64(uint32_t addr) {
  unsigned long long v;
  asm volatile("ld.shared.b64 %0, [%1];\n" : "=l"(v) : "r"(addr));
  return v;
}

// one packed word (8 two's-complement nibbles, k0..k7) -> 8 bytes sign << 7 | |w| in K order.
// Per nibble: mask = 0xF where negative; (w ^ mask) + 1 negates it (no carry leaves a nibble: the
// complemented value of a negative nibble is at most 7).
__device__ __forceinline__ uint2 signmag8(uint32_t w) {
  const uint32_t s = w & 0x88888888u, t = s >> 3;
  const uint32_t mag = (w ^ (s | (s - t))) + t;
  const uint32_t e = (mag & 0x0F0F0F0Fu) | ((s << 4) & 0x80808080u);
  const uint32_t o = ((mag >> 4) & 0x0F0F0F0Fu) | (s & 0x80808080u);
  return make_uint2(__byte_perm(e, o, 0x5140), __byte_perm(e, o, 0x7362));
}

// packed nibbles [N, K/2] -> sign-magnitude bytes [N, K]; a thread converts 8 packed bytes into one 16-byte store, so a
// warp's loads (256 bytes) and stores (512 bytes) are contiguous.  `chunks` counts 16-byte packed pieces.
__global__ void __launch_bounds__(256) w44_expand_kernel(const uint4* __restrict__ packed, uint4* __restrict__ bytes, size_t chunks) {
  const uint2* src = reinterpret_cast<const uint2*>(packed);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < 2 * chunks; i += (size_t)gridDim.x * blockDim.x) {
    const uint2 v = __ldg(src + i);
    const uint2 a = signmag8(v.x), b = signmag8(v.y);
    bytes[i] = make_uint4(a.x, a.y, b.x, b.y);
  }
}

// The drain role as a function of its own (not inlined): its register allocation then holds nothing of the
// other roles' state.
template <typename OutT>
__device__ __noinline__ void w44_drain(const W4A4Params& p, uint32_t tmem_base, uint32_t bar0, uint32_t scale_addr,
                                       volatile unsigned int* s_abort) {
  using namespace w4a4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nslots = (uint32_t)p.stages + kScaleSlotsExtra;
  uint32_t slot = 0;                                  // ring slot of the stage being drained
  const int total_tiles = p.mtiles * p.ntiles;
  auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };
  auto guarded_wait = [&](uint32_t b, uint32_t parity) {
    if (*s_abort == 0u && !mbar_wait(b, parity)) {
      *s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };
  const int quarter = warp & 3, colq = (warp - kFirstDrainWarp) >> 2;
  const int rq = lane >> 2, c2 = lane & 3;
  const uint32_t tlane = tmem_base + colq * 32 + ((uint32_t)(quarter * 32) << 16);
  uint32_t local = 0, pair = 0;                       // pair: hand-overs so far (one per stage, one per rank-R slab)
  for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
    const int mt = tile % p.mtiles, nt = tile / p.mtiles;
    const int row0 = mt * kBM + quarter * 32 + rq;       // the thread's rows are row0 + 8 i
    // Two 16-register buffers: rows 0-15 and rows 16-31 of the warp's 32 x 32 part of a slab (one tcgen05.ld each).
    // While one is folded the other is in flight: a tensor-memory load takes about 150 cycles, and one warp's
    // share of the arithmetic between two waits has to cover it.
    uint32_t ra[16], rb[16];
    guarded_wait(bar(kBarPairFull + pair % kPairBufs), (pair / kPairBufs) & 1);
    tc_fence_after();
    tmem_ld_16x256b_x4(tlane + (pair % kPairBufs) * (2 * kBN), ra);
    const uint32_t sw = scale_addr + (colq * 32 + 2 * c2) * 4;                  // this thread's first column pair of a w_scale row
    const uint32_t sr = scale_addr + 1024 + (quarter * 32 + rq) * 4;            // its first row of an a_scale row
    unsigned long long acc[16];                       // [row i][column group j]: columns (8 j + 2 c2, + 1) of row row0 + 8 i as one f32x2
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0ull;
    // 16 rows (i0, i0 + 1) x 32 columns: acc += r * (a_s[row] * w_s[column]), two columns per packed instruction
    auto fold = [&](const uint32_t (&r)[16], const unsigned long long (&ws)[4], const float (&sa)[4], int i0) {
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        const int i = i0 + ii;
        const unsigned long long sa2 = f32x2_pack(sa[i], sa[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const unsigned long long r2 = f32x2_pack(__uint_as_float(r[4 * j + 2 * ii]), __uint_as_float(r[4 * j + 2 * ii + 1]));
          acc[4 * i + j] = f32x2_fma(r2, f32x2_mul(sa2, ws[j]), acc[4 * i + j]);
        }
      }
    };
    const int kstages = p.kstages;
    for (int ks = 0; ks < kstages; ++ks, ++pair) {
      const int pb = pair % kPairBufs;
      const uint32_t npair = pair + 1;
      // A barrier test answers after about 200 cycles even when the phase is complete: ask for the next
      // hand-over now and read the answer after this stage's arithmetic.
      const bool next_full = mbar_test_wait(bar(kBarPairFull + npair % kPairBufs), (npair / kPairBufs) & 1);   // non-blocking
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t swg = sw + slot * kScaleSlotBytes + h * (kBN * 4);
        const uint32_t srg = sr + slot * kScaleSlotBytes + h * (kBM * 4);
        const uint32_t tslab = tlane + pb * (2 * kBN) + h * kBN;
        unsigned long long ws[4];
        float sa[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) ws[j] = w44_lds64(swg + j * 32);     // columns 8 j + 2 c2, + 1
#pragma unroll
        for (int i = 0; i < 4; ++i) sa[i] = w44_lds32f(srg + 32 * i);   // rows row0 + 8 i
        tmem_wait_ld_dep(ra);                          // rows 0-15 of the slab
        tmem_ld_16x256b_x4(tslab + (16u << 16), rb);
        fold(ra, ws, sa, 0);
        tmem_wait_ld_dep(rb);                          // rows 16-31
        if (h == 0) {
          tmem_ld_16x256b_x4(tslab + kBN, ra);         // the stage's second slab
        } else {
          tc_fence_before();                           // both slabs are in registers: hand the buffer back
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(kBarPairEmpty + pb));
          // the next hand-over: the following stage, or the tile's rank-R slab
          if (!next_full) guarded_wait(bar(kBarPairFull + npair % kPairBufs), (npair / kPairBufs) & 1);
          tc_fence_after();
          tmem_ld_16x256b_x4(tlane + (npair % kPairBufs) * (2 * kBN), ra);
        }
        fold(rb, ws, sa, 2);
      }
      if (++slot == nslots) slot = 0;
    }
    // rank-R branch: one more slab (la * up^T from the tensor core), added as it is; its first half is in flight
    {
      const int pb = pair % kPairBufs;
      const uint32_t tslab = tlane + pb * (2 * kBN);
      tmem_wait_ld_dep(ra);
      tmem_ld_16x256b_x4(tslab + (16u << 16), rb);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int ii = 0; ii < 2; ++ii)
          acc[4 * ii + j] = f32x2_add(acc[4 * ii + j], f32x2_pack(__uint_as_float(ra[4 * j + 2 * ii]), __uint_as_float(ra[4 * j + 2 * ii + 1])));
      }
      tmem_wait_ld_dep(rb);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPairEmpty + pb));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int ii = 0; ii < 2; ++ii)
          acc[4 * (2 + ii) + j] = f32x2_add(acc[4 * (2 + ii) + j], f32x2_pack(__uint_as_float(rb[4 * j + 2 * ii]), __uint_as_float(rb[4 * j + 2 * ii + 1])));
      }
      ++pair;
    }
    // bias and store.  The four lanes of a row group exchange their column pairs so that each stores eight
    // adjacent columns (16 bytes) of one row: lane c2 ends up with column group j = c2 of rows row0 + 8 i.
    OutT* out = reinterpret_cast<OutT*>(p.out);
    const int col = nt * kBN + colq * 32 + 8 * c2;
    float b8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) b8[e] = (p.bias != nullptr && col < p.n) ? __ldg(p.bias + col + e) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // before: v[j] holds columns 8 j + 2 c2 (+1); after: columns 8 c2 + 2 j (+1).
      unsigned long long v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = acc[4 * i + j];
      // 4 x 4 transpose over the lanes c2 = 0..3 in two exchange steps
#pragma unroll
      for (int step = 1; step <= 2; step <<= 1) {
        const bool upper = (c2 & step) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if ((j & step) == 0) {
            // lanes without the bit keep [j] and give [j + step]; lanes with it keep [j + step] and give [j]
            const unsigned long long give = upper ? v[j] : v[j + step];
            const unsigned long long got = __shfl_xor_sync(0xffffffffu, give, step);
            if (upper) v[j] = got; else v[j + step] = got;
          }
        }
      }
      const int row = row0 + 8 * i;
      if (row < p.m && col < p.n) {            // N is a multiple of 8: the eight columns are inside together
        float f[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) f32x2_unpack(v[q], f[2 * q], f[2 * q + 1]);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += b8[e];
        OutT* dst = out + (size_t)row * p.n + col;
        *reinterpret_cast<uint4*>(dst) = make_uint4(w44_pack2(dst, f[0], f[1]), w44_pack2(dst, f[2], f[3]), w44_pack2(dst, f[4], f[5]),
                                                    w44_pack2(dst, f[6], f[7]));
      }
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(w4a4::kThreads, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ W4A4Params p) {
  using namespace w4a4;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[kBarCount];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;

  constexpr uint32_t kTmemCols = kPairBufs * 2 * kBN;   // 512
  constexpr uint32_t kIdesc = umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, kBM, kBN);
  constexpr uint32_t kIdescLora = umma_idesc(kAccF32, kFmtBF16, kFmtBF16, kBM, kBN);

  const int warp = threadIdx.x >> 5;
  const int ns = p.stages;
  // dynamic shared memory: operand stages | scale ring | up-factor image | low-rank activation image
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  const int scale_bytes = p.groups * 512;            // one tile's w_scale rows in `aux` (the up image follows them)
  unsigned char* scale_base = tiles + (size_t)ns * kStageBytes;
  const uint32_t nslots = (uint32_t)ns + kScaleSlotsExtra;
  unsigned char* up_base = scale_base + (size_t)nslots * kScaleSlotBytes;
  unsigned char* la_base = up_base + kUpBytes;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };

  if (threadIdx.x == 0) {
    s_abort = 0u;
    for (int s = 0; s < ns; ++s) {
      mbar_init(bar(kBarFull + s), 1);
      mbar_init(bar(kBarEmpty + s), 1);
    }
    for (int b = 0; b < kPairBufs; ++b) {
      mbar_init(bar(kBarPairFull + b), 1);
      mbar_init(bar(kBarPairEmpty + b), kDrainWarps);
    }
    mbar_init(bar(kBarEpiFull), 1);
    mbar_init(bar(kBarEpiEmpty), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_addr(&s_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = p.mtiles * p.ntiles;

  // Every wait is bounded: when one runs out the CTA stops waiting anywhere, reports and drains out.
  auto guarded_wait = [&](uint32_t b, uint32_t parity) {
    if (s_abort == 0u && !mbar_wait(b, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };
  // two independent barrier tests in flight at once (each takes about 200 cycles to answer)
  auto guarded_wait2 = [&](uint32_t b0, uint32_t parity0, uint32_t b1, uint32_t parity1) {
    if (s_abort == 0u && !mbar_wait2(b0, parity0, b1, parity1)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      uint32_t it = 0, local = 0, slot = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const int mt = tile % p.mtiles, nt = tile / p.mtiles;
        const uint8_t* wsrc = p.aux + (size_t)nt * p.aux_tile_bytes;
        const uint8_t* asrc = reinterpret_cast<const uint8_t*>(p.a_scale_t) + (size_t)mt * scale_bytes;
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          const int s = it % ns;
          guarded_wait(bar(kBarEmpty + s), ((it / ns) & 1) ^ 1);
          unsigned char* st = tiles + (size_t)s * kStageBytes;
          const uint32_t sc = smem_addr(scale_base + (size_t)slot * kScaleSlotBytes);
          mbar_expect_tx(bar(kBarFull + s), kStageBytes + kScaleSlotBytes);
          tma_load_2d(smem_addr(st), &tm_a, ks * kStageK, mt * kBM, bar(kBarFull + s));
          tma_load_2d(smem_addr(st + kABytes), &tm_b, ks * kStageK, nt * kBN, bar(kBarFull + s));
          bulk_g2s(sc, wsrc + (size_t)ks * 1024, 1024, bar(kBarFull + s));             // groups 2 ks, 2 ks + 1
          bulk_g2s(sc + 1024, asrc + (size_t)ks * 1024, 1024, bar(kBarFull + s));
          if (++slot == nslots) slot = 0;
        }
        // the tile's rank-R operand images; the MMAs of the previous tile's rank-R slab have released the buffers
        guarded_wait(bar(kBarEpiEmpty), (local & 1) ^ 1);
        mbar_expect_tx(bar(kBarEpiFull), kUpBytes + kLaBytes);
        bulk_g2s(smem_addr(up_base), p.aux + (size_t)nt * p.aux_tile_bytes + scale_bytes, kUpBytes, bar(kBarEpiFull));
        bulk_g2s(smem_addr(la_base), p.la_tiles + (size_t)mt * kLaBytes, kLaBytes, bar(kBarEpiFull));
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0, pair = 0, local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        for (int ks = 0; ks < p.kstages; ++ks, ++it, ++pair) {
          const int s = it % ns, pb = pair % kPairBufs;
          guarded_wait2(bar(kBarFull + s), (it / ns) & 1, bar(kBarPairEmpty + pb), ((pair / kPairBufs) & 1) ^ 1);
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr), bdesc = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int h = 0; h < 2; ++h) {                  // two 64-K slabs per stage, 128 columns each
            const uint32_t d_tmem = tmem_base + pb * (2 * kBN) + h * kBN;
            umma_ss_f8(d_tmem, adesc + h * 4, bdesc + h * 4, kIdesc, 0u);
            umma_ss_f8(d_tmem, adesc + h * 4 + 2, bdesc + h * 4 + 2, kIdesc, 1u);
          }
          umma_commit(bar(kBarPairFull + pb));
          umma_commit(bar(kBarEmpty + s));
        }
        // the rank-R branch as one more slab: [la_hi | la_lo] x [up_hi | up_lo]^T without the lo x lo term, bf16
        // operands (kind::f16), six K = 16 steps over the two 128-byte-row images the producer has brought in
        {
          const int pb = pair % kPairBufs;
          guarded_wait2(bar(kBarEpiFull), local & 1, bar(kBarPairEmpty + pb), ((pair / kPairBufs) & 1) ^ 1);
          tc_fence_after();
          const uint64_t ladesc = umma_desc_sw128(smem_addr(la_base)), updesc = umma_desc_sw128(smem_addr(up_base));
          const uint32_t d_tmem = tmem_base + pb * (2 * kBN);
          umma_ss<false>(d_tmem, ladesc + 0, updesc + 0, kIdescLora, 0u);     // hi x hi
          umma_ss<false>(d_tmem, ladesc + 2, updesc + 2, kIdescLora, 1u);
          umma_ss<false>(d_tmem, ladesc + 4, updesc + 0, kIdescLora, 1u);     // lo x hi
          umma_ss<false>(d_tmem, ladesc + 6, updesc + 2, kIdescLora, 1u);
          umma_ss<false>(d_tmem, ladesc + 0, updesc + 4, kIdescLora, 1u);     // hi x lo
          umma_ss<false>(d_tmem, ladesc + 2, updesc + 6, kIdescLora, 1u);
          umma_commit(bar(kBarPairFull + pb));
          umma_commit(bar(kBarEpiEmpty));                                      // the two images may be overwritten
          ++pair;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- drain warps
    w44_drain<OutT>(p, tmem_base, bar0, smem_addr(scale_base), &s_abort);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// Operand image of the low-rank activations for one 128-row tile: row r holds [hi(32) | lo(32)] bf16 with
// hi = bf16(v), lo = bf16(v - hi) -- 128 bytes, stored in the 128-byte-swizzled order the MMA descriptors read
// (16-byte chunk c of row r at chunk c ^ (r & 7)).  The up factors get the same image on the host, once.
__global__ void __launch_bounds__(128) w44_la_image_kernel(const float* __restrict__ la, uint8_t* __restrict__ tiles) {
  const int r = threadIdx.x;
  const float4* src = reinterpret_cast<const float4*>(la + ((size_t)blockIdx.x * 128 + r) * w4a4::kRank);
  uint8_t* dst = tiles + (size_t)blockIdx.x * w4a4::kLaBytes + (size_t)r * 128;
  uint32_t hi[16], lo[16];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 v = __ldg(src + q);
    const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const __nv_bfloat16 h0 = __float2bfloat16_rn(f[2 * e]), h1 = __float2bfloat16_rn(f[2 * e + 1]);
      const __nv_bfloat16 l0 = __float2bfloat16_rn(f[2 * e] - __bfloat162float(h0)), l1 = __float2bfloat16_rn(f[2 * e + 1] - __bfloat162float(h1));
      hi[2 * q + e] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
      lo[2 * q + e] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
    *reinterpret_cast<uint4*>(dst + (((c + 4) ^ (r & 7)) << 4)) = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
  }
}

// activation scales [M, G] -> [Mpad/128][G][128] (rows past M zero): one stage's two groups of a 128-row tile are 1 KiB
__global__ void __launch_bounds__(256) w44_scale_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int m, int groups,
                                                                  int mpad) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.x * 32, g0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;     // 32 x 8
  for (int y = ty; y < 32; y += 8) {
    const int r = r0 + y, g = g0 + tx;
    tile[y][tx] = (r < m && g < groups) ? __ldg(src + (size_t)r * groups + g) : 0.f;
  }
  __syncthreads();
  for (int y = ty; y < 32; y += 8) {
    const int g = g0 + y, r = r0 + tx;
    if (g < groups && r < mpad) dst[((size_t)(r >> 7) * groups + g) * 128 + (r & 127)] = tile[tx][y];
  }
}

// ----------------------------------------------------------------------------------------- host

size_t w4a4_aux_tile_bytes(int k) { return (size_t)(k / 64) * 512 + w4a4::kUpBytes; }

// shared-memory plan: operand stages, the scale ring that follows them, the two rank-R images
static size_t w4a4_smem_bytes(int stages) {
  using namespace w4a4;
  return (size_t)stages * kStageBytes + (size_t)(stages + kScaleSlotsExtra) * kScaleSlotBytes + kUpBytes + kLaBytes + 1024;
}
static int w4a4_stages() {
  int ns = w4a4::kMaxStages;
  while (ns > 2 && w4a4_smem_bytes(ns) > (size_t)w4a4::kSmemBudget) --ns;
  return ns;
}

bool w4a4_gemm_supported(int m, int n, int k) {
  return m >= 1 && n % 8 == 0 && k % 128 == 0 && k > 0;
}

template <typename OutT>
static int launch_w4a4(const void* a_codes, const void* b_bytes, W4A4Params p, cudaStream_t stream) {
  using namespace w4a4;
  CUtensorMap tm_a, tm_b;
  XQT_CUDA((cudaError_t)make_tile_map(&tm_a, a_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.m, p.k, kBM));
  XQT_CUDA((cudaError_t)make_tile_map(&tm_b, b_bytes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.n, p.k, kBN));
  p.stages = w4a4_stages();
  p.mtiles = ceil_div(p.m, kBM);
  p.ntiles = ceil_div(p.n, kBN);
  p.kstages = p.k / kStageK;
  const size_t smem_bytes = w4a4_smem_bytes(p.stages);
  auto kern = gemm_w4a4_kernel<OutT>;
  XQT_SMEM_OPT_IN(kern, kSmemBudget);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms > 0 ? sms : 148;
  if (grid > p.mtiles * p.ntiles) grid = p.mtiles * p.ntiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, tm_b, p);
  return launch_status();
}

// workspace: status word (256 bytes) | one low-rank activation image per 128-row tile | the activation scales
// transposed [K/64, mtiles*128] | the weights as bytes [N, K]
static size_t w4a4_images_bytes(int m) { return (size_t)ceil_div(m, w4a4::kBM) * w4a4::kLaBytes; }
static size_t w4a4_scales_bytes(int m, int k) { return (size_t)ceil_div(m, w4a4::kBM) * w4a4::kBM * (k / 64) * sizeof(float); }
size_t w4a4_workspace_bytes(int m, int n, int k) { return 256 + w4a4_images_bytes(m) + w4a4_scales_bytes(m, k) + (size_t)n * k; }

int w4a4_expand_weight_launch(const void* qweight, void* weight_bytes, int n, int k, cudaStream_t stream) {
  XQT_REQUIRE(qweight != nullptr && weight_bytes != nullptr && n > 0 && k > 0 && k % 32 == 0);
  XQT_REQUIRE(((uintptr_t)qweight & 15) == 0 && ((uintptr_t)weight_bytes & 15) == 0);
  const size_t chunks = (size_t)n * k / 32;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t want = (chunks + 255) / 256;
  w44_expand_kernel<<<(unsigned)(want < (size_t)sms * 8 ? want : (size_t)sms * 8), 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(qweight), reinterpret_cast<uint4*>(weight_bytes), chunks);
  return launch_status();
}

// weight_bytes: null, or the [N, K] sign-magnitude bytes w4a4_expand_weight_launch made of qweight (a caller-held
// operand cache: the per-call widening pass is skipped).  flags bit 0: a_scale is already tile-major
// [ceil(M/128)][K/64][128] (rotate_quant mode 6); bit 1: la points at the operand images lowrank_down wrote, not at
// fp32 [M, 32] -- the two preparation launches are skipped.
int w4a4_gemm_launch(const void* a_codes, const float* a_scale, const void* qweight, const void* weight_bytes,
                     const void* aux, const float* la, const float* bias, void* out, int m, int n, int k, int out_dtype,
                     int flags, void* workspace, cudaStream_t stream) {
  unsigned int* status = reinterpret_cast<unsigned int*>(workspace);
  XQT_REQUIRE(w4a4_gemm_supported(m, n, k));
  XQT_REQUIRE(a_codes != nullptr && a_scale != nullptr && (qweight != nullptr || weight_bytes != nullptr) && aux != nullptr &&
              la != nullptr && out != nullptr && status != nullptr);
  XQT_REQUIRE(((uintptr_t)aux & 15) == 0 && ((uintptr_t)la & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
              ((uintptr_t)a_codes & 15) == 0 && ((uintptr_t)weight_bytes & 15) == 0);
  W4A4Params p{};
  p.m = m; p.n = n; p.k = k; p.groups = k / 64;
  p.aux_tile_bytes = (int)w4a4_aux_tile_bytes(k);
  p.aux = (const uint8_t*)aux; p.bias = bias;
  uint8_t* images = reinterpret_cast<uint8_t*>(workspace) + 256;
  float* scales_t = reinterpret_cast<float*>(images + w4a4_images_bytes(m));
  const uint8_t* b_bytes = reinterpret_cast<const uint8_t*>(weight_bytes);
  const int mpad = ceil_div(m, w4a4::kBM) * w4a4::kBM;
  if (flags & 1) {
    XQT_REQUIRE(((uintptr_t)a_scale & 15) == 0);
    p.a_scale_t = a_scale;
  } else {
    w44_scale_transpose_kernel<<<dim3(mpad / 32, ceil_div(p.groups, 32)), 256, 0, stream>>>(a_scale, scales_t, m, p.groups, mpad);
    XQT_CUDA(cudaGetLastError());
    p.a_scale_t = scales_t;
  }
  XQT_REQUIRE(((uintptr_t)images & 15) == 0);
  if (flags & 2) {
    XQT_REQUIRE(((uintptr_t)la & 127) == 0);
    images = const_cast<uint8_t*>(reinterpret_cast<const uint8_t*>(la));
  } else {
    w44_la_image_kernel<<<ceil_div(m, w4a4::kBM), 128, 0, stream>>>(la, images);
    XQT_CUDA(cudaGetLastError());
  }
  if (b_bytes == nullptr) {
    uint8_t* scratch_bytes = reinterpret_cast<uint8_t*>(scales_t) + w4a4_scales_bytes(m, k);
    const int rc = w4a4_expand_weight_launch(qweight, scratch_bytes, n, k, stream);
    if (rc != 0) return rc;
    b_bytes = scratch_bytes;
  }
  p.la_tiles = images;
  p.out = out; p.status = status;
  if (out_dtype == XQT_B200_BF16) return launch_w4a4<__nv_bfloat16>(a_codes, b_bytes, p, stream);
  XQT_REQUIRE(out_dtype == XQT_B200_FP16);
  return launch_w4a4<__half>(a_codes, b_bytes, p, stream);
}

}  // namespace xqt_b200

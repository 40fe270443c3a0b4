// W4A16 decode (M <= 16) with the inner product on tcgen05: the Blackwell-native form of the
// persistent stream-K decode kernel.
//
// Roles inside the one CTA per SM (320 threads):
//   warps 0-3, 4-7  two dequantisation warpgroups.  Thread (warp % 4, lane) owns output channel
//                   32*(warp%4)+lane of the 128-channel tile -- the same index as its tensor-memory
//                   lane.  Per unit (one quantisation group: 128 or 64 K of its channel) it reads
//                   its packed weights from the shared-memory stage, turns the nibbles into exact
//                   bf16/fp16 integers (code - zero point, one lop3 + one sub per pair), stores
//                   them to tensor memory as the A operand (tcgen05.st), and later drains the
//                   16 fp32 results of the unit and folds them into its 16 running sums with the
//                   group scale:  y[m] += s * sum_k x[m,k] (q[k] - z).
//   warp 8          producer: per 256-K stage one bulk copy of the weights (16 KiB), one of the
//                   scales/zero points, one tiled TMA load of the activations [16 x 256] into the
//                   128-byte-swizzled layout tcgen05 reads (rows >= M arrive as zeros).
//   warp 9          MMA issuer: for each unit, M=128 x N=16 x K=16 tcgen05.mma steps with A from
//                   tensor memory and B (activations) from shared memory, committed to mbarriers.
// The dequantised weight is an exact small integer, the scale is applied in fp32 to the fp32 group
// sum, so the result equals the contract reference (xqt/kernels/ops/gemm/reference.py:263-271,527)
// up to fp32 summation order.  Zero points must be integers in [0, 127] (true of every RTN / AWQ
// checkpoint); other weights are served by the mma.sync decode kernel.
// Stream-K partition, partial-sum scratch, ticket-elected finisher and bounded waits are those of
// w4a16_decode.cu.
#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

#ifdef XQT_TRACE
// instrumented build only: nanosecond timestamps of CTA 0 into the 256-byte status block
#define XQT_TRACE_AT(slot)                                                                   \
  do {                                                                                       \
    if (blockIdx.x == 0) {                                                                   \
      unsigned long long t__;                                                                \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                \
      reinterpret_cast<unsigned long long*>(p.status)[(slot)] = t__;                         \
    }                                                                                        \
  } while (0)
#else
#define XQT_TRACE_AT(slot) do { } while (0)
#endif

namespace dtc {
constexpr int kTileRows = 128;
constexpr int kStageK = 256;
constexpr int kDequantThreads = 256;
constexpr int kThreads = 320;
constexpr int kWBytes = 128 * kStageK / 2;   // 16 KiB
constexpr int kXBytes = 16 * kStageK * 2;    // 8 KiB: four 64-K atoms of [16 rows x 128 B]
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 216 * 1024;
constexpr int kPartialFloats = 16 * kTileRows;
constexpr int kMaxTiles = 8192;
constexpr int kMaxGrid = 256;
constexpr uint32_t kTmemCols = 512;
enum Status : unsigned int { kTimeout = 32 };
constexpr int kNB = 3;   // tensor-memory buffers (A operand + result) per warpgroup: units in flight
__host__ __device__ constexpr uint32_t a_col(int wg, int buf) { return wg * 240 + buf * 64; }
__host__ __device__ constexpr uint32_t d_col(int wg, int buf) { return wg * 240 + 192 + buf * 16; }
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
__device__ __forceinline__ void dq_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

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

template <typename T>
__device__ __forceinline__ uint32_t dq_col(uint32_t word, int i, uint32_t off2) {
  using Tr = TcTraits<T>;
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(word >> (4 * i)), "n"(0x000f000f), "r"(Tr::kMagic));
  typename Tr::h2 v = __hsub2(*reinterpret_cast<typename Tr::h2*>(&r), *reinterpret_cast<const typename Tr::h2*>(&off2));
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ int cta_of_stage(long long x, long long total, int grid) {
  return (int)(((x + 1) * grid - 1) / total);
}

// GK: K per unit = quantisation group size (128 or 64)
template <typename T, typename P, bool SIGNED, int GK>
__global__ void __launch_bounds__(dtc::kThreads, 1)
w4a16_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const DecodeTcParams p) {
  using namespace dtc;
  using Tr = TcTraits<T>;
  constexpr int kUnits = kStageK / GK;        // units per stage: 2 or 4
  constexpr int kUnitsPerWg = kUnits / 2;
  constexpr int kColsPerUnit = GK / 2;        // 32-bit tensor-memory columns of A per unit
  constexpr uint32_t kIdesc = umma_idesc(kAccF32, Tr::kFmt, Tr::kFmt, 128, 16);

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + 4 * kNB];
  __shared__ uint32_t s_tmem_base;
  __shared__ unsigned int s_flag;
  __shared__ volatile unsigned int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long s_begin = (long long)cta * p.total / grid, s_end = (long long)(cta + 1) * p.total / grid;
  const int ns = p.nstages;
  if (tid == 0) XQT_TRACE_AT(1);
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(stages + (size_t)ns * p.stage_bytes);   // [16][128] fp32
  auto full_bar = [&](int s) { return smem_addr(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_addr(&bars[kMaxStages + s]); };
  auto aready_bar = [&](int wg, int b) { return smem_addr(&bars[2 * kMaxStages + wg * kNB + b]); };
  auto dready_bar = [&](int wg, int b) { return smem_addr(&bars[2 * kMaxStages + 2 * kNB + wg * kNB + b]); };

  if (tid == 0) {
    s_abort = 0u;
    for (int i = 0; i < ns; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), 1);
    }
    for (int wg = 0; wg < 2; ++wg)
      for (int b = 0; b < kNB; ++b) {
        mbar_init(aready_bar(wg, b), 4);   // one arrival per warp of the warpgroup
        mbar_init(dready_bar(wg, b), 1);   // tcgen05.commit
      }
    fence_barrier_init();
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 9) {
    tmem_alloc(smem_addr(&s_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  if (tid == 0) XQT_TRACE_AT(2);

  auto guarded_wait = [&](uint32_t bar, uint32_t parity) {
    if (s_abort == 0u && !mbar_wait(bar, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == 8) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      const uint32_t tx = kWBytes + kXBytes + p.sz_stage_bytes;
      uint32_t it = 0;
      for (long long s = s_begin; s < s_end; ++s, ++it) {
        const int slot = it % ns;
        guarded_wait(empty_bar(slot), ((it / ns) & 1) ^ 1);
        const long long tile = s / p.spt;
        const int ks = (int)(s % p.spt);
        unsigned char* st = stages + (size_t)slot * p.stage_bytes;
        const long long unit = tile * (long long)(p.k / 128) + (long long)ks * 2;   // first (tile, 128-K block)
        mbar_expect_tx(full_bar(slot), tx);
        bulk_g2s(smem_addr(st + kXBytes), p.wt + unit * 8192, kWBytes, full_bar(slot));
        bulk_g2s(smem_addr(st + kXBytes + kWBytes), p.sz + unit * (p.sz_stage_bytes / 2), p.sz_stage_bytes, full_bar(slot));
        tma_load_3d(smem_addr(st), &tm_x, 0, 0, ks * 4, full_bar(slot));
        if (it == 0) XQT_TRACE_AT(3);
      }
      XQT_TRACE_AT(4);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      uint32_t it = 0;
      for (long long s = s_begin; s < s_end; ++s, ++it) {
        const int slot = it % ns;
        guarded_wait(full_bar(slot), (it / ns) & 1);
        if (it == 0) XQT_TRACE_AT(5);
        const uint32_t xbase = smem_addr(stages + (size_t)slot * p.stage_bytes);
#pragma unroll
        for (int u = 0; u < kUnits; ++u) {
          const int wg = u & 1;
          const uint32_t iw = it * kUnitsPerWg + (u >> 1);   // this warpgroup's unit counter
          const int buf = iw % kNB;
          guarded_wait(aready_bar(wg, buf), (iw / kNB) & 1);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < GK / 16; ++kk) {
            const int koff = u * GK + kk * 16;               // K offset inside the stage
            const uint64_t bdesc = umma_desc_sw128(xbase + (koff >> 6) * 2048 + (koff & 63) * 2);
            umma_ts_f16(tmem_base + d_col(wg, buf), tmem_base + a_col(wg, buf) + kk * 8, bdesc, kIdesc, kk != 0 ? 1u : 0u);
          }
          umma_commit(dready_bar(wg, buf));
          if (it == 0 && u == 0) XQT_TRACE_AT(6);
        }
        umma_commit(empty_bar(slot));   // all reads of this stage (weights by threads, activations by MMA) are done
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
    uint32_t iw = 0;        // units issued by this warpgroup
    uint32_t drained = 0;   // units already folded into acc; units [drained, iw) are in tensor memory
    float s_ring[kNB];      // their scales
#pragma unroll
    for (int i = 0; i < kNB; ++i) s_ring[i] = 0.f;

    auto drain = [&]() {
      // fold the oldest outstanding unit of this warpgroup into the running sums
      const uint32_t j = drained;
      const int buf = j % kNB;
      guarded_wait(dready_bar(wg, buf), (j / kNB) & 1);
      tc_fence_after();
      uint32_t r[16];
      tmem_ld_32x16(tmem_base + lane_addr + d_col(wg, buf), r);
      tmem_wait_ld();
      const float sc = buf == 0 ? s_ring[0] : (buf == 1 ? s_ring[1] : s_ring[2]);
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(sc, __uint_as_float(r[i]), acc[i]);
      ++drained;
    };

    uint32_t it = 0;
    for (long long s = s_begin; s < s_end; ++s, ++it) {
      const int slot = it % ns;
      const long long tile = s / p.spt;
      const int ks = (int)(s % p.spt);
      const unsigned char* st = stages + (size_t)slot * p.stage_bytes;
      guarded_wait(full_bar(slot), (it / ns) & 1);
#pragma unroll
      for (int uu = 0; uu < kUnitsPerWg; ++uu) {
        const int u = uu * 2 + wg;                       // unit of the stage handled by this warpgroup
        const int kb = (u * GK) >> 7;                    // 128-K block of the stage
        const int sub = ((u * GK) & 127) / GK;           // group inside the block
        // scale and zero point of (channel, group)
        const P* q = reinterpret_cast<const P*>(st + kXBytes + kWBytes) + ((size_t)(kb * (128 / GK) + sub) * kTileRows + ch) * 2;
        const float sc = to_float<P>(q[0]);
        const float zp = to_float<P>(q[1]);
        const uint32_t off2 = Tr::pair(Tr::kBase + zp + (SIGNED ? 8.f : 0.f));
        // packed weights: [kblock][chunk][channel][16 B]; a chunk is 32 K
        uint32_t cols[kColsPerUnit];
#pragma unroll
        for (int c = 0; c < GK / 32; ++c) {
          const int chunk = ((u * GK) & 127) / 32 + c;
          const uint4 v = *reinterpret_cast<const uint4*>(st + kXBytes + ((size_t)(kb * 4 + chunk) * kTileRows + ch) * 16);
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const uint32_t word = SIGNED ? (words[w] ^ 0x88888888u) : words[w];
#pragma unroll
            for (int i = 0; i < 4; ++i) cols[c * 16 + w * 4 + i] = dq_col<T>(word, i, off2);
          }
        }
        // buffer iw % kNB was last used by unit iw - kNB: make sure that one has been drained
        if (iw - drained >= (uint32_t)kNB) drain();
        const int buf = iw % kNB;
        const uint32_t a_addr = tmem_base + lane_addr + a_col(wg, buf);
#pragma unroll
        for (int c = 0; c < kColsPerUnit / 32; ++c) {
          uint32_t chunk32[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) chunk32[i] = cols[c * 32 + i];
          tmem_st_32x32(a_addr + c * 32, chunk32);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(aready_bar(wg, buf));
        if (buf == 0) s_ring[0] = sc; else if (buf == 1) s_ring[1] = sc; else s_ring[2] = sc;
        ++iw;
      }
      if (tid == 0 && it == 0) XQT_TRACE_AT(7);
      if (tid == 0 && s == s_end - 1) XQT_TRACE_AT(8);
      if (ks != p.spt - 1 && s != s_end - 1) continue;

      // ---------------------------------------------------------------- end of this CTA's run in `tile`
      while (drained < iw) drain();
      if (tid == 0 && s == s_end - 1) XQT_TRACE_AT(9);
      if (wg == 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) red[i * kTileRows + ch] = acc[i];
      }
      dq_sync();
      if (wg == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] += red[i * kTileRows + ch];
      }
      const long long t_first = tile * p.spt, t_last = t_first + p.spt - 1;
      const int c_first = cta_of_stage(t_first, p.total, grid), c_last = cta_of_stage(t_last, p.total, grid);
      bool finish = true;
      if (c_first != c_last) {
        const int seg = (s_begin / p.spt == tile) ? 0 : 1;
        float* mine = p.partials + ((size_t)cta * 2 + seg) * kPartialFloats;
        if (wg == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i < p.m) mine[i * kTileRows + ch] = acc[i];
          __threadfence();
        }
        dq_sync();
        if (tid == 0) s_flag = atomicAdd(&p.tickets[tile], 1u);
        dq_sync();
        finish = (s_flag == (unsigned int)(c_last - c_first));
        if (finish) {
          __threadfence();
          // the two warpgroups add alternate contributors (always in the same order), then combine
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = 0.f;
          // four contributors per batch: all their loads are in flight before the first add
          for (int c0 = c_first + wg; c0 <= c_last; c0 += 8) {
            float v[4][16];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int c = c0 + 2 * b;
              const int cseg = (((long long)c * p.total / grid) / p.spt == tile) ? 0 : 1;
              const float* src = p.partials + ((size_t)c * 2 + cseg) * kPartialFloats;
#pragma unroll
              for (int i = 0; i < 16; ++i) v[b][i] = (c <= c_last && i < p.m) ? __ldcg(src + i * kTileRows + ch) : 0.f;
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] += v[b][i];
            }
          }
          if (wg == 1) {
#pragma unroll
            for (int i = 0; i < 16; ++i) red[i * kTileRows + ch] = acc[i];
          }
          dq_sync();
          if (wg == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += red[i * kTileRows + ch];
          }
          if (tid == 0) p.tickets[tile] = 0u;
        }
      }
      if (finish && wg == 0) {
        const long long chn = tile * kTileRows + ch;
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
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    }
  }
  if (tid == 0) XQT_TRACE_AT(10);
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0) XQT_TRACE_AT(11);
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

template <typename T, typename P>
static int dtc_launch(const CUtensorMap& tm, const DecodeTcParams& p, int group_size, bool is_signed, int grid,
                      size_t smem_bytes, cudaStream_t stream) {
#define XQT_DTC(SG, GKV)                                                                                     \
  do {                                                                                                       \
    auto kern = w4a16_decode_tc_kernel<T, P, SG, GKV>;                                                       \
    static bool configured = false;                                                                          \
    if (!configured) {                                                                                       \
      XQT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dtc::kSmemBudget));   \
      configured = true;                                                                                     \
    }                                                                                                        \
    kern<<<grid, dtc::kThreads, smem_bytes, stream>>>(tm, p);                                                \
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
  int ns = (kSmemBudget - 1024 - kPartialFloats * 4) / p.stage_bytes;
  p.nstages = ns > kMaxStages ? kMaxStages : ns;
  XQT_REQUIRE(p.nstages >= 2);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<unsigned int*>(ws);
  p.tickets = reinterpret_cast<unsigned int*>(ws + 256);
  p.partials = reinterpret_cast<float*>(ws + 256 + (size_t)kMaxTiles * sizeof(unsigned int));
  long long grid = dtc_sm_count();
  if (grid > kMaxGrid) grid = kMaxGrid;
  if (grid > p.total) grid = p.total;
  const size_t smem_bytes = (size_t)p.nstages * p.stage_bytes + kPartialFloats * 4 + 1024;
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

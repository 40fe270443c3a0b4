// W4A4 SVDQuant / ConvRot GEMM on tcgen05:
//   Y[m,n] = sum_g a_s[m,g] w_s[n,g] * ( sum_{k in g} a_q[m,k] w_q[n,k] )  +  sum_r la[m,r] up[n,r]  + bias[n]
// with 64-K groups g, int4 codes on both sides, fp32 scales and an fp32 accumulation across groups.
//
// Blackwell has no int4 MMA: the activation codes arrive as int8 (written by the rotate+quantise
// prologue) and the weight nibbles are widened to int8 on the fly, as 16*w (a nibble moved to the
// high half of a byte IS the signed value times 16, no sign extension needed; the factor is folded
// into the weight scale).  Each 64-K slab is two tcgen05.mma kind::i8 steps into its own int32
// tensor-memory buffer (a ring of four); the epilogue warps drain every slab, convert exactly
// (|sum| <= 2^16) and fold it into fp32 register accumulators with a_s*w_s -- the per-slab scaling
// the reference does in half precision (jit/include/nunchaku/gemm_base.cuh:367-446,
// gemm_w4a4.cuh:833-930), here in fp32.  The rank-R branch and the bias are added at the end of
// the tile (reference: lora.cuh:110-243 "LoRA up").  That per-slab drain is CUDA-core work of
// M*N*K/64 scaled adds and bounds the kernel well below the int8 tensor peak; it is what exact
// per-group scales cost.
//
// Warp roles (448 threads): warp 0 TMA producer (activation codes, per-tile scales / low-rank
// factors), warp 1 MMA issuer, warps 2-9 epilogue (quarter = warp % 4, column half = (warp-2)/4),
// warps 10-13 weight unpack (one thread per weight row, bytes prefetched one stage ahead).
#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows);

namespace w4a4 {
constexpr int kBM = 128, kBN = 128, kStageK = 128, kGroup = 64, kRank = 32;
constexpr int kThreads = 448;
constexpr int kMaxStages = 6;
constexpr int kSlabBufs = 4;
constexpr int kABytes = kBM * 128, kBBytes = kBN * 128, kStageBytes = kABytes + kBBytes;
constexpr int kLaBytes = kBM * kRank * 4, kUpBytes = kBN * kRank * 4;
constexpr int kSmemBudget = 220 * 1024;
enum Status : unsigned int { kTimeout = 64 };
}  // namespace w4a4

struct W4A4Params {
  int m, n, k, groups;
  int mtiles, ntiles, kstages, stages, aux_bufs;
  int aux_tile_bytes;          // groups * 512 + kUpBytes
  const uint8_t* qweight;      // canonical signed nibbles [N, K/2]
  const float* a_scale;        // [M, groups]
  const uint8_t* aux;          // per n-tile: w_scale/16 as [groups][128] fp32, then up factors [128][32] fp32
  const float* la;             // [mtiles*128, 32] fp32 (zeros when there is no low-rank branch)
  const float* bias;
  void* out;
  unsigned int* status;
};

template <typename OutT>
__device__ __forceinline__ void w44_store8(OutT* dst, const float (&v)[8]);
template <>
__device__ __forceinline__ void w44_store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void w44_store8<__half>(__half* dst, const float (&v)[8]) {
  uint4 o;
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}

// two packed words (16 nibbles, k0..k15) -> 16 int8 values 16*w in K order
__device__ __forceinline__ uint4 widen16(uint32_t w0, uint32_t w1) {
  const uint32_t e0 = (w0 << 4) & 0xF0F0F0F0u, o0 = w0 & 0xF0F0F0F0u;
  const uint32_t e1 = (w1 << 4) & 0xF0F0F0F0u, o1 = w1 & 0xF0F0F0F0u;
  uint4 r;
  r.x = __byte_perm(e0, o0, 0x5140);
  r.y = __byte_perm(e0, o0, 0x7362);
  r.z = __byte_perm(e1, o1, 0x5140);
  r.w = __byte_perm(e1, o1, 0x7362);
  return r;
}

template <typename OutT>
__global__ void __launch_bounds__(w4a4::kThreads, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tm_a, const W4A4Params p) {
  using namespace w4a4;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[3 * kMaxStages + 2 * kSlabBufs + 4];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;

  constexpr uint32_t kTmemCols = kSlabBufs * kBN;   // 512
  constexpr uint32_t kIdesc = umma_idesc(kAccS32, kFmtS8, kFmtS8, kBM, kBN);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ns = p.stages;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  const int aux_bytes = p.aux_tile_bytes + kLaBytes;            // one buffer: w scales, up factors, la tile
  unsigned char* aux_base = tiles + (size_t)ns * kStageBytes;
  auto full_bar = [&](int s) { return smem_addr(&bars[s]); };
  auto bready_bar = [&](int s) { return smem_addr(&bars[kMaxStages + s]); };
  auto empty_bar = [&](int s) { return smem_addr(&bars[2 * kMaxStages + s]); };
  auto sfull_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + b]); };
  auto sempty_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + kSlabBufs + b]); };
  auto afull_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + 2 * kSlabBufs + b]); };
  auto aempty_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + 2 * kSlabBufs + 2 + b]); };

  if (threadIdx.x == 0) {
    s_abort = 0u;
    for (int s = 0; s < ns; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(bready_bar(s), 4);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < kSlabBufs; ++b) {
      mbar_init(sfull_bar(b), 1);
      mbar_init(sempty_bar(b), 8);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(afull_bar(b), 1);
      mbar_init(aempty_bar(b), 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tm_a);
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
  const int nab = p.aux_bufs;

  auto guarded_wait = [&](uint32_t bar, uint32_t parity) {
    if (s_abort == 0u && !mbar_wait(bar, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      uint32_t it = 0, local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const int mt = tile % p.mtiles, nt = tile / p.mtiles;
        const int ab = local % nab;
        guarded_wait(aempty_bar(ab), ((local / nab) & 1) ^ 1);
        unsigned char* ax = aux_base + (size_t)ab * aux_bytes;
        mbar_expect_tx(afull_bar(ab), aux_bytes);
        bulk_g2s(smem_addr(ax), p.aux + (size_t)nt * p.aux_tile_bytes, p.aux_tile_bytes, afull_bar(ab));
        bulk_g2s(smem_addr(ax + p.aux_tile_bytes), p.la + (size_t)mt * kBM * kRank, kLaBytes, afull_bar(ab));
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          const int s = it % ns;
          guarded_wait(empty_bar(s), ((it / ns) & 1) ^ 1);
          mbar_expect_tx(full_bar(s), kABytes);
          tma_load_2d(smem_addr(tiles + (size_t)s * kStageBytes), &tm_a, ks * kStageK, mt * kBM, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0, slab = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        for (int ks = 0; ks < p.kstages; ++ks, ++it) {
          const int s = it % ns;
          guarded_wait(bready_bar(s), (it / ns) & 1);
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr), bdesc = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int h = 0; h < 2; ++h, ++slab) {          // two 64-K slabs per stage
            const int sb = slab % kSlabBufs;
            guarded_wait(sempty_bar(sb), ((slab / kSlabBufs) & 1) ^ 1);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + sb * kBN;
            umma_ss<true>(d_tmem, adesc + h * 4, bdesc + h * 4, kIdesc, 0u);
            umma_ss<true>(d_tmem, adesc + h * 4 + 2, bdesc + h * 4 + 2, kIdesc, 1u);
            umma_commit(sfull_bar(sb));
          }
          umma_commit(empty_bar(s));
        }
      }
    }
  } else if (warp < 10) {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    uint32_t local = 0, slab = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int mt = tile % p.mtiles, nt = tile / p.mtiles;
      const int ab = local % nab;
      const int row_in_tile = quarter * 32 + lane;
      const int row = mt * kBM + row_in_tile;
      const float* sa = p.a_scale + (size_t)(row < p.m ? row : p.m - 1) * p.groups;
      guarded_wait(afull_bar(ab), (local / nab) & 1);
      const unsigned char* ax = aux_base + (size_t)ab * aux_bytes;
      const float* sw = reinterpret_cast<const float*>(ax) + half * 64;            // [groups][128]
      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      float sa_next = __ldg(sa);
      for (int g = 0; g < p.groups; ++g, ++slab) {
        const int sb = slab % kSlabBufs;
        const float sa_g = sa_next;
        if (g + 1 < p.groups) sa_next = __ldg(sa + g + 1);
        guarded_wait(sfull_bar(sb), (slab / kSlabBufs) & 1);
        tc_fence_after();
        const uint32_t taddr = tmem_base + sb * kBN + half * 64 + ((uint32_t)(quarter * 32) << 16);
        const float* swg = sw + (size_t)g * kBN;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_wait_ld();
          if (c == 1) {          // both halves are in registers: hand the buffer back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sempty_bar(sb));
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 w4 = *reinterpret_cast<const float4*>(swg + c * 32 + j * 4);
            const float ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // exact int -> float for |v| < 2^22: bias the exponent, subtract the bias
              const float f = __int_as_float((int)r[j * 4 + e] + 0x4B400000) - 12582912.f;
              acc[c * 32 + j * 4 + e] = fmaf(f, sa_g * ws[e], acc[c * 32 + j * 4 + e]);
            }
          }
        }
      }
      // rank-R branch, bias, store
      const float* la = reinterpret_cast<const float*>(ax + p.aux_tile_bytes) + row_in_tile * kRank;
      const float* up = reinterpret_cast<const float*>(ax + (size_t)p.groups * 512) + (size_t)half * 64 * kRank;
      float lar[kRank];
#pragma unroll
      for (int r4 = 0; r4 < kRank / 4; ++r4) {
        const float4 v = *reinterpret_cast<const float4*>(la + r4 * 4);
        lar[r4 * 4] = v.x; lar[r4 * 4 + 1] = v.y; lar[r4 * 4 + 2] = v.z; lar[r4 * 4 + 3] = v.w;
      }
      const int col0 = nt * kBN + half * 64;
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // fully unrolled: acc[] must stay in registers
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float* u = up + (size_t)(j * 8 + e) * kRank;
          float s = 0.f;
#pragma unroll
          for (int r4 = 0; r4 < kRank / 4; ++r4) {
            const float4 uu = *reinterpret_cast<const float4*>(u + r4 * 4);
            s = fmaf(lar[r4 * 4], uu.x, s); s = fmaf(lar[r4 * 4 + 1], uu.y, s);
            s = fmaf(lar[r4 * 4 + 2], uu.z, s); s = fmaf(lar[r4 * 4 + 3], uu.w, s);
          }
          v[e] = acc[j * 8 + e] + s;
        }
        const int col = col0 + j * 8;
        if (row < p.m && col < p.n) {
          if (p.bias != nullptr) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += __ldg(p.bias + col + e);
          }
          w44_store8<OutT>(out + (size_t)row * p.n + col, v);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(aempty_bar(ab));
    }
  } else {
    // ---------------------------------------------------------------- weight unpack warps (one thread per row)
    const int row_in_tile = threadIdx.x - 10 * 32;   // 0..127
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int nt = tile / p.mtiles;
      int row = nt * kBN + row_in_tile;
      row = row < p.n ? row : p.n - 1;
      const uint4* wrow = reinterpret_cast<const uint4*>(p.qweight + (size_t)row * (p.k / 2));
      uint4 nxt[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) nxt[c] = __ldg(wrow + c);
      for (int ks = 0; ks < p.kstages; ++ks, ++it) {
        const int s = it % ns;
        uint4 cur[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) cur[c] = nxt[c];
        if (ks + 1 < p.kstages) {
#pragma unroll
          for (int c = 0; c < 4; ++c) nxt[c] = __ldg(wrow + (size_t)(ks + 1) * 4 + c);
        }
        guarded_wait(full_bar(s), (it / ns) & 1);
        unsigned char* brow = tiles + (size_t)s * kStageBytes + kABytes + row_in_tile * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {          // 16 raw bytes = 32 K = two 16-byte chunks of the swizzled row
          const int j0 = c * 2;
          *reinterpret_cast<uint4*>(brow + (((j0) ^ (row_in_tile & 7)) << 4)) = widen16(cur[c].x, cur[c].y);
          *reinterpret_cast<uint4*>(brow + (((j0 + 1) ^ (row_in_tile & 7)) << 4)) = widen16(cur[c].z, cur[c].w);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bready_bar(s));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ----------------------------------------------------------------------------------------- host

bool w4a4_gemm_supported(int m, int n, int k) { return m >= 1 && n % 8 == 0 && k % 128 == 0 && k / 64 <= 160; }

size_t w4a4_aux_tile_bytes(int k) { return (size_t)(k / 64) * 512 + w4a4::kUpBytes; }

template <typename OutT>
static int launch_w4a4(const void* a_codes, W4A4Params p, cudaStream_t stream) {
  using namespace w4a4;
  CUtensorMap tm_a;
  XQT_CUDA((cudaError_t)make_tile_map(&tm_a, a_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.m, p.k, kBM));
  const int aux_bytes = p.aux_tile_bytes + kLaBytes;
  // two aux buffers when at least three stages still fit, else one
  int nab = 2;
  int stages = (kSmemBudget - 1024 - nab * aux_bytes) / kStageBytes;
  if (stages < 3) {
    nab = 1;
    stages = (kSmemBudget - 1024 - aux_bytes) / kStageBytes;
  }
  XQT_REQUIRE(stages >= 2);
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  p.aux_bufs = nab;
  p.mtiles = ceil_div(p.m, kBM);
  p.ntiles = ceil_div(p.n, kBN);
  p.kstages = p.k / kStageK;
  const size_t smem_bytes = (size_t)p.stages * kStageBytes + (size_t)nab * aux_bytes + 1024;
  auto kern = gemm_w4a4_kernel<OutT>;
  XQT_SMEM_OPT_IN(kern, kSmemBudget);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms > 0 ? sms : 148;
  if (grid > p.mtiles * p.ntiles) grid = p.mtiles * p.ntiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, p);
  return launch_status();
}

int w4a4_gemm_launch(const void* a_codes, const float* a_scale, const void* qweight, const void* aux, const float* la,
                     const float* bias, void* out, int m, int n, int k, int out_dtype, unsigned int* status,
                     cudaStream_t stream) {
  XQT_REQUIRE(w4a4_gemm_supported(m, n, k));
  XQT_REQUIRE(a_codes != nullptr && a_scale != nullptr && qweight != nullptr && aux != nullptr && la != nullptr &&
              out != nullptr && status != nullptr);
  XQT_REQUIRE(((uintptr_t)qweight & 15) == 0 && ((uintptr_t)aux & 15) == 0 && ((uintptr_t)la & 15) == 0 &&
              ((uintptr_t)out & 15) == 0);
  W4A4Params p{};
  p.m = m; p.n = n; p.k = k; p.groups = k / 64;
  p.aux_tile_bytes = (int)w4a4_aux_tile_bytes(k);
  p.qweight = (const uint8_t*)qweight; p.a_scale = a_scale; p.aux = (const uint8_t*)aux; p.la = la; p.bias = bias;
  p.out = out; p.status = status;
  if (out_dtype == XQT_B200_BF16) return launch_w4a4<__nv_bfloat16>(a_codes, p, stream);
  XQT_REQUIRE(out_dtype == XQT_B200_FP16);
  return launch_w4a4<__half>(a_codes, p, stream);
}

}  // namespace xqt_b200

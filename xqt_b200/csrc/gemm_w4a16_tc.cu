// W4A16 GEMM for M > 16 on tcgen05: Y[M,N] = X[M,K] * dequant(W)[N,K]^T, weights read straight from
// the canonical xqt_int4_nk_v1 bytes.
//
// Per 64-K stage: TMA brings the activation tile [128 x 64] (128-byte swizzle); eight dequantisation
// warps (one thread per weight row, its packed bytes prefetched one stage ahead with 16-byte loads) turn the
// nibbles into fp16 values (code - zero) * scale and store them in the 128-byte-swizzled K-major
// layout tcgen05 reads; one thread issues the MMAs; fp32 accumulators live in tensor memory,
// double-buffered so the epilogue (bias, residual, cast, store) of one tile overlaps the next.
//
// Precision.  (code - zero) is formed exactly (the zero point is folded into the magic-number
// subtraction) and multiplied by the scale with ONE rounding to fp16 (11-bit significand): a
// relative error of at most 2^-12 per weight, i.e. ~1e-4 rel-L2 on the output, against the 1e-3
// bar; rounding the weights to bf16 (8-bit significand) instead would cost ~8e-4.  Both MMA
// operands are therefore fp16: bf16 activations are first converted to fp16 by a small
// element-wise kernel into the caller's scratch buffer, once per call rather than once per weight
// tile: exact for 2^-14 <= |x| <= 65504 (smaller values lose bits to fp16's subnormals), NaN kept,
// anything larger clamped to +-65504 with bit 256 set in the status word.
// Envelope: group size 64 or 128, K a multiple of 64, integer zero points; anything else is served
// by the generic CUDA-core kernel.  Reference arithmetic: xqt/kernels/ops/gemm/reference.py:263-271,527.
#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"
#include <type_traits>

namespace xqt_b200 {

using namespace sm100;

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows);

namespace w4gemm {
constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 448;   // producer, MMA, 4 epilogue warps, 8 dequantisation warps
constexpr int kMaxStages = 6;
constexpr int kSmemBudget = 216 * 1024;
enum Status : unsigned int { kTimeout = 48 };
}  // namespace w4gemm

struct W4GemmParams {
  int m, n, k, group_size, groups;
  int mtiles, ntiles, kblocks, stages;
  int param_dtype, nibble_signed, out_f32;
  const uint8_t* qweight;   // canonical [N, K/2]
  const void* scales;
  const void* zeros;
  const float* bias;
  const void* residual;
  void* out;
  unsigned int* status;
};

template <typename OutT>
__device__ __forceinline__ void w4_store8(OutT* dst, const float (&v)[8]);
template <>
__device__ __forceinline__ void w4_store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void w4_store8<__half>(__half* dst, const float (&v)[8]) {
  uint4 o;
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}

template <typename T>
__device__ __forceinline__ void load8(const T* src, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = to_float<T>(e[i]);
}

// 8 nibbles of `word` (k0..k7, canonical order) -> fp16 (code - zero) * scale as 4 registers in K order
__device__ __forceinline__ uint4 dequant_word(uint32_t word, __half2 off2, __half2 scale2) {
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

template <int BN, typename T>
__global__ void __launch_bounds__(w4gemm::kThreads, 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tm_a, const W4GemmParams p) {
  using namespace w4gemm;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[3 * kMaxStages + 4];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;

  constexpr int kABytes = kBM * 128, kBBytes = BN * 128;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kIdesc = umma_idesc(kAccF32, kFmtF16, kFmtF16, kBM, BN);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ns = p.stages;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  auto full_bar = [&](int s) { return smem_addr(&bars[s]); };
  auto bready_bar = [&](int s) { return smem_addr(&bars[kMaxStages + s]); };
  auto empty_bar = [&](int s) { return smem_addr(&bars[2 * kMaxStages + s]); };
  auto tfull_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + b]); };
  auto tempty_bar = [&](int b) { return smem_addr(&bars[3 * kMaxStages + 2 + b]); };

  if (threadIdx.x == 0) {
    s_abort = 0u;
    for (int s = 0; s < ns; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(bready_bar(s), 8);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
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

  auto guarded_wait = [&](uint32_t bar, uint32_t parity) {
    if (s_abort == 0u && !mbar_wait(bar, parity)) {
      s_abort = 1u;
      atomicExch(p.status, (unsigned int)kTimeout);
    }
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int m0 = (tile % p.mtiles) * kBM;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % ns;
          guarded_wait(empty_bar(s), ((it / ns) & 1) ^ 1);
          unsigned char* st = tiles + (size_t)s * kStageBytes;
          mbar_expect_tx(full_bar(s), kABytes);
          tma_load_2d(smem_addr(st), &tm_a, kb * kBK, m0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t local = 0, phase = 0;
      int s = 0;
      bool ready = false;   // the current stage's barrier has already been seen complete
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        guarded_wait(tempty_bar(buf), ((local >> 1) & 1) ^ 1);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const bool last_tile = tile + (int)gridDim.x >= total_tiles;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!ready) guarded_wait(bready_bar(s), phase);   // weights dequantised (and the activation tile landed)
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr), bdesc = umma_desc_sw128(a_addr + kABytes);
          int sn = s + 1;
          uint32_t pn = phase;
          if (sn == ns) { sn = 0; pn ^= 1; }
          // four K steps, the commit that frees the stage, and the poll of the next stage's barrier
          // (its 150-cycle round trip runs while the MMAs are issued)
          ready = umma_ss_x4_commit_poll<false>(d_tmem, adesc, bdesc, kIdesc, kb != 0 ? 1u : 0u, empty_bar(s), bready_bar(sn), pn);
          if (last_tile && kb == p.kblocks - 1) ready = false;
          s = sn;
          phase = pn;
        }
        umma_commit(tfull_bar(buf));
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;
    T* out = reinterpret_cast<T*>(p.out);
    const T* res = reinterpret_cast<const T*>(p.residual);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % p.mtiles) * kBM, n0 = (tile / p.mtiles) * BN;
      guarded_wait(tfull_bar(buf), (local >> 1) & 1);
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row < p.m) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = n0 + c * 32 + j * 8;
            if (col < p.n) {   // N is a multiple of 8
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
              if (p.bias != nullptr) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += __ldg(p.bias + col + e);
              }
              if (res != nullptr) {
                float rv[8];
                load8<T>(res + (size_t)row * p.n + col, rv);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += rv[e];
              }
              if (p.out_f32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)row * p.n + col);
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                w4_store8<T>(out + (size_t)row * p.n + col, v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  } else {
    // ---------------------------------------------------------------- dequantisation warps
    const int dt = threadIdx.x - 6 * 32;                 // 0..255
    const int row_in_tile = dt % BN;
    constexpr int kChunks = BN == 256 ? 2 : 1;           // 16-byte raw chunks (32 K) per thread and stage
    const int chunk0 = (dt / BN) * kChunks;
    const float zbase = 1024.f + (p.nibble_signed ? 8.f : 0.f);
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int n0 = (tile / p.mtiles) * BN;
      int row = n0 + row_in_tile;
      row = row < p.n ? row : p.n - 1;
      const size_t prow = (size_t)row * p.groups;
      // this thread's packed weights: 16 bytes (32 K) per chunk, read straight from the canonical row
      const uint4* wrow = reinterpret_cast<const uint4*>(p.qweight + (size_t)row * (p.k / 2)) + chunk0;
      int g_cur = -1;
      __half2 off2 = __float2half2_rn(zbase), scale2 = __float2half2_rn(0.f);
      uint4 nxt[kChunks];
#pragma unroll
      for (int c = 0; c < kChunks; ++c) nxt[c] = __ldg(wrow + c);
      for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
        const int s = it % ns;
        uint4 cur[kChunks];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) cur[c] = nxt[c];
        if (kb + 1 < p.kblocks) {   // next stage's weights are in flight while this one is converted
#pragma unroll
          for (int c = 0; c < kChunks; ++c) nxt[c] = __ldg(wrow + (size_t)(kb + 1) * 2 + c);
        }
        const int g = (kb * kBK) / p.group_size;
        if (g != g_cur) {
          const float sc = load_param(p.scales, p.param_dtype, prow + g);
          const float zp = p.zeros != nullptr ? load_param(p.zeros, p.param_dtype, prow + g) : 0.f;
          off2 = __float2half2_rn(zbase + zp);
          scale2 = __float2half2_rn(sc);
          g_cur = g;
        }
        // the stage's B buffer is free once its full barrier has been armed and completed again
        guarded_wait(full_bar(s), (it / ns) & 1);
        unsigned char* st = tiles + (size_t)s * kStageBytes;
        unsigned char* brow = st + kABytes + row_in_tile * 128;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const uint32_t words[4] = {cur[c].x, cur[c].y, cur[c].z, cur[c].w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const uint32_t word = p.nibble_signed ? (words[w] ^ 0x88888888u) : words[w];
            const int j = (chunk0 + c) * 4 + w;          // 16-byte chunk of the 128-byte row, K order
            *reinterpret_cast<uint4*>(brow + ((j ^ (row_in_tile & 7)) << 4)) = dequant_word(word, off2, scale2);
          }
        }
        fence_proxy_async();     // make the generic-proxy stores visible to the tensor core's reads
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

// bf16 -> fp16, 8 elements per thread.  NaN stays NaN.  A finite value (or infinity) beyond fp16's
// range is clamped to +-65504 and reported: the kernel ORs kActivationRange into the status word, so
// a caller that reads the status learns that the result is not the reference's.
constexpr unsigned int kActivationRange = 256;
__global__ void __launch_bounds__(256) bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ src, __half* __restrict__ dst, size_t n8,
                                                          unsigned int* __restrict__ status) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
  const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
  uint4 o;
  __half2* out = reinterpret_cast<__half2*>(&o);
  bool clipped = false;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = __bfloat1622float2(in[j]);
    clipped |= fabsf(f.x) > 65504.f || fabsf(f.y) > 65504.f;          // false for NaN
    f.x = f.x != f.x ? f.x : fminf(fmaxf(f.x, -65504.f), 65504.f);
    f.y = f.y != f.y ? f.y : fminf(fmaxf(f.y, -65504.f), 65504.f);
    out[j] = __floats2half2_rn(f.x, f.y);
  }
  reinterpret_cast<uint4*>(dst)[i] = o;
  if (clipped) atomicOr(status, kActivationRange);
}

// Canonical int4 weights -> fp16 [N, K] row-major, value = fp16((code - zero) * scale) computed in
// fp32 and rounded once.  One thread converts 32 weights (16 packed bytes -> 64 bytes).
template <typename P>
__global__ void __launch_bounds__(256) dequant_w4_f16_kernel(const uint8_t* __restrict__ qweight, const P* __restrict__ scales,
                                                            const P* __restrict__ zeros, __half* __restrict__ dst, int n,
                                                            int k, int group_size, int nibble_signed) {
  const int chunks = k / 32;                                   // 16-byte chunks per row
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n * chunks) return;
  const int row = (int)(i / chunks), c = (int)(i % chunks);
  const int g = (c * 32) / group_size;
  const size_t pi = (size_t)row * (k / group_size) + g;
  const float sc = to_float<P>(scales[pi]);
  const float zp = (zeros != nullptr ? to_float<P>(zeros[pi]) : 0.f) + (nibble_signed ? 8.f : 0.f);
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)row * (k / 2)) + c);
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  uint4* out = reinterpret_cast<uint4*>(dst + (size_t)row * k + (size_t)c * 32);
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t word = nibble_signed ? (words[w] ^ 0x88888888u) : words[w];   // two's complement -> code + 8
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = ((float)((word >> (8 * j)) & 15u) - zp) * sc;
      const float b = ((float)((word >> (8 * j + 4)) & 15u) - zp) * sc;
      h[j] = __floats2half2_rn(a, b);
    }
    out[w] = o;
  }
}

// From this M on the weights are dequantised once per call into an fp16 scratch and multiplied by the
// dense tcgen05 GEMM.  Measured on the 4096 x 14336 MLP block the two passes beat the fused
// single-pass kernel at every M above the decode range (261 vs 328 us at M = 64, 342 vs 474 us at
// M = 512, 1250 vs 2560 us at M = 4096), so the default threshold is the first M the decode kernels do
// not serve; the single-pass kernel stays reachable as its own variant (no N*K*2 scratch).
// XQT_B200_TWO_PASS_MIN_M in the environment moves the threshold (read once; tuning and tests).
static int dense_min_m() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("XQT_B200_TWO_PASS_MIN_M");
    const int parsed = e != nullptr ? atoi(e) : 0;
    v = parsed >= 17 ? parsed : 17;
  }
  return v;
}

// [0,256) status, [256, 256+16 KiB) reserved for the ticket area of the M <= 16 kernel that shares this
// workspace, then the fp16 copy of bf16 activations
constexpr size_t kScratchOffset = 256 + 16384;
size_t w4a16_gemm_tc_workspace_bytes(int m, int n, int k) {
  size_t bytes = kScratchOffset + (((size_t)m * k * 2 + 255) & ~(size_t)255);
  if (m >= dense_min_m()) bytes += (size_t)n * k * 2;   // fp16 weights of the two-pass form
  return bytes;
}
bool w4a16_gemm_tc_any_zero_point(int m) { return m >= dense_min_m(); }

int gemm_f16_launch(const void* a, const void* b, const float* bias, const void* residual, void* out, int m, int n,
                    int k, int out_dtype, int out_f32, unsigned int* status, cudaStream_t stream);

bool w4a16_gemm_tc_supported(int m, int n, int k, int padded_k, int group_size) {
  return m >= 1 && n % 8 == 0 && k == padded_k && k % 64 == 0 && (group_size == 64 || group_size == 128);
}

template <int BN, typename T>
static int launch_w4gemm(const void* x, const void* qw, W4GemmParams p, cudaStream_t stream) {
  using namespace w4gemm;
  CUtensorMap tm_a;
  XQT_CUDA((cudaError_t)make_tile_map(&tm_a, x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.m, p.k, kBM));
  p.qweight = reinterpret_cast<const uint8_t*>(qw);
  constexpr int stage_bytes = kBM * 128 + BN * 128;
  int stages = (kSmemBudget - 1024) / stage_bytes;
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  p.mtiles = ceil_div(p.m, kBM);
  p.ntiles = ceil_div(p.n, BN);
  p.kblocks = p.k / kBK;
  const size_t smem_bytes = (size_t)p.stages * stage_bytes + 1024;
  auto kern = gemm_w4a16_kernel<BN, T>;
  XQT_SMEM_OPT_IN(kern, kSmemBudget);
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = sms > 0 ? sms : 148;
  if (grid > p.mtiles * p.ntiles) grid = p.mtiles * p.ntiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, p);
  return launch_status();
}

int w4a16_gemm_tc_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                         const void* residual, void* out, int m, int n, int k, int group_size, int nibble_signed,
                         int act_dtype, int param_dtype, int out_f32, int single_pass, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream) {
  XQT_REQUIRE(w4a16_gemm_tc_supported(m, n, k, k, group_size));
  const bool two_pass = !single_pass && m >= dense_min_m();
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= 256 && ((uintptr_t)out & 15) == 0);
  unsigned int* status = reinterpret_cast<unsigned int*>(workspace);
  unsigned char* scratch = reinterpret_cast<unsigned char*>(workspace) + kScratchOffset;
  if (two_pass) XQT_REQUIRE(workspace_bytes >= w4a16_gemm_tc_workspace_bytes(m, n, k));
  else if (act_dtype == XQT_B200_BF16) XQT_REQUIRE(workspace_bytes >= kScratchOffset + (size_t)m * k * 2);
  if (act_dtype == XQT_B200_BF16) {
    __half* x16 = reinterpret_cast<__half*>(scratch);
    const size_t n8 = (size_t)m * k / 8;
    bf16_to_f16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x, x16, n8, status);
    XQT_CUDA(cudaGetLastError());
    x = x16;
  }
  if (two_pass) {
    // two passes: weights -> fp16 scratch (any zero point, fp32 arithmetic), then the dense GEMM
    __half* w16 = reinterpret_cast<__half*>(scratch + (((size_t)m * k * 2 + 255) & ~(size_t)255));
    const size_t threads = (size_t)n * (k / 32);
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    if (param_dtype == XQT_B200_BF16)
      dequant_w4_f16_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const uint8_t*)qw, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)zeros, w16, n, k, group_size, nibble_signed);
    else if (param_dtype == XQT_B200_FP16)
      dequant_w4_f16_kernel<__half><<<blocks, 256, 0, stream>>>((const uint8_t*)qw, (const __half*)scales, (const __half*)zeros, w16, n, k, group_size, nibble_signed);
    else
      dequant_w4_f16_kernel<float><<<blocks, 256, 0, stream>>>((const uint8_t*)qw, (const float*)scales, (const float*)zeros, w16, n, k, group_size, nibble_signed);
    XQT_CUDA(cudaGetLastError());
    return gemm_f16_launch(x, w16, bias, residual, out, m, n, k, act_dtype, out_f32, status, stream);
  }
  W4GemmParams p{};
  p.m = m; p.n = n; p.k = k; p.group_size = group_size; p.groups = k / group_size;
  p.param_dtype = param_dtype; p.nibble_signed = nibble_signed; p.out_f32 = out_f32;
  XQT_REQUIRE(!out_f32 || residual == nullptr);
  p.scales = scales; p.zeros = zeros; p.bias = bias; p.residual = residual; p.out = out; p.status = status;
  const bool wide = n % 256 == 0 && (long long)ceil_div(m, 128) * (n / 256) >= 148;
  if (act_dtype == XQT_B200_BF16)
    return wide ? launch_w4gemm<256, __nv_bfloat16>(x, qw, p, stream) : launch_w4gemm<128, __nv_bfloat16>(x, qw, p, stream);
  return wide ? launch_w4gemm<256, __half>(x, qw, p, stream) : launch_w4gemm<128, __half>(x, qw, p, stream);
}

}  // namespace xqt_b200

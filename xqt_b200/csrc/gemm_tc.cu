// Tensor-core GEMM core for sm_100a: TMA-staged operands in 128-byte-swizzled shared memory,
// tcgen05.mma issued by one thread, fp32 / int32 accumulators in tensor memory, a persistent tile
// loop and double-buffered accumulators so the epilogue of one tile overlaps the main loop of the
// next.  Y[M,N] = A[M,K] * B[N,K]^T with both operands K-major.
//
// Warp roles (192 threads, one CTA per SM):
//   warp 0      TMA producer: one elected thread arms the stage barrier and issues two tiled loads
//   warp 1      allocates tensor memory; one elected thread issues the MMAs and commits
//   warps 2..5  epilogue: each owns one 32-lane quarter of tensor memory (quarter = warp % 4)
//
// This file holds the int8 instantiation (W8A8: kind::i8, int32 accumulators over the whole K,
// epilogue acc * a_scale[m] * w_scale[n] in fp32, the arithmetic of xqt's per-token int8 contract,
// xqt/kernels/ops/gemm/reference.py:278-323 and quantize.py:60-131 written in its integer form).
#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

namespace gemm {
constexpr int kBM = 128;
constexpr int kRowBytes = 128;           // one swizzle row: 128 int8 or 64 16-bit elements of K
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 208 * 1024;
enum Status : unsigned int { kOk = 0, kTimeout = 16 };
}  // namespace gemm

struct GemmTcParams {
  int m, n, k;
  int mtiles, ntiles, kblocks, stages;
  const float* row_scale;   // [M]  activation scale per token
  const float* col_scale;   // [N]  weight scale per output channel
  const float* bias;        // [N] or null
  void* out;                // [M, N]
  unsigned int* status;
};

template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* dst, const float (&v)[8]) {
  uint4 o;
  __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
  __half2 c = __floats2half2_rn(v[4], v[5]), d = __floats2half2_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  *reinterpret_cast<uint4*>(dst) = o;
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmTcParams p) {
  using namespace gemm;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + 4];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;

  constexpr int kABytes = kBM * kRowBytes, kBBytes = BN * kRowBytes, kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kIdesc = umma_idesc(kAccS32, kFmtS8, kFmtS8, kBM, BN);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ns = p.stages;
  // dynamic shared memory is only guaranteed 16-byte aligned by the launch: align by hand
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  auto full_bar = [&](int s) { return smem_addr(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_addr(&bars[kMaxStages + s]); };
  auto tfull_bar = [&](int b) { return smem_addr(&bars[2 * kMaxStages + b]); };
  auto tempty_bar = [&](int b) { return smem_addr(&bars[2 * kMaxStages + 2 + b]); };

  if (threadIdx.x == 0) {
    s_abort = 0u;
    for (int s = 0; s < ns; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
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
        const int m0 = (tile % p.mtiles) * kBM, n0 = (tile / p.mtiles) * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % ns;
          guarded_wait(empty_bar(s), ((it / ns) & 1) ^ 1);
          unsigned char* st = tiles + (size_t)s * kStageBytes;
          mbar_expect_tx(full_bar(s), kStageBytes);
          tma_load_2d(smem_addr(st), &tm_a, kb * kRowBytes, m0, full_bar(s));
          tma_load_2d(smem_addr(st + kABytes), &tm_b, kb * kRowBytes, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0, local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        guarded_wait(tempty_bar(buf), ((local >> 1) & 1) ^ 1);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % ns;
          guarded_wait(full_bar(s), (it / ns) & 1);
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr), bdesc = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kRowBytes / 32; ++k)  // 32 bytes of K per MMA: the descriptor start advances by 2 units
            umma_ss<true>(d_tmem, adesc + 2 * k, bdesc + 2 * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar(s));     // the stage is free once these MMAs have read it
        }
        umma_commit(tfull_bar(buf));      // accumulator complete
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % p.mtiles) * kBM, n0 = (tile / p.mtiles) * BN;
      guarded_wait(tfull_bar(buf), (local >> 1) & 1);
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const float rs = row < p.m ? __ldg(p.row_scale + row) : 0.f;
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
              for (int e = 0; e < 8; ++e) {
                v[e] = (float)(int)r[j * 8 + e] * (rs * __ldg(p.col_scale + col + e));
                if (p.bias != nullptr) v[e] += __ldg(p.bias + col + e);
              }
              store8<OutT>(out + (size_t)row * p.n + col, v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ----------------------------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// row-major [rows, cols] matrix of `esize`-byte elements; box = 128 bytes of a row x box_rows rows,
// written to shared memory with the 128-byte swizzle; out-of-range elements read as zero
int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if (((uintptr_t)base & 15) != 0 || (cols * esize) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static int sm_count_now() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  return v;
}

template <int BN, typename OutT>
static int launch_i8(const void* a, const void* b, GemmTcParams p, cudaStream_t stream) {
  using namespace gemm;
  CUtensorMap tm_a, tm_b;
  XQT_CUDA((cudaError_t)make_tile_map(&tm_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.m, p.k, kBM));
  XQT_CUDA((cudaError_t)make_tile_map(&tm_b, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.n, p.k, BN));
  constexpr int stage_bytes = kBM * kRowBytes + BN * kRowBytes;
  int stages = (kSmemBudget - 1024) / stage_bytes;
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  p.mtiles = ceil_div(p.m, kBM);
  p.ntiles = ceil_div(p.n, BN);
  p.kblocks = ceil_div(p.k, kRowBytes);
  const size_t smem_bytes = (size_t)p.stages * stage_bytes + 1024;
  auto kern = gemm_i8_kernel<BN, OutT>;
  static bool configured = false;
  if (!configured) {
    XQT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    configured = true;
  }
  int grid = sm_count_now();
  if (grid > p.mtiles * p.ntiles) grid = p.mtiles * p.ntiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, tm_b, p);
  return launch_status();
}

// int8 A [M,K] x int8 B [N,K]^T, out = acc * row_scale[m] * col_scale[n] (+ bias[n])
int gemm_i8_launch(const void* a, const void* b, const float* row_scale, const float* col_scale, const float* bias,
                   void* out, int m, int n, int k, int out_dtype, unsigned int* status, cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 16 == 0 && n % 8 == 0);
  XQT_REQUIRE(out_dtype == XQT_B200_BF16 || out_dtype == XQT_B200_FP16);
  XQT_REQUIRE(a != nullptr && b != nullptr && row_scale != nullptr && col_scale != nullptr && out != nullptr && status != nullptr);
  XQT_REQUIRE(((uintptr_t)out & 15) == 0);
  GemmTcParams p{};
  p.m = m; p.n = n; p.k = k;
  p.row_scale = row_scale; p.col_scale = col_scale; p.bias = bias; p.out = out; p.status = status;
  const bool wide = (n % 256 == 0);
  if (out_dtype == XQT_B200_BF16)
    return wide ? launch_i8<256, __nv_bfloat16>(a, b, p, stream) : launch_i8<128, __nv_bfloat16>(a, b, p, stream);
  return wide ? launch_i8<256, __half>(a, b, p, stream) : launch_i8<128, __half>(a, b, p, stream);
}

}  // namespace xqt_b200

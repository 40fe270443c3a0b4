// Tensor-core GEMM core for sm_100a: TMA-staged operands in 128-byte-swizzled shared memory,
// tcgen05.mma issued by one thread, fp32 / int32 accumulators in tensor memory, a persistent tile
// loop and double-buffered accumulators so the epilogue of one tile overlaps the main loop of the
// next.  Y[M,N] = A[M,K] * B[N,K]^T with both operands K-major.
//
// Warp roles (192 threads, one CTA per SM):
//   warp 0      TMA producer: one elected thread arms the stage barrier and issues two tiled loads
//   warp 1      allocates tensor memory; one elected thread issues the MMAs and commits
//   warps 2..9  epilogue: each owns one 32-lane quarter of tensor memory (quarter = warp % 4) and one
//               half of the tile's columns (warps 2-5 the left half, 6-9 the right half)
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
constexpr int kThreads = 320;            // producer, MMA issuer, 8 epilogue warps
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
  const void* residual;     // [M, N] in the output dtype or null (fp16 kind only)
  const float* addend;      // [M, N] fp32 or null (int8 kind only): added before the one rounding (a low-rank branch)
  int out_f32;              // fp16 kind only: 1 = the output is fp32 (partial sums of a K-sharded layer)
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

// KIND 0: int8 operands, int32 accumulators, scaled epilogue.  KIND 1 / 2: fp16 / bf16 operands (both
// sides the same format), fp32 accumulators, epilogue acc (+ bias) (+ residual).
template <int BN, typename OutT, int KIND>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmTcParams& p) {
  using namespace gemm;
  constexpr bool I8 = KIND == 0;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + 4];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile unsigned int s_abort;

  constexpr int kABytes = kBM * kRowBytes, kBBytes = BN * kRowBytes, kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kIdesc = I8 ? umma_idesc(kAccS32, kFmtS8, kFmtS8, kBM, BN)
                                 : (KIND == 1 ? umma_idesc(kAccF32, kFmtF16, kFmtF16, kBM, BN) : umma_idesc(kAccF32, kFmtBF16, kFmtBF16, kBM, BN));
  constexpr int kElemsPerRow = I8 ? kRowBytes : kRowBytes / 2;   // K elements per 128-byte swizzle row

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
      mbar_init(tempty_bar(b), 8);
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
          tma_load_2d(smem_addr(st), &tm_a, kb * kElemsPerRow, m0, full_bar(s));
          tma_load_2d(smem_addr(st + kABytes), &tm_b, kb * kElemsPerRow, n0, full_bar(s));
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
          if (!ready) guarded_wait(full_bar(s), phase);
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * kStageBytes);
          const uint64_t adesc = umma_desc_sw128(a_addr), bdesc = umma_desc_sw128(a_addr + kABytes);
          // the next stage in ring order (the first of the next tile after the last K block)
          int sn = s + 1;
          uint32_t pn = phase;
          if (sn == ns) { sn = 0; pn ^= 1; }
          // four 32-byte K steps, the commit that frees the stage, and the poll of the next stage's
          // barrier in one go: the poll's round trip is hidden behind the MMA issue
          ready = umma_ss_x4_commit_poll<I8>(d_tmem, adesc, bdesc, kIdesc, kb != 0 ? 1u : 0u, empty_bar(s), full_bar(sn), pn);
          if (last_tile && kb == p.kblocks - 1) ready = false;
          s = sn;
          phase = pn;
        }
        umma_commit(tfull_bar(buf));      // accumulator complete
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % p.mtiles) * kBM, n0 = (tile / p.mtiles) * BN;
      guarded_wait(tfull_bar(buf), (local >> 1) & 1);
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      float rs = 0.f;
      if (I8) rs = row < p.m ? __ldg(p.row_scale + row) : 0.f;
      const OutT* res = reinterpret_cast<const OutT*>(p.residual);
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_wait_ld();
        if (row < p.m) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = n0 + c * 32 + j * 8;
            if (col < p.n) {   // N is a multiple of 8
              float v[8];
              if (I8) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  v[e] = (float)(int)r[j * 8 + e] * (rs * __ldg(p.col_scale + col + e));
                  if (p.bias != nullptr) v[e] += __ldg(p.bias + col + e);
                }
                if (p.addend != nullptr) {
                  const float4* add = reinterpret_cast<const float4*>(p.addend + (size_t)row * p.n + col);
                  const float4 a0 = __ldg(add), a1 = __ldg(add + 1);
                  v[0] += a0.x; v[1] += a0.y; v[2] += a0.z; v[3] += a0.w;
                  v[4] += a1.x; v[5] += a1.y; v[6] += a1.z; v[7] += a1.w;
                }
                store8<OutT>(out + (size_t)row * p.n + col, v);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
                if (p.bias != nullptr) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += __ldg(p.bias + col + e);
                }
                if (res != nullptr) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(res + (size_t)row * p.n + col);
                  const OutT* re = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[e] += to_float<OutT>(re[e]);
                }
                if (p.out_f32) {
                  float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)row * p.n + col);
                  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                  dst[1] = make_float4(v[4], v[5], v[6], v[7]);
                } else {
                  store8<OutT>(out + (size_t)row * p.n + col, v);
                }
              }
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

template <int BN, typename OutT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmTcParams p) {
  gemm_tc_body<BN, OutT, 0>(tm_a, tm_b, p);
}

// fp16 x fp16 -> fp32: the second pass of the W4A16 linear at large M (weights dequantised once per
// call into an fp16 scratch by dequant_w4_f16_kernel)
template <int BN, typename OutT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmTcParams p) {
  gemm_tc_body<BN, OutT, 1>(tm_a, tm_b, p);
}

// bf16 x bf16 -> fp32 (the rank-32 down projection of the rotated activations)
template <int BN, typename OutT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmTcParams p) {
  gemm_tc_body<BN, OutT, 2>(tm_a, tm_b, p);
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
int make_tile_map_ld(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                     long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if (((uintptr_t)base & 15) != 0 || (ld * esize) % 16 != 0 || ld < cols) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// unswizzled byte tile: `box_rows` rows of `box_bytes` bytes out of a [rows][row_bytes] byte matrix
int make_byte_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if (((uintptr_t)base & 15) != 0 || row_bytes % 16 != 0 || box_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows) {
  return make_tile_map_ld(map, base, dtype, esize, rows, cols, cols, box_rows);
}

static int sm_count_now() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  return v;
}

template <int BN, typename OutT, int KIND>
static int launch_tc(const void* a, long long lda, const void* b, long long ldb, GemmTcParams p, cudaStream_t stream) {
  using namespace gemm;
  CUtensorMap tm_a, tm_b;
  constexpr bool I8 = KIND == 0;
  const int esize = I8 ? 1 : 2;
  const CUtensorMapDataType dt = I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : (KIND == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  XQT_CUDA((cudaError_t)make_tile_map_ld(&tm_a, a, dt, esize, p.m, p.k, lda, kBM));
  XQT_CUDA((cudaError_t)make_tile_map_ld(&tm_b, b, dt, esize, p.n, p.k, ldb, BN));
  constexpr int stage_bytes = kBM * kRowBytes + BN * kRowBytes;
  int stages = (kSmemBudget - 1024) / stage_bytes;
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  p.mtiles = ceil_div(p.m, kBM);
  p.ntiles = ceil_div(p.n, BN);
  p.kblocks = ceil_div(p.k * esize, kRowBytes);
  const size_t smem_bytes = (size_t)p.stages * stage_bytes + 1024;
  void (*kern)(const CUtensorMap, const CUtensorMap, const GemmTcParams) =
      I8 ? gemm_i8_kernel<BN, OutT> : (KIND == 1 ? gemm_f16_kernel<BN, OutT> : gemm_bf16_kernel<BN, OutT>);
  XQT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
  int grid = sm_count_now();
  if (grid > p.mtiles * p.ntiles) grid = p.mtiles * p.ntiles;
  kern<<<grid, kThreads, smem_bytes, stream>>>(tm_a, tm_b, p);
  return launch_status();
}

// int8 A [M,K] x int8 B [N,K]^T, out = acc * row_scale[m] * col_scale[n] (+ bias[n]) (+ addend[m,n], fp32)
int gemm_i8_addend_launch(const void* a, const void* b, const float* row_scale, const float* col_scale, const float* bias,
                          const float* addend, void* out, int m, int n, int k, int out_dtype, unsigned int* status,
                          cudaStream_t stream);
int gemm_i8_launch(const void* a, const void* b, const float* row_scale, const float* col_scale, const float* bias,
                   void* out, int m, int n, int k, int out_dtype, unsigned int* status, cudaStream_t stream) {
  return gemm_i8_addend_launch(a, b, row_scale, col_scale, bias, nullptr, out, m, n, k, out_dtype, status, stream);
}
int gemm_i8_addend_launch(const void* a, const void* b, const float* row_scale, const float* col_scale, const float* bias,
                          const float* addend, void* out, int m, int n, int k, int out_dtype, unsigned int* status,
                          cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && n > 0 && k > 0 && k % 16 == 0 && n % 8 == 0 && ((uintptr_t)addend & 15) == 0);
  XQT_REQUIRE(out_dtype == XQT_B200_BF16 || out_dtype == XQT_B200_FP16);
  XQT_REQUIRE(a != nullptr && b != nullptr && row_scale != nullptr && col_scale != nullptr && out != nullptr && status != nullptr);
  XQT_REQUIRE(((uintptr_t)out & 15) == 0);
  GemmTcParams p{};
  p.m = m; p.n = n; p.k = k;
  p.row_scale = row_scale; p.col_scale = col_scale; p.bias = bias; p.addend = addend; p.out = out; p.status = status;
  const bool wide = (n % 256 == 0);
  if (out_dtype == XQT_B200_BF16)
    return wide ? launch_tc<256, __nv_bfloat16, 0>(a, k, b, k, p, stream) : launch_tc<128, __nv_bfloat16, 0>(a, k, b, k, p, stream);
  return wide ? launch_tc<256, __half, 0>(a, k, b, k, p, stream) : launch_tc<128, __half, 0>(a, k, b, k, p, stream);
}


// 16-bit A [M,K] x 16-bit B [N,K]^T (both fp16, or both bf16 with operand_bf16) with fp32
// accumulation; out = acc (+ bias[n]) (+ residual[m,n]) in bf16 / fp16 (out_dtype) or fp32 (out_f32).
// `lda` / `ldb` are the row strides in elements (>= k, multiples of 8).
int gemm_f16_launch_strided(const void* a, long long lda, const void* b, long long ldb, const float* bias,
                            const void* residual, void* out, int m, int n, int k, int out_dtype, int out_f32,
                            int operand_bf16, unsigned int* status, cudaStream_t stream);

int gemm_f16_launch(const void* a, const void* b, const float* bias, const void* residual, void* out, int m, int n,
                    int k, int out_dtype, int out_f32, unsigned int* status, cudaStream_t stream) {
  return gemm_f16_launch_strided(a, k, b, k, bias, residual, out, m, n, k, out_dtype, out_f32, 0, status, stream);
}

int gemm_f16_launch_strided(const void* a, long long lda, const void* b, long long ldb, const float* bias,
                            const void* residual, void* out, int m, int n, int k, int out_dtype, int out_f32,
                            int operand_bf16, unsigned int* status, cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && n > 0 && k > 0 && n % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && lda >= k && ldb >= k);
  XQT_REQUIRE(out_dtype == XQT_B200_BF16 || out_dtype == XQT_B200_FP16);
  XQT_REQUIRE(a != nullptr && b != nullptr && out != nullptr && status != nullptr && ((uintptr_t)out & 15) == 0);
  XQT_REQUIRE(!out_f32 || residual == nullptr);
  GemmTcParams p{};
  p.m = m; p.n = n; p.k = k;
  p.bias = bias; p.residual = residual; p.out_f32 = out_f32; p.out = out; p.status = status;
  const bool wide = (n % 256 == 0);
#define XQT_F16_GO(OUT, KIND) (wide ? launch_tc<256, OUT, KIND>(a, lda, b, ldb, p, stream) : launch_tc<128, OUT, KIND>(a, lda, b, ldb, p, stream))
  if (out_dtype == XQT_B200_BF16) return operand_bf16 ? XQT_F16_GO(__nv_bfloat16, 2) : XQT_F16_GO(__nv_bfloat16, 1);
  return operand_bf16 ? XQT_F16_GO(__half, 2) : XQT_F16_GO(__half, 1);
#undef XQT_F16_GO
}

}  // namespace xqt_b200

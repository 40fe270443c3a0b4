// Low-rank down projection of the SVDQuant linear: la[M, R] = x_rot[M, K] * L1[R, K]^T, fp32 out.
//
// It is the "LoRA down" step the reference fuses into its activation-quantisation kernel
// (jit/include/nunchaku/lora.cuh:110-243, gemm_w4a4.cuh:1149-1188): the rank-R branch is taken from
// the rotated, un-quantised activation.  R <= 32 makes this a skinny GEMM (1.3 % of the layer's
// flops); a warp computes a 16-row x 32-column strip over its share of K with mma.m16n8k16, both operands read
// straight from global memory with 16-byte loads.  K order inside an MMA is free as long as both
// operands agree, so lane t simply takes 8 consecutive K of its row for two consecutive MMA steps.
#include "common.cuh"

namespace xqt_b200 {

constexpr int kLrWarps = 4;

template <typename T>
__device__ __forceinline__ void lr_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1);
template <>
__device__ __forceinline__ void lr_mma<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void lr_mma<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                      uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// down: [32, K] (rows >= rank are zero), out: [M, 32] fp32 (may be null).  image (may be null): the same values as the
// W4A4 GEMM's tensor-core operand, one 16 KiB image per 128 rows: row r holds bf16 [hi(32) | lo(32)], hi = bf16(v),
// lo = bf16(v - hi), its eight 16-byte chunks stored at chunk index c ^ (r & 7) (128-byte swizzle).  A CTA owns 16 rows; its four warps take every fourth
// 32-K chunk each and add their partial strips through shared memory in warp order (M / 16 CTAs: 256 at M = 4096,
// enough to keep every SM streaming).
template <typename T>
__global__ void __launch_bounds__(kLrWarps * 32)
lowrank_down_kernel(const T* __restrict__ x, const T* __restrict__ down, float* __restrict__ out,
                    unsigned char* __restrict__ image, int m, int k) {
  __shared__ float part[kLrWarps][16][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  const int ra = min(row0 + g, m - 1), rb = min(row0 + g + 8, m - 1);
  const uint4* xa = reinterpret_cast<const uint4*>(x + (size_t)ra * k) + t;
  const uint4* xb = reinterpret_cast<const uint4*>(x + (size_t)rb * k) + t;
  const uint4* w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) w[j] = reinterpret_cast<const uint4*>(down + (size_t)(8 * j + g) * k) + t;
  float acc[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int chunks = k / 32;   // 32 K per iteration: 4 lanes x 8 K
#pragma unroll 4
  for (int c = warp; c < chunks; c += kLrWarps) {
    const uint4 a = __ldg(xa + c * 4), b = __ldg(xb + c * 4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v = __ldg(w[j] + c * 4);
      lr_mma<T>(acc[j], a.x, b.x, a.y, b.y, v.x, v.y);
      lr_mma<T>(acc[j], a.z, b.z, a.w, b.w, v.z, v.w);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int col = 8 * j + 2 * t;
    part[warp][g][col] = acc[j][0];
    part[warp][g][col + 1] = acc[j][1];
    part[warp][g + 8][col] = acc[j][2];
    part[warp][g + 8][col + 1] = acc[j][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * 32; i += kLrWarps * 32) {
    const int r = i >> 5, c = i & 31;
    if (row0 + r < m) {
      float s = 0.f;
#pragma unroll
      for (int wv = 0; wv < kLrWarps; ++wv) s += part[wv][r][c];
      if (out != nullptr) out[(size_t)(row0 + r) * 32 + c] = s;
      if (image != nullptr) {
        const int row = row0 + r;
        unsigned char* dst = image + (size_t)row * 128;        // tiles of 128 rows x 128 bytes are contiguous
        const __nv_bfloat16 hi = __float2bfloat16_rn(s), lo = __float2bfloat16_rn(s - __bfloat162float(hi));
        *reinterpret_cast<__nv_bfloat16*>(dst + ((((c >> 3)) ^ (row & 7)) << 4) + (c & 7) * 2) = hi;
        *reinterpret_cast<__nv_bfloat16*>(dst + ((((c >> 3) + 4) ^ (row & 7)) << 4) + (c & 7) * 2) = lo;
      }
    }
  }
}

int lowrank_down_launch(const void* x, const void* down, float* out, void* image, int m, int k, int act_dtype,
                        cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && k > 0 && k % 32 == 0 && (out != nullptr || image != nullptr));
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)down & 15) == 0 && ((uintptr_t)out & 7) == 0 && ((uintptr_t)image & 127) == 0);
  const int grid = ceil_div(m, 16);
  if (act_dtype == XQT_B200_BF16)
    lowrank_down_kernel<__nv_bfloat16><<<grid, kLrWarps * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)down, out, (unsigned char*)image, m, k);
  else
    lowrank_down_kernel<__half><<<grid, kLrWarps * 32, 0, stream>>>((const __half*)x, (const __half*)down, out, (unsigned char*)image, m, k);
  return launch_status();
}

}  // namespace xqt_b200

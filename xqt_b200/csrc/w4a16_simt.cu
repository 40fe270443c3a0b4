// Generic W4A16 kernel on CUDA cores: any M, N, K, group size, signedness, parameter dtype
// and the full epilogue.  It is the complete-but-slow member of the family, used for shapes
// outside the envelopes of the tensor-core kernels (ragged K, group sizes 32/64 at small M,
// gelu/silu epilogues) and as an independent device-side cross-check in the tests.
//
// Arithmetic is exactly the contract reference's: w = (code - zero) * scale evaluated in fp32
// (xqt/kernels/ops/gemm/reference.py:263-271), fp32 accumulation, bias -> residual ->
// activation -> one cast (reference.py:362-390).
#include "common.cuh"

namespace xqt_b200 {

constexpr int kSimtRowsPerBlock = 8;   // one warp per output channel
constexpr int kSimtMChunk = 8;         // activation rows accumulated per pass

template <typename T>
__global__ void __launch_bounds__(kSimtRowsPerBlock * 32)
w4a16_simt_kernel(const T* __restrict__ x, const uint8_t* __restrict__ qw, const void* __restrict__ scales,
                  const void* __restrict__ zeros, const float* __restrict__ bias,
                  const T* __restrict__ residual, T* __restrict__ out, int m, int n, int k,
                  int padded_k, int group_size, int nibble_signed, int param_dtype, int activation) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kSimtRowsPerBlock + (threadIdx.x >> 5);
  if (row >= n) return;
  const int row_bytes = (padded_k + 1) / 2;
  const int groups = padded_k / group_size;
  const uint8_t* wrow = qw + (size_t)row * row_bytes;
  const int kbytes = (k + 1) / 2;

  for (int m0 = 0; m0 < m; m0 += kSimtMChunk) {
    float acc[kSimtMChunk];
#pragma unroll
    for (int i = 0; i < kSimtMChunk; ++i) acc[i] = 0.f;
    for (int b = lane; b < kbytes; b += 32) {
      const int k0 = 2 * b;
      const uint8_t byte = wrow[b];
      int c0 = byte & 0x0F, c1 = byte >> 4;
      if (nibble_signed) {
        c0 = (c0 ^ 8) - 8;
        c1 = (c1 ^ 8) - 8;
      }
      const int g0 = k0 / group_size, g1 = (k0 + 1) / group_size;
      const float s0 = load_param(scales, param_dtype, (size_t)row * groups + g0);
      const float s1 = (g1 == g0) ? s0 : load_param(scales, param_dtype, (size_t)row * groups + (g1 < groups ? g1 : g0));
      float z0 = 0.f, z1 = 0.f;
      if (zeros != nullptr) {
        z0 = load_param(zeros, param_dtype, (size_t)row * groups + g0);
        z1 = (g1 == g0) ? z0 : load_param(zeros, param_dtype, (size_t)row * groups + (g1 < groups ? g1 : g0));
      }
      const float w0 = ((float)c0 - z0) * s0;
      const float w1 = (k0 + 1 < k) ? ((float)c1 - z1) * s1 : 0.f;
#pragma unroll
      for (int i = 0; i < kSimtMChunk; ++i) {
        if (m0 + i < m) {
          const T* xr = x + (size_t)(m0 + i) * k;
          acc[i] = fmaf(to_float<T>(xr[k0]), w0, acc[i]);
          if (k0 + 1 < k) acc[i] = fmaf(to_float<T>(xr[k0 + 1]), w1, acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kSimtMChunk; ++i) {
      float v = acc[i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && m0 + i < m) {
        if (bias != nullptr) v += bias[row];
        const size_t o = (size_t)(m0 + i) * n + row;
        if (residual != nullptr) v += to_float<T>(residual[o]);
        if (activation == XQT_B200_ACT_RELU) v = fmaxf(v, 0.f);
        else if (activation == XQT_B200_ACT_GELU) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        else if (activation == XQT_B200_ACT_SILU) v = v / (1.f + expf(-v));
        out[o] = from_float<T>(v);
      }
    }
  }
}

int w4a16_simt_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                      const void* residual, void* out, int m, int n, int k, int padded_k, int group_size,
                      int nibble_signed, int act_dtype, int param_dtype, int activation, cudaStream_t stream) {
  const dim3 grid(ceil_div(n, kSimtRowsPerBlock)), block(kSimtRowsPerBlock * 32);
  if (act_dtype == XQT_B200_BF16) {
    w4a16_simt_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        (const __nv_bfloat16*)x, (const uint8_t*)qw, scales, zeros, bias, (const __nv_bfloat16*)residual,
        (__nv_bfloat16*)out, m, n, k, padded_k, group_size, nibble_signed, param_dtype, activation);
  } else {
    w4a16_simt_kernel<__half><<<grid, block, 0, stream>>>(
        (const __half*)x, (const uint8_t*)qw, scales, zeros, bias, (const __half*)residual, (__half*)out, m,
        n, k, padded_k, group_size, nibble_signed, param_dtype, activation);
  }
  return launch_status();
}

}  // namespace xqt_b200

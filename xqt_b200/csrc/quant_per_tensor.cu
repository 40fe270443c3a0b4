// Per-tensor dynamic int8 quantisation of an activation: the activation side of xqt's reference W8A8
// linear, Int8MmaLinear (xqt/contracts/int8_mma.py:135-149,308-319):
//     scale = max(absmax(x), eps) / 127        (one scale for the whole [M, K] tensor)
//     q     = clamp(rint(x / scale), -127, 127)
// Two kernels on one stream: a grid-wide absolute maximum (non-negative floats order like their bit
// patterns, so an integer atomicMax suffices), then the quantisation, which also writes the scale once
// per row so that the per-token epilogue of the int8 GEMM consumes it unchanged.  IEEE division and
// round-half-to-even throughout: the codes are bit-identical to the reference's.
#include "common.cuh"

namespace xqt_b200 {

template <typename T>
__global__ void __launch_bounds__(256) per_tensor_amax_kernel(const T* __restrict__ x, size_t vecs, unsigned int* __restrict__ stats) {
  float amax = 0.f;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + v);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(to_float<T>(e[i])));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  __shared__ float s_red[8];
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mx = 0.f;
    for (int w = 0; w < 8; ++w) mx = fmaxf(mx, s_red[w]);
    atomicMax(stats, __float_as_uint(mx));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) per_tensor_quant_kernel(const T* __restrict__ x, int8_t* __restrict__ codes,
                                                               float* __restrict__ row_scales, float* __restrict__ stats,
                                                               size_t vecs, int vecs_per_row, float eps) {
  const float scale = __fdiv_rn(fmaxf(stats[0], eps), 127.0f);
  if (blockIdx.x == 0 && threadIdx.x == 0) stats[1] = scale;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + v);
    const T* e = reinterpret_cast<const T*>(&raw);
    int8_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      q[i] = (int8_t)(int)fminf(fmaxf(rintf(__fdiv_rn(to_float<T>(e[i]), scale)), -127.f), 127.f);
    reinterpret_cast<uint2*>(codes)[v] = *reinterpret_cast<const uint2*>(q);
    if (v % vecs_per_row == 0) row_scales[v / vecs_per_row] = scale;
  }
}

// stats: two floats of scratch owned by the caller: [0] the absolute maximum, [1] the scale
int quant_per_tensor_launch(const void* x, void* codes, float* row_scales, float* stats, int m, int k, int act_dtype,
                            float eps, cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && k > 0 && k % 8 == 0 && eps > 0.f);
  XQT_REQUIRE(act_dtype == XQT_B200_BF16 || act_dtype == XQT_B200_FP16);
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 7) == 0);
  const size_t vecs = (size_t)m * k / 8;
  size_t blocks = (vecs + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  XQT_CUDA(cudaMemsetAsync(stats, 0, 2 * sizeof(float), stream));
  if (act_dtype == XQT_B200_BF16) {
    per_tensor_amax_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, vecs, (unsigned int*)stats);
    per_tensor_quant_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (int8_t*)codes, row_scales,
                                                                                 stats, vecs, k / 8, eps);
  } else {
    per_tensor_amax_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>((const __half*)x, vecs, (unsigned int*)stats);
    per_tensor_quant_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>((const __half*)x, (int8_t*)codes, row_scales, stats, vecs,
                                                                          k / 8, eps);
  }
  return launch_status();
}

}  // namespace xqt_b200

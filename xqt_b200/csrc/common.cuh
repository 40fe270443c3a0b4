// Shared helpers for the sm_100a kernels of the quantized-linear path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/xqt_b200.h"

namespace xqt_b200 {

// Every entry point returns a cudaError_t as int, cudaErrorInvalidValue for a
// request it cannot serve; nothing is thrown across the C boundary.
#define XQT_REQUIRE(cond)                        \
  do {                                           \
    if (!(cond)) return (int)cudaErrorInvalidValue; \
  } while (0)

#define XQT_CUDA(call)                           \
  do {                                           \
    cudaError_t err__ = (call);                  \
    if (err__ != cudaSuccess) return (int)err__; \
  } while (0)

inline int launch_status() { return (int)cudaGetLastError(); }

// Opt a kernel in to more than 48 KiB of dynamic shared memory.  The attribute belongs to the
// (function, device) pair, so it is set once per device the process launches on, with that device
// current.
#define XQT_SMEM_OPT_IN(kern, bytes)                                                                    \
  do {                                                                                                  \
    static bool configured__[64] = {};                                                                  \
    int dev__ = 0;                                                                                      \
    XQT_CUDA(cudaGetDevice(&dev__));                                                                    \
    if (dev__ < 0 || dev__ >= 64 || !configured__[dev__]) {                                             \
      XQT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes)));  \
      if (dev__ >= 0 && dev__ < 64) configured__[dev__] = true;                                         \
    }                                                                                                   \
  } while (0)

__host__ __device__ constexpr int ceil_div(int a, int b) { return (a + b - 1) / b; }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Read element i of a scale / zero-point array whose dtype is only known at run
// time (fp16, bf16 or fp32, XQT_B200_FP16/BF16/FP32).
__device__ __forceinline__ float load_param(const void* base, int dtype, size_t i) {
  if (dtype == XQT_B200_FP32) return reinterpret_cast<const float*>(base)[i];
  if (dtype == XQT_B200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}

// The same in two steps, so that a prefetch does not wait for its own data: the raw bits now, the value when needed.
__device__ __forceinline__ uint32_t load_param_bits(const void* base, int dtype, size_t i) {
  if (dtype == XQT_B200_FP32) return reinterpret_cast<const uint32_t*>(base)[i];
  return reinterpret_cast<const unsigned short*>(base)[i];
}
__device__ __forceinline__ float param_from_bits(uint32_t bits, int dtype) {
  if (dtype == XQT_B200_FP32) return __uint_as_float(bits);
  if (dtype == XQT_B200_BF16) return __uint_as_float(bits << 16);
  return __half2float(__ushort_as_half((unsigned short)bits));
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + __expf(-v)); }

}  // namespace xqt_b200

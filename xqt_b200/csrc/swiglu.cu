// SwiGLU gating of an MLP block: out[m, i] = silu(g[m, i]) * u[m, i] with the gate and up projections
// stored side by side in one [M, 2*inter] tensor (they are computed by ONE horizontally fused linear).
// fp32 arithmetic, one rounding; 8 elements per thread.  Reference: the vectorised silu(g)*u kernel of
// xqt's ConvRot W8A8 backend (xqt/kernels/jit/csrc/quantization/convrot_w8a8_sm89_kernel.cu:756-837).
#include "common.cuh"

namespace xqt_b200 {

template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int m, int inter) {
  const size_t chunks_per_row = inter / 8;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * chunks_per_row) return;
  const size_t row = i / chunks_per_row, c = i % chunks_per_row;
  const uint4 gv = reinterpret_cast<const uint4*>(gate_up + row * 2 * inter)[c];
  const uint4 uv = reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter)[c];
  const T* g = reinterpret_cast<const T*>(&gv);
  const T* u = reinterpret_cast<const T*>(&uv);
  uint4 ov;
  T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float x = to_float<T>(g[e]);
    o[e] = from_float<T>(x / (1.0f + expf(-x)) * to_float<T>(u[e]));
  }
  reinterpret_cast<uint4*>(out + row * inter)[c] = ov;
}

int swiglu_launch(const void* gate_up, void* out, int m, int inter, int dtype, cudaStream_t stream) {
  XQT_REQUIRE(((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0);
  const size_t total = (size_t)m * (inter / 8);
  const unsigned grid = (unsigned)((total + 255) / 256);
  if (dtype == XQT_B200_BF16)
    swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, m, inter);
  else
    swiglu_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)gate_up, (__half*)out, m, inter);
  return launch_status();
}

}  // namespace xqt_b200

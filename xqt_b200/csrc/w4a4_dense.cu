// W4A4 SVDQuant / ConvRot linear in its operand-dequantised form, for M >= 256.
//
// The per-(token, 64-K) activation scales and per-(channel, 64-K) weight scales make the integer
// GEMM pay one int32 drain and one fp32 scaling pass per 64-K group on the CUDA cores, which bounds
// gemm_w4a4_kernel at a few per cent of the tensor peak.  Here both operands are expanded once per
// call to fp16 -- x^[m,k] = code_a * s_a[m, k/64] and w^[n,k] = code_w * s_w[n, k/64], each an exact
// fp32 product rounded once -- and the low-rank branch is appended along K:
//     A' = [ x^ | la ]   (M x (K+32))       B' = [ w^ | up ]   (N x (K+32))
// so that one dense tcgen05 GEMM gives  x^ w^T + la up^T (+ bias), the arithmetic of the composite
// artifact's forward (xqt/compression/quant/contracts/composite.py:92-227) on the fake-quantised
// activation of the W4A4 contract.  The integer codes and scales are those of the prologue kernel,
// bit for bit; only the accumulation differs from the integer form (fp16 operands, fp32 sums).
#include "common.cuh"

namespace xqt_b200 {

int gemm_f16_launch_strided(const void* a, long long lda, const void* b, long long ldb, const float* bias,
                            const void* residual, void* out, int m, int n, int k, int out_dtype, int out_f32,
                            int operand_bf16, unsigned int* status, cudaStream_t stream);

namespace w4a4d {
constexpr int kGroup = 64, kRank = 32;
}

// one thread: 16 codes of one row (a quarter group) -> 16 fp16; the threads of the last column
// block also write the rank-32 low-rank activations
__global__ void __launch_bounds__(256) w4a4_expand_act_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales,
                                                             const float* __restrict__ la, __half* __restrict__ dst, int m,
                                                             int k) {
  using namespace w4a4d;
  const int chunks = k / 16 + 2;                               // 16-element chunks per row incl. the 32 low-rank columns
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * chunks) return;
  const int row = (int)(i / chunks), c = (int)(i % chunks);
  __half* out = dst + (size_t)row * (k + kRank) + (size_t)c * 16;
  float v[16];
  if (c * 16 < k) {
    const float s = scales[(size_t)row * (k / kGroup) + (c * 16) / kGroup];
    const int4 raw = *reinterpret_cast<const int4*>(codes + (size_t)row * k + (size_t)c * 16);
    const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = (float)q[j] * s;
  } else {
    const int r0 = c * 16 - k;                                 // 0 or 16
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = la != nullptr ? la[(size_t)row * kRank + r0 + j] : 0.f;
  }
  uint4 o[2];
  __half2* h = reinterpret_cast<__half2*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
  reinterpret_cast<uint4*>(out)[0] = o[0];
  reinterpret_cast<uint4*>(out)[1] = o[1];
}

// one thread: 32 signed nibbles (16 packed bytes) of one weight row -> 32 fp16, or 16 of the 32 up factors
__global__ void __launch_bounds__(256) w4a4_expand_weight_kernel(const uint8_t* __restrict__ qweight, const float* __restrict__ scales,
                                                                const float* __restrict__ up, __half* __restrict__ dst, int n,
                                                                int k) {
  using namespace w4a4d;
  const int chunks = k / 32 + 1;                               // 32-element chunks per row incl. the up factors
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n * chunks) return;
  const int row = (int)(i / chunks), c = (int)(i % chunks);
  uint4* out = reinterpret_cast<uint4*>(dst + (size_t)row * (k + kRank) + (size_t)c * 32);
  if (c * 32 < k) {
    const float s = scales[(size_t)row * (k / kGroup) + (c * 32) / kGroup];
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)row * (k / 2)) + c);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t word = words[w] ^ 0x88888888u;            // two's-complement nibble -> code + 8
      uint4 o;
      __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = ((float)((word >> (8 * j)) & 15u) - 8.f) * s;        // even k: low nibble
        const float b = ((float)((word >> (8 * j + 4)) & 15u) - 8.f) * s;
        h[j] = __floats2half2_rn(a, b);
      }
      out[w] = o;
    }
  } else {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint4 o;
      __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = w * 8 + j * 2;
        h[j] = up != nullptr ? __floats2half2_rn(up[(size_t)row * kRank + r], up[(size_t)row * kRank + r + 1]) : __floats2half2_rn(0.f, 0.f);
      }
      out[w] = o;
    }
  }
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t w4a4_dense_workspace_bytes(int m, int n, int k) {
  using namespace w4a4d;
  return 256 + align256((size_t)m * (k + kRank) * 2) + align256((size_t)n * (k + kRank) * 2);
}

bool w4a4_dense_supported(int m, int n, int k) { return m >= 1 && n >= 8 && n % 8 == 0 && k >= 64 && k % 64 == 0; }

// codes int8 [M,K] (values in [-8,7]), a_scale fp32 [M,K/64], qweight signed nibbles [N,K/2], w_scale
// fp32 [N,K/64], la fp32 [M,32] or null, up fp32 [N,32] or null, bias fp32 [N] or null
int w4a4_dense_launch(const void* codes, const float* a_scale, const void* qweight, const float* w_scale, const float* la,
                      const float* up, const float* bias, void* out, int m, int n, int k, int out_dtype, void* workspace,
                      size_t workspace_bytes, cudaStream_t stream) {
  using namespace w4a4d;
  XQT_REQUIRE(w4a4_dense_supported(m, n, k));
  XQT_REQUIRE(codes != nullptr && a_scale != nullptr && qweight != nullptr && w_scale != nullptr && out != nullptr);
  XQT_REQUIRE((la == nullptr) == (up == nullptr));
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= w4a4_dense_workspace_bytes(m, n, k));
  XQT_REQUIRE(((uintptr_t)codes & 15) == 0 && ((uintptr_t)qweight & 15) == 0 && ((uintptr_t)workspace & 255) == 0);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  unsigned int* status = reinterpret_cast<unsigned int*>(ws);
  __half* a16 = reinterpret_cast<__half*>(ws + 256);
  __half* b16 = reinterpret_cast<__half*>(ws + 256 + align256((size_t)m * (k + kRank) * 2));
  {
    const size_t threads = (size_t)m * (k / 16 + 2);
    w4a4_expand_act_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const int8_t*)codes, a_scale, la, a16, m, k);
    XQT_CUDA(cudaGetLastError());
  }
  {
    const size_t threads = (size_t)n * (k / 32 + 1);
    w4a4_expand_weight_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const uint8_t*)qweight, w_scale, up, b16, n, k);
    XQT_CUDA(cudaGetLastError());
  }
  const int kk = k + kRank;
  return gemm_f16_launch_strided(a16, kk, b16, kk, bias, nullptr, out, m, n, kk, out_dtype, 0, 0, status, stream);
}

// la[M,32] fp32 = x[M,K] (bf16 or fp16) * down[32,K]^T on the dense tcgen05 GEMM
int lowrank_down_tc_launch(const void* x, const void* down, float* la, int m, int k, int dtype, unsigned int* status,
                           cudaStream_t stream) {
  XQT_REQUIRE(m >= 1 && k >= 64 && k % 8 == 0 && x != nullptr && down != nullptr && la != nullptr && status != nullptr);
  return gemm_f16_launch_strided(x, k, down, k, nullptr, nullptr, la, m, w4a4d::kRank, k, dtype, 1, dtype == XQT_B200_BF16 ? 1 : 0,
                                 status, stream);
}

}  // namespace xqt_b200

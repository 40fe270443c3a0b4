// W4A16 GEMM for M > 16 on tcgen05, host side and the two-pass form: Y[M,N] = X[M,K] * dequant(W)[N,K]^T.
//
// Two forms share this entry.  The fused kernel (gemm_w4a16_fused.cu) dequantises the packed weights in
// registers on their way to the tensor core and is the choice while M is a few hundred tokens.  At large M the
// weights are dequantised once per call into an fp16 scratch (any real zero point, fp32 arithmetic, one
// rounding) and multiplied by the dense tcgen05 GEMM: the N*K*2-byte round trip is then small against the
// 2*M*N*K flops, and the dense kernel's 256-wide tiles run nearer the tensor peak.
//
// Precision.  Both MMA operands are fp16: (code - zero) * scale rounded once to fp16 (11-bit significand) is a
// relative error of at most 2^-12 per weight, ~1e-4 rel-L2 on the output against the 1e-3 bar; bf16 weights
// (8-bit significand) would cost ~8e-4.  bf16 activations are converted to fp16 once per call into the caller's
// scratch: exact for 2^-14 <= |x| <= 65504 (smaller values lose bits to fp16's subnormals), NaN kept, anything
// larger clamped to +-65504 with bit 256 set in the status word.
// Envelope: group size 64 or 128, K a multiple of 64; anything else is served by the generic CUDA-core
// kernel.  Reference arithmetic: xqt/kernels/ops/gemm/reference.py:263-271,527.
#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"
#include <type_traits>

namespace xqt_b200 {

size_t w4a16_gemm_fused_workspace_bytes(int m, int n, int k);

using namespace sm100;

int make_tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int esize, long long rows,
                  long long cols, int box_rows);

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
// fp32 and rounded once.  A warp converts a span of 128 packed words (1024 weights) of one row: lane l takes the
// words l, l + 32, l + 64, l + 96, so every load instruction reads 128 contiguous bytes and every store instruction
// writes 512 contiguous bytes (one thread per 16 packed bytes, each storing four separate 16-byte pieces of its own
// 64-byte run, measured 3.5 TB/s on the stores of this pass).
constexpr int kDqSpanWords = 128;
template <typename P>
__global__ void __launch_bounds__(256) dequant_w4_f16_kernel(const uint8_t* __restrict__ qweight, const P* __restrict__ scales,
                                                            const P* __restrict__ zeros, __half* __restrict__ dst, int n,
                                                            int k, int group_size, int nibble_signed) {
  const int words_per_row = k / 8, spans = (words_per_row + kDqSpanWords - 1) / kDqSpanWords;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (size_t)n * spans) return;
  const int row = (int)(warp / spans), span = (int)(warp % spans);
  const uint32_t* src = reinterpret_cast<const uint32_t*>(qweight + (size_t)row * (k / 2));
  const size_t prow = (size_t)row * (k / group_size);
  uint4* out = reinterpret_cast<uint4*>(dst + (size_t)row * k);
  const float zoff = nibble_signed ? 8.f : 0.f;
  uint32_t words[4];
  int wi[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    wi[j] = span * kDqSpanWords + j * 32 + lane;
    words[j] = wi[j] < words_per_row ? __ldg(src + wi[j]) : 0u;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (wi[j] >= words_per_row) continue;
    const size_t pi = prow + (wi[j] * 8) / group_size;
    const float sc = to_float<P>(scales[pi]);
    const float zp = (zeros != nullptr ? to_float<P>(zeros[pi]) : 0.f) + zoff;
    const uint32_t word = nibble_signed ? (words[j] ^ 0x88888888u) : words[j];   // two's complement -> code + 8
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = ((float)((word >> (8 * e)) & 15u) - zp) * sc;
      const float b = ((float)((word >> (8 * e + 4)) & 15u) - zp) * sc;
      h[e] = __floats2half2_rn(a, b);
    }
    out[wi[j]] = o;
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
  const size_t fused = w4a16_gemm_fused_workspace_bytes(m, n, k);
  return bytes > fused ? bytes : fused;
}
bool w4a16_gemm_tc_any_zero_point(int m) { return m >= dense_min_m(); }

int gemm_f16_launch(const void* a, const void* b, const float* bias, const void* residual, void* out, int m, int n,
                    int k, int out_dtype, int out_f32, unsigned int* status, cudaStream_t stream);

bool w4a16_gemm_tc_supported(int m, int n, int k, int padded_k, int group_size) {
  return m >= 1 && n % 8 == 0 && k == padded_k && k % 64 == 0 && (group_size == 64 || group_size == 128);
}

int w4a16_gemm_fused_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                            const void* residual, void* out, int m, int n, int k, int group_size, int nibble_signed,
                            int act_dtype, int param_dtype, int out_f32, void* workspace, size_t workspace_bytes,
                            cudaStream_t stream);
int bf16_to_f16_launch(const void* src, void* dst, size_t elements, unsigned int* status, cudaStream_t stream) {
  const size_t n8 = elements / 8;
  bf16_to_f16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)src, (__half*)dst, n8, status);
  return launch_status();
}

int w4a16_gemm_tc_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                         const void* residual, void* out, int m, int n, int k, int group_size, int nibble_signed,
                         int act_dtype, int param_dtype, int out_f32, int single_pass, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream) {
  XQT_REQUIRE(w4a16_gemm_tc_supported(m, n, k, k, group_size));
  if (single_pass)
    return w4a16_gemm_fused_launch(x, qw, scales, zeros, bias, residual, out, m, n, k, group_size, nibble_signed, act_dtype,
                                   param_dtype, out_f32, workspace, workspace_bytes, stream);
  const bool two_pass = m >= dense_min_m();
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
    const size_t threads = (size_t)n * ((k / 8 + kDqSpanWords - 1) / kDqSpanWords) * 32;     // one warp per 128-word span of a row
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
  return (int)cudaErrorInvalidValue;   // unreachable: the single-pass form returned above
}

}  // namespace xqt_b200

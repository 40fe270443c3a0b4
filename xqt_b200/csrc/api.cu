// C-ABI entry points: argument validation and kernel selection.  No kernel code lives here.
#include "common.cuh"

namespace xqt_b200 {
int w4a16_simt_launch(const void*, const void*, const void*, const void*, const float*, const void*, void*, int, int,
                      int, int, int, int, int, int, int, cudaStream_t);
int w4a16_gemv_launch(const void*, const void*, const void*, const void*, const float*, const void*, void*, int, int,
                      int, int, int, int, void*, size_t, cudaStream_t);
size_t w4a16_gemv_workspace_bytes(int n, int k);
bool w4a16_gemv_supported(int m, int n, int k, int padded_k, int group_size);
int w4a16_decode_launch(const void*, const void*, const void*, const float*, const void*, void*, int, int, int, int, int,
                        int, int, int, void*, size_t, cudaStream_t);
size_t w4a16_decode_workspace_bytes();
bool w4a16_decode_supported(int m, int n, int k, int group_size);
int w4a16_decode_launch_static(const void*, const void*, const void*, const float*, const void*, void*, int, int, int,
                               int, int, int, int, int, cudaStream_t);
size_t w4a16_decode_static_scratch_bytes();
int w4a16_decode_static_max_n();
int w4a16_decode_tc_launch(const void*, const void*, const void*, const float*, const void*, void*, int, int, int, int,
                           int, int, int, int, void*, size_t, cudaStream_t);
size_t w4a16_decode_tc_workspace_bytes();
bool w4a16_decode_tc_supported(int m, int n, int k, int group_size);
int w4a16_decode_cl_launch(const void*, const void*, const void*, const void*, const float*, const void*, void*, int, int, int,
                           int, int, int, int, int, int, const unsigned int*, long long, unsigned int*, cudaStream_t);
bool w4a16_decode_cl_supported(int m, int n, int k, int group_size);
void w4a16_decode_cl_set_plan(int kw, int s);
void w4a16_decode_cl_get_plan(int m, int n, int k, int* kw, int* s);
int w4a16_gemm_tc_launch(const void*, const void*, const void*, const void*, const float*, const void*, void*, int, int,
                         int, int, int, int, int, int, int, void*, size_t, cudaStream_t);
int swiglu_launch(const void*, void*, int, int, int, cudaStream_t);
size_t w4a16_gemm_tc_workspace_bytes(int m, int n, int k);
bool w4a16_gemm_tc_any_zero_point(int m);
bool w4a16_gemm_tc_supported(int m, int n, int k, int padded_k, int group_size);
bool w4a16_gemm_fused_preferred(int m, int n, int k, int padded_k, int group_size);
int lowrank_down_launch(const void*, const void*, float*, void*, int, int, int, cudaStream_t);
size_t w4a4_workspace_bytes(int m, int n, int k);
int w4a4_gemm_launch(const void*, const float*, const void*, const void*, const void*, const float*, const float*, void*, int,
                     int, int, int, int, void*, cudaStream_t);
int w4a4_expand_weight_launch(const void*, void*, int, int, cudaStream_t);
size_t w4a4_aux_tile_bytes(int k);
bool w4a4_gemm_supported(int m, int n, int k);
int rotate_quant_launch(const void*, const float*, void*, float*, void*, int, int, int, int, int, int, int, cudaStream_t);
int gemm_i8_launch(const void*, const void*, const float*, const float*, const float*, void*, int, int, int, int,
                   unsigned int*, cudaStream_t);
int gemm_i8_addend_launch(const void*, const void*, const float*, const float*, const float*, const float*, void*, int, int, int,
                          int, unsigned int*, cudaStream_t);
int gemm_f16_launch_strided(const void*, long long, const void*, long long, const float*, const void*, void*, int, int, int, int,
                            int, int, unsigned int*, cudaStream_t);
size_t w4a4_dense_workspace_bytes(int m, int n, int k);
bool w4a4_dense_supported(int m, int n, int k);
int w4a4_dense_launch(const void*, const float*, const void*, const float*, const float*, const float*, const float*, void*,
                      int, int, int, int, void*, size_t, cudaStream_t);
int lowrank_down_tc_launch(const void*, const void*, float*, int, int, int, unsigned int*, cudaStream_t);
int peer_allreduce_launch(const void* const*, void* const*, int, int, unsigned int, long long, int, const float*, void*, int,
                          unsigned int, unsigned int*, unsigned int*, long long, cudaStream_t);
int peer_allgather_launch(const void* const*, void* const*, int, int, unsigned int*, long long, long long, void*, unsigned int,
                          unsigned int*, cudaStream_t);
int w4a16_decode_static_status(unsigned int*, cudaStream_t);
int quant_per_tensor_launch(const void*, void*, float*, float*, int, int, int, float, cudaStream_t);
}  // namespace xqt_b200

using namespace xqt_b200;

extern "C" {

const char* xqt_b200_version(void) { return "xqt-b200 0.1 (sm_100a)"; }

const char* xqt_b200_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

int xqt_b200_device_supported(int device) {
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) return 0;
  return (major == 10 && minor == 0) ? 1 : 0;
}

size_t xqt_b200_w4a16_workspace_bytes(int m, int n, int k) {
  if (n <= 0 || k <= 0) return 0;
  const size_t a = w4a16_gemv_workspace_bytes(n, k);
  const size_t b = m > 16 ? w4a16_gemm_tc_workspace_bytes(m, n, k) : 0;   // fp16 activations (+ fp16 weights at large M)
  return a > b ? a : b;
}

int xqt_b200_w4a16_select_variant(int m, int n, int k, int padded_k, int group_size, int epilogue_activation,
                                  int has_residual) {
  (void)has_residual;
  if (epilogue_activation == XQT_B200_ACT_NONE && w4a16_gemv_supported(m, n, k, padded_k, group_size))
    return XQT_B200_VARIANT_GEMV;
  if (epilogue_activation == XQT_B200_ACT_NONE && m > 16 && w4a16_gemm_tc_supported(m, n, k, padded_k, group_size))
    return XQT_B200_VARIANT_TCGEN05;
  return XQT_B200_VARIANT_SIMT;
}

int xqt_b200_w4a16_two_pass(int m) { return w4a16_gemm_tc_any_zero_point(m) ? 1 : 0; }

int xqt_b200_w4a16_fused_preferred(int m, int n, int k, int padded_k, int group_size) {
  return w4a16_gemm_fused_preferred(m, n, k, padded_k, group_size) ? 1 : 0;
}

int xqt_b200_w4a16_run(const void* activation, const void* qweight, const void* scales, const void* zero_points,
                       const float* bias, const void* residual, void* output, int m, int n, int k, int padded_k,
                       int group_size, int nibble_signed, int act_dtype, int param_dtype, int out_dtype,
                       int epilogue_activation, void* workspace, size_t workspace_bytes, int variant,
                       xqt_b200_stream_t stream) {
  XQT_REQUIRE(m >= 0 && n > 0 && k > 0 && padded_k >= k);
  XQT_REQUIRE(group_size == 32 || group_size == 64 || group_size == 128);
  XQT_REQUIRE(padded_k % group_size == 0);
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(param_dtype == XQT_B200_FP16 || param_dtype == XQT_B200_BF16 || param_dtype == XQT_B200_FP32);
  XQT_REQUIRE(epilogue_activation >= XQT_B200_ACT_NONE && epilogue_activation <= XQT_B200_ACT_SILU);
  XQT_REQUIRE(out_dtype == act_dtype || out_dtype == XQT_B200_FP32);
  const int out_f32 = out_dtype == XQT_B200_FP32 && act_dtype != XQT_B200_FP32 ? 1 : 0;
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && qweight != nullptr && scales != nullptr && output != nullptr);
  if (out_f32) {
    // fp32 partial sums (K-sharded layers) are produced by the tensor-core GEMM only
    XQT_REQUIRE(variant == XQT_B200_VARIANT_AUTO || variant == XQT_B200_VARIANT_TCGEN05 ||
                variant == XQT_B200_VARIANT_TCGEN05_FUSED);
    if (variant == XQT_B200_VARIANT_AUTO) variant = XQT_B200_VARIANT_TCGEN05;
  }
  if (variant == XQT_B200_VARIANT_AUTO) {
    variant = xqt_b200_w4a16_select_variant(m, n, k, padded_k, group_size, epilogue_activation, residual != nullptr);
    // the tensor-core GEMM folds the zero point into an exact integer subtraction: only a caller who
    // knows its zero points are integers may ask for it; AUTO takes it for symmetric weights only
    // (at large M the weights are dequantised in fp32 first, which serves any zero point)
    if (variant == XQT_B200_VARIANT_TCGEN05 && zero_points != nullptr && !w4a16_gemm_tc_any_zero_point(m))
      variant = XQT_B200_VARIANT_SIMT;
    // the fused form where it measures faster; with zero points only a caller who knows they are integers asks for it
    if (variant == XQT_B200_VARIANT_TCGEN05 && zero_points == nullptr && !out_f32 &&
        w4a16_gemm_fused_preferred(m, n, k, padded_k, group_size))
      variant = XQT_B200_VARIANT_TCGEN05_FUSED;
  }
  cudaStream_t s = (cudaStream_t)stream;
  switch (variant) {
    case XQT_B200_VARIANT_SIMT:
      return w4a16_simt_launch(activation, qweight, scales, zero_points, bias, residual, output, m, n, k, padded_k,
                               group_size, nibble_signed, act_dtype, param_dtype, epilogue_activation, s);
    case XQT_B200_VARIANT_GEMV:
      XQT_REQUIRE(epilogue_activation == XQT_B200_ACT_NONE);
      XQT_REQUIRE(w4a16_gemv_supported(m, n, k, padded_k, group_size));
      XQT_REQUIRE(((uintptr_t)activation & 15) == 0 && ((uintptr_t)qweight & 15) == 0);
      return w4a16_gemv_launch(activation, qweight, scales, zero_points, bias, residual, output, m, n, k,
                               nibble_signed, act_dtype, param_dtype, workspace, workspace_bytes, s);
    case XQT_B200_VARIANT_TCGEN05:
    case XQT_B200_VARIANT_TCGEN05_FUSED:
      XQT_REQUIRE(epilogue_activation == XQT_B200_ACT_NONE);
      XQT_REQUIRE(w4a16_gemm_tc_supported(m, n, k, padded_k, group_size));
      XQT_REQUIRE(workspace != nullptr && workspace_bytes >= 256);
      XQT_REQUIRE(((uintptr_t)activation & 15) == 0 && ((uintptr_t)qweight & 15) == 0);
      return w4a16_gemm_tc_launch(activation, qweight, scales, zero_points, bias, residual, output, m, n, k,
                                  group_size, nibble_signed, act_dtype, param_dtype, out_f32,
                                  variant == XQT_B200_VARIANT_TCGEN05_FUSED ? 1 : 0, workspace, workspace_bytes, s);
    default:
      return (int)cudaErrorInvalidValue;
  }
}

size_t xqt_b200_w4a16_decode_workspace_bytes(void) { return w4a16_decode_workspace_bytes(); }

int xqt_b200_w4a16_decode_supported(int m, int n, int k, int group_size) {
  return w4a16_decode_supported(m, n, k, group_size) ? 1 : 0;
}

int xqt_b200_w4a16_decode_tiled(const void* activation, const void* tiled_weights, const void* tiled_params,
                                const float* bias, const void* residual, void* output, int m, int n, int k,
                                int group_size, int nibble_signed, int has_zero_point, int act_dtype, int param_dtype,
                                void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  XQT_REQUIRE(m >= 0 && n > 0 && k > 0);
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(param_dtype == XQT_B200_FP16 || param_dtype == XQT_B200_BF16 || param_dtype == XQT_B200_FP32);
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && tiled_weights != nullptr && tiled_params != nullptr && output != nullptr);
  return w4a16_decode_launch(activation, tiled_weights, tiled_params, bias, residual, output, m, n, k, group_size,
                             nibble_signed, has_zero_point, act_dtype, param_dtype, workspace, workspace_bytes,
                             (cudaStream_t)stream);
}

size_t xqt_b200_w4a16_decode_tc_workspace_bytes(void) { return w4a16_decode_tc_workspace_bytes(); }

int xqt_b200_w4a16_decode_tc_supported(int m, int n, int k, int group_size) {
  return w4a16_decode_tc_supported(m, n, k, group_size) ? 1 : 0;
}

int xqt_b200_w4a16_decode_tc(const void* activation, const void* row_weights, const void* tiled_params,
                             const float* bias, const void* residual, void* output, int m, int n, int k,
                             int group_size, int nibble_signed, int act_dtype, int param_dtype, int out_dtype,
                             void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  XQT_REQUIRE(m >= 0 && n > 0 && k > 0);
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(param_dtype == XQT_B200_FP16 || param_dtype == XQT_B200_BF16 || param_dtype == XQT_B200_FP32);
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && row_weights != nullptr && tiled_params != nullptr && output != nullptr);
  XQT_REQUIRE(out_dtype == act_dtype || out_dtype == XQT_B200_FP32);
  return w4a16_decode_tc_launch(activation, row_weights, tiled_params, bias, residual, output, m, n, k, group_size,
                                nibble_signed, act_dtype, param_dtype, out_dtype == XQT_B200_FP32 ? 1 : 0, workspace,
                                workspace_bytes, (cudaStream_t)stream);
}

int xqt_b200_w4a16_decode_lanes_supported(int m, int n, int k, int group_size) {
  return w4a16_decode_cl_supported(m, n, k, group_size) ? 1 : 0;
}

int xqt_b200_w4a16_decode_lanes_plan(int m, int n, int k, int group_size, int* warp_quads, int* cluster) {
  XQT_REQUIRE(warp_quads != nullptr && cluster != nullptr);
  XQT_REQUIRE(w4a16_decode_cl_supported(m, n, k, group_size));
  w4a16_decode_cl_get_plan(m, n, k, warp_quads, cluster);
  return 0;
}

int xqt_b200_w4a16_decode_lanes_set_plan(int warp_quads, int cluster) {
  XQT_REQUIRE((warp_quads == 0 && cluster == 0) ||
              ((warp_quads == 1 || warp_quads == 2) && cluster >= 1 && cluster <= 8));
  w4a16_decode_cl_set_plan(warp_quads, cluster);
  return 0;
}

int xqt_b200_w4a16_decode_lanes_select(const void* activation, const void* lane_weights, const void* lane_scales,
                                       const void* lane_zeros, const float* bias, const void* residual, void* output, int m,
                                       int n, int k, int group_size, int nibble_signed, int act_dtype, int param_dtype,
                                       int out_dtype, int epilogue_flags, const unsigned int* out_select,
                                       size_t out_select_stride, unsigned int* status, xqt_b200_stream_t stream);

int xqt_b200_w4a16_decode_lanes(const void* activation, const void* lane_weights, const void* lane_scales,
                                const void* lane_zeros, const float* bias, const void* residual, void* output, int m, int n, int k,
                                int group_size, int nibble_signed, int act_dtype, int param_dtype, int out_dtype,
                                int epilogue_flags, unsigned int* status, xqt_b200_stream_t stream) {
  return xqt_b200_w4a16_decode_lanes_select(activation, lane_weights, lane_scales, lane_zeros, bias, residual, output, m, n, k,
                                            group_size, nibble_signed, act_dtype, param_dtype, out_dtype, epilogue_flags,
                                            nullptr, 0, status, stream);
}

int xqt_b200_w4a16_decode_lanes_select(const void* activation, const void* lane_weights, const void* lane_scales,
                                       const void* lane_zeros, const float* bias, const void* residual, void* output, int m,
                                       int n, int k, int group_size, int nibble_signed, int act_dtype, int param_dtype,
                                       int out_dtype, int epilogue_flags, const unsigned int* out_select,
                                       size_t out_select_stride, unsigned int* status, xqt_b200_stream_t stream) {
  XQT_REQUIRE(m >= 0 && n > 0 && k > 0 && (epilogue_flags & ~3) == 0);
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(param_dtype == XQT_B200_FP16 || param_dtype == XQT_B200_BF16 || param_dtype == XQT_B200_FP32);
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && lane_weights != nullptr && lane_scales != nullptr && output != nullptr);
  XQT_REQUIRE(out_dtype == act_dtype || out_dtype == XQT_B200_FP32);
  return w4a16_decode_cl_launch(activation, lane_weights, lane_scales, lane_zeros, bias, residual, output, m, n, k, group_size,
                                nibble_signed, act_dtype, param_dtype, out_dtype == XQT_B200_FP32 ? 1 : 0, epilogue_flags,
                                out_select, (long long)out_select_stride, status, (cudaStream_t)stream);
}

int xqt_b200_w4a16_decode_tiled_static(const void* activation, const void* tiled_weights, const void* tiled_params,
                                       const float* bias, const void* residual, void* output, int m, int n, int k,
                                       int group_size, int nibble_signed, int has_zero_point, int act_dtype,
                                       int param_dtype, xqt_b200_stream_t stream) {
  XQT_REQUIRE(m >= 0 && n > 0 && k > 0);
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(param_dtype == XQT_B200_FP16 || param_dtype == XQT_B200_BF16 || param_dtype == XQT_B200_FP32);
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && tiled_weights != nullptr && tiled_params != nullptr && output != nullptr);
  return w4a16_decode_launch_static(activation, tiled_weights, tiled_params, bias, residual, output, m, n, k,
                                    group_size, nibble_signed, has_zero_point, act_dtype, param_dtype,
                                    (cudaStream_t)stream);
}

size_t xqt_b200_w4a16_decode_static_scratch_bytes(void) { return w4a16_decode_static_scratch_bytes(); }

int xqt_b200_w4a16_decode_static_status(unsigned int* host_status, xqt_b200_stream_t stream) {
  XQT_REQUIRE(host_status != nullptr);
  return w4a16_decode_static_status(host_status, (cudaStream_t)stream);
}

int xqt_b200_w4a16_decode_static_max_n(void) { return w4a16_decode_static_max_n(); }

int xqt_b200_rotate_quantize(const void* activation, const float* column_scale, void* codes, float* scales,
                             void* rotated, int m, int k, int rot_kind, int rot_block, int quant_bits, int group_size,
                             int act_dtype, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && codes != nullptr && scales != nullptr);
  return rotate_quant_launch(activation, column_scale, codes, scales, rotated, m, k, rot_kind, rot_block, quant_bits,
                             group_size, act_dtype, (cudaStream_t)stream);
}

int xqt_b200_quantize_per_tensor(const void* activation, void* codes, float* row_scales, float* stats, int m, int k,
                                 int act_dtype, float eps, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(activation != nullptr && codes != nullptr && row_scales != nullptr && stats != nullptr);
  return quant_per_tensor_launch(activation, codes, row_scales, stats, m, k, act_dtype, eps, (cudaStream_t)stream);
}

int xqt_b200_w8a8_gemm(const void* act_codes, const void* weight_codes, const float* act_scale,
                       const float* weight_scale, const float* bias, void* output, int m, int n, int k, int out_dtype,
                       void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= 256);
  return gemm_i8_launch(act_codes, weight_codes, act_scale, weight_scale, bias, output, m, n, k, out_dtype,
                        reinterpret_cast<unsigned int*>(workspace), (cudaStream_t)stream);
}

int xqt_b200_w8a8_gemm_addend(const void* act_codes, const void* weight_codes, const float* act_scale,
                              const float* weight_scale, const float* bias, const float* addend, void* output, int m, int n,
                              int k, int out_dtype, void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= 256);
  return gemm_i8_addend_launch(act_codes, weight_codes, act_scale, weight_scale, bias, addend, output, m, n, k, out_dtype,
                               reinterpret_cast<unsigned int*>(workspace), (cudaStream_t)stream);
}

int xqt_b200_lowrank_up(const void* la, const void* up, float* output, int m, int n, int rank_padded, int act_dtype,
                        void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(la != nullptr && up != nullptr && output != nullptr && workspace != nullptr && workspace_bytes >= 256);
  XQT_REQUIRE(rank_padded >= 64 && rank_padded % 64 == 0 && (act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16));
  return gemm_f16_launch_strided(la, rank_padded, up, rank_padded, nullptr, nullptr, output, m, n, rank_padded, act_dtype, 1,
                                 act_dtype == XQT_B200_BF16 ? 1 : 0, reinterpret_cast<unsigned int*>(workspace),
                                 (cudaStream_t)stream);
}

int xqt_b200_lowrank_down(const void* rotated, const void* down, float* la, void* la_image, int m, int k, int act_dtype,
                          xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(rotated != nullptr && down != nullptr && (la != nullptr || la_image != nullptr));
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  return lowrank_down_launch(rotated, down, la, la_image, m, k, act_dtype, (cudaStream_t)stream);
}

size_t xqt_b200_w4a4_aux_tile_bytes(int k) { return k > 0 && k % 64 == 0 ? w4a4_aux_tile_bytes(k) : 0; }

int xqt_b200_w4a4_supported(int m, int n, int k) { return w4a4_gemm_supported(m, n, k) ? 1 : 0; }

int xqt_b200_w4a4_gemm(const void* act_codes, const float* act_scales, const void* qweight, const void* weight_bytes,
                       const void* aux, const float* la, const float* bias, void* output, int m, int n, int k,
                       int out_dtype, int flags, void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(m > 0 && workspace != nullptr && workspace_bytes >= w4a4_workspace_bytes(m, n, k) && ((uintptr_t)workspace & 255) == 0);
  XQT_REQUIRE((flags & ~3) == 0);
  return w4a4_gemm_launch(act_codes, act_scales, qweight, weight_bytes, aux, la, bias, output, m, n, k, out_dtype, flags,
                          workspace, (cudaStream_t)stream);
}

int xqt_b200_w4a4_expand_weight(const void* qweight, void* weight_bytes, int n, int k, xqt_b200_stream_t stream) {
  return w4a4_expand_weight_launch(qweight, weight_bytes, n, k, (cudaStream_t)stream);
}

size_t xqt_b200_w4a4_workspace_bytes(int m, int n, int k) {
  return m > 0 && n > 0 && k > 0 ? w4a4_workspace_bytes(m, n, k) : 256;
}

size_t xqt_b200_w4a4_dense_workspace_bytes(int m, int n, int k) {
  return w4a4_dense_supported(m, n, k) ? w4a4_dense_workspace_bytes(m, n, k) : 0;
}

// The dense form is the faster one from M = 256 on, but its fp16 operand rounding leaves about 1.2e-3
// of rel-L2 (after the bf16 output rounding) at K = 3072 where the integer form leaves 1e-4: it is
// reported as available, not chosen by default.
int xqt_b200_w4a4_dense_preferred(int m, int n, int k) { return (m >= 256 && w4a4_dense_supported(m, n, k)) ? 1 : 0; }

int xqt_b200_w4a4_dense(const void* act_codes, const float* act_scales, const void* qweight, const float* weight_scales,
                        const float* la, const float* up, const float* bias, void* output, int m, int n, int k,
                        int out_dtype, void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(out_dtype == XQT_B200_FP16 || out_dtype == XQT_B200_BF16);
  return w4a4_dense_launch(act_codes, act_scales, qweight, weight_scales, la, up, bias, output, m, n, k, out_dtype,
                           workspace, workspace_bytes, (cudaStream_t)stream);
}

int xqt_b200_lowrank_down_tc(const void* rotated, const void* down, float* la, int m, int k, int act_dtype,
                             void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(act_dtype == XQT_B200_FP16 || act_dtype == XQT_B200_BF16);
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= 256);
  return lowrank_down_tc_launch(rotated, down, la, m, k, act_dtype, reinterpret_cast<unsigned int*>(workspace),
                                (cudaStream_t)stream);
}

int xqt_b200_peer_allreduce(const void* const* partials, void* const* flags, int rank, int world, unsigned int call,
                            long long count, int n, const float* bias, void* output, int out_dtype,
                            unsigned int spin_limit, unsigned int* status, xqt_b200_stream_t stream) {
  XQT_REQUIRE(status != nullptr);
  return peer_allreduce_launch(partials, flags, rank, world, call, count, n, bias, output, out_dtype, spin_limit, status,
                               nullptr, 0, (cudaStream_t)stream);
}

int xqt_b200_peer_allreduce_counted(const void* const* partials, void* const* flags, int rank, int world,
                                    unsigned int* counter, long long slot_stride, long long count, int n,
                                    const float* bias, void* output, int out_dtype, unsigned int spin_limit,
                                    unsigned int* status, xqt_b200_stream_t stream) {
  XQT_REQUIRE(status != nullptr && counter != nullptr);
  return peer_allreduce_launch(partials, flags, rank, world, 0u, count, n, bias, output, out_dtype, spin_limit, status,
                               counter, slot_stride, (cudaStream_t)stream);
}

int xqt_b200_peer_allgather_counted(const void* const* sources, void* const* flags, int rank, int world,
                                    unsigned int* counter, long long slot_stride_bytes, long long bytes, void* output,
                                    unsigned int spin_limit, unsigned int* status, xqt_b200_stream_t stream) {
  return peer_allgather_launch(sources, flags, rank, world, counter, slot_stride_bytes, bytes, output, spin_limit, status,
                               (cudaStream_t)stream);
}

int xqt_b200_swiglu(const void* gate_up, void* output, int m, int inter, int dtype, xqt_b200_stream_t stream) {
  if (m == 0) return 0;
  XQT_REQUIRE(gate_up != nullptr && output != nullptr && inter > 0 && inter % 8 == 0);
  XQT_REQUIRE(dtype == XQT_B200_FP16 || dtype == XQT_B200_BF16);
  return swiglu_launch(gate_up, output, m, inter, dtype, (cudaStream_t)stream);
}

int xqt_b200_workspace_status(const void* workspace, unsigned int* host_status, xqt_b200_stream_t stream) {
  XQT_REQUIRE(workspace != nullptr && host_status != nullptr);
  XQT_CUDA(cudaMemcpyAsync(host_status, workspace, sizeof(unsigned int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  XQT_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}

}  // extern "C"

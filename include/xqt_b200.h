/*
 * C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Conventions (the same ones xqt's own native artifacts follow,
 * xqt/kernels/jit/csrc/gemm/w4a16_sm89.cu:435-521 and
 * xqt/kernels/jit/csrc/quantization/awq_w4a16_sm89_kernel.cu:728-911):
 *   - plain pointers and sizes, no framework types;
 *   - every function returns a cudaError_t as int: 0 on success,
 *     cudaErrorInvalidValue (1) for a request outside the supported envelope,
 *     otherwise the CUDA error of the launch (cudaGetLastError());
 *   - all pointers are device pointers on the current device unless stated;
 *   - work is enqueued on `stream`; no entry point synchronises the host;
 *   - inputs are borrowed and never written; outputs are caller-allocated.
 * Logical convention everywhere: Y[M,N] = A[M,K] * W[N,K]^T.
 */
#ifndef XQT_B200_H_
#define XQT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* xqt_b200_stream_t; /* == cudaStream_t */

/* element types of activations, outputs, scales and zero points */
#define XQT_B200_FP16 0
#define XQT_B200_BF16 1
#define XQT_B200_FP32 2

/* epilogue activation, xqt EpilogueSpec.activation (ops/gemm/contracts.py:308-326) */
#define XQT_B200_ACT_NONE 0
#define XQT_B200_ACT_RELU 1
#define XQT_B200_ACT_GELU 2
#define XQT_B200_ACT_SILU 3

/* kernel choice for the *_run entry points */
#define XQT_B200_VARIANT_AUTO 0
#define XQT_B200_VARIANT_SIMT 1     /* generic CUDA-core kernel: any shape, any group size        */
#define XQT_B200_VARIANT_GEMV 2     /* M <= 16: split-K tensor-core GEMV, HBM-bound                */
#define XQT_B200_VARIANT_TCGEN05 3  /* M > 16: TMA + tcgen05.mma with TMEM accumulators; needs group  */
                                    /* size 64/128, K % 64 == 0, N % 8 == 0.  Where                   */
                                    /* xqt_b200_w4a16_two_pass(m) is 1 (every M > 16 by default) the  */
                                    /* weights are first dequantised to an fp16 scratch, any zero     */
                                    /* point; otherwise the single-pass kernel below                  */
#define XQT_B200_VARIANT_TCGEN05_FUSED 4  /* single-pass form of 3: dequantisation inside the GEMM, no */
                                    /* N*K*2 scratch, INTEGER zero points only                        */

/* Replaces xqt_w4a16_sm89_version / xqt_awq_w4a16_sm89_version
 * (w4a16_sm89.cu:519-521, awq_w4a16_sm89_kernel.cu:909-911). */
const char* xqt_b200_version(void);

/* cudaGetErrorString for the codes returned below. */
const char* xqt_b200_error_string(int code);

/* 1 when `device` has compute capability 10.0, else 0 (the sm_89 bindings gate the same
 * way on (8,9): _impl/gemm_backends/sm89/w4a16_sm89.py:265-267). */
int xqt_b200_device_supported(int device);

/* ------------------------------------------------------------------------------------------
 * W4A16: group-wise int4 weights, fp16/bf16 activations.
 *
 * Replaces xqt_w4a16_sm89_{fp16,bf16}_run[_persistent] (w4a16_sm89.cu:435-517, bound by
 * _impl/gemm_backends/sm89/w4a16_sm89.py:278-299), the fused variant
 * (w4a16_cutlass_fused_sm89.cu:433-553) and the decode GEMV xqt_awq_w4a16_sm89_decode
 * (awq_w4a16_sm89_kernel.cu:746-784).  Same argument meaning; the additions are the element
 * type of scales/zero points (the sm_89 kernels take fp32 only), residual/activation, the
 * caller-owned scratch buffer and the kernel choice.
 *
 *   activation  [M, K] act_dtype, row stride K
 *   qweight     [N, ceil(padded_k/2)] uint8, canonical xqt_int4_nk_v1: low nibble = even k;
 *               two's-complement nibbles when nibble_signed, codes 0..15 otherwise
 *   scales      [N, padded_k/group_size] param_dtype;  zero_points same shape or NULL
 *   bias        [N] fp32 or NULL;  residual [M, N] act_dtype or NULL
 *   output      [M, N] out_dtype: act_dtype, or XQT_B200_FP32 for the unrounded partial sums of a
 *               K-sharded (row-parallel) layer (then no residual; tensor-core GEMM only)
 *   W = (code - zero_point) * scale, fp32 accumulate, bias -> residual -> activation -> one cast
 *   (xqt/kernels/ops/gemm/reference.py:263-271,362-390,527).
 *   workspace   scratch of at least xqt_b200_w4a16_workspace_bytes(m, n, k) bytes; must be zero
 *               before its first use (the kernels leave it zeroed where it matters); one
 *               workspace must not be shared by launches that can overlap on the GPU, nor with
 *               the decode / GEMM entry points below, whose scratch layouts differ.
 * group_size in {32, 64, 128}; M >= 0 (M == 0 is a no-op).
 */
size_t xqt_b200_w4a16_workspace_bytes(int m, int n, int k);

int xqt_b200_w4a16_run(const void* activation, const void* qweight, const void* scales,
                       const void* zero_points, const float* bias, const void* residual,
                       void* output, int m, int n, int k, int padded_k, int group_size,
                       int nibble_signed, int act_dtype, int param_dtype, int out_dtype,
                       int epilogue_activation, void* workspace, size_t workspace_bytes, int variant,
                       xqt_b200_stream_t stream);

/* Kernel the AUTO variant would pick for this problem (one of XQT_B200_VARIANT_*). */
int xqt_b200_w4a16_select_variant(int m, int n, int k, int padded_k, int group_size,
                                  int epilogue_activation, int has_residual);

/* 1 when the fused form (XQT_B200_VARIANT_TCGEN05_FUSED: packed weights dequantised in registers on their way to the
 * tensor core, K split over CTAs when there are few channel tiles) measures faster than the two-pass form for this
 * problem; it needs integer zero points (or none), which only the caller can know. */
int xqt_b200_w4a16_fused_preferred(int m, int n, int k, int padded_k, int group_size);

/* 1 when XQT_B200_VARIANT_TCGEN05 serves this M in two passes (weights dequantised once per call
 * into an fp16 scratch in fp32 arithmetic, then a dense tcgen05 GEMM): in that form any zero
 * point is accepted, integer or not, and xqt_b200_w4a16_workspace_bytes includes N*K*2 bytes for
 * the scratch.  The single-pass form (XQT_B200_VARIANT_TCGEN05_FUSED) needs integer zero points.  No counterpart in
 * xqt: its sm_89 GEMM has one form (xqt/kernels/ops/_impl/cute/awq_w4a16_sm89.py:225-262). */
int xqt_b200_w4a16_two_pass(int m);

/* ------------------------------------------------------------------------------------------
 * W4A16 decode (M <= 16) on the tile-ordered execution layout b200_w4_tile128_v1.
 *
 * Replaces the decode entry xqt_awq_w4a16_sm89_decode and its pack step
 * xqt_awq_w4a16_sm89_pack (awq_w4a16_sm89_kernel.cu:728-784), which also run on a
 * backend-private interleaved layout derived once from the canonical weight
 * (_impl/gemm_backends/sm89/awq_w4a16_decode_sm89.py:16-98).
 *
 *   tiled_weights  uint8 [ceil(N/128)][K/128][16][32][16]   (xqt_b200/prepack.py: tile_w4)
 *   tiled_params   param_dtype [ceil(N/128)][K/128][128/group_size][128][2] = (scale, zero point)
 *   K a multiple of 256; group_size in {32, 64, 128}; 1 <= M <= 16.
 *   workspace      at least xqt_b200_w4a16_decode_workspace_bytes() bytes, zero before first use;
 *                  its first 32-bit word is a status word (0 = ok) that a kernel whose bounded
 *                  wait ran out sets to a non-zero code; read it with xqt_b200_workspace_status.
 */
size_t xqt_b200_w4a16_decode_workspace_bytes(void);
int xqt_b200_w4a16_decode_supported(int m, int n, int k, int group_size);
int xqt_b200_w4a16_decode_tiled(const void* activation, const void* tiled_weights,
                                const void* tiled_params, const float* bias, const void* residual,
                                void* output, int m, int n, int k, int group_size,
                                int nibble_signed, int has_zero_point, int act_dtype,
                                int param_dtype, void* workspace, size_t workspace_bytes,
                                xqt_b200_stream_t stream);

/* W4A16 decode (M <= 16) on tcgen05, execution layout b200_w4_rows128_v1:
 *   row_weights   uint8 [ceil(N/128)][K/128][4 chunks of 32 K][128 channels][16]   (prepack.py: rows_w4)
 *   tiled_params  as above.  Zero points must be integers in [0, 119]; group_size in {64, 128};
 *   K a multiple of 256.  Same replaced reference entry points, arithmetic, workspace and status
 *   rules as xqt_b200_w4a16_decode_tiled; the inner product runs as tcgen05.mma with the
 *   dequantised weights in tensor memory. */
size_t xqt_b200_w4a16_decode_tc_workspace_bytes(void);
int xqt_b200_w4a16_decode_tc_supported(int m, int n, int k, int group_size);
int xqt_b200_w4a16_decode_tc(const void* activation, const void* row_weights, const void* tiled_params,
                             const float* bias, const void* residual, void* output, int m, int n,
                             int k, int group_size, int nibble_signed, int act_dtype, int param_dtype,
                             int out_dtype, void* workspace, size_t workspace_bytes,
                             xqt_b200_stream_t stream);

/* W4A16 decode (M <= 16) as a cluster split-K GEMV, execution layout b200_w4_lanes_v1: the default
 * decode kernel.  Same replaced reference entry points and arithmetic as xqt_b200_w4a16_decode_tiled
 * (xqt_awq_w4a16_sm89_decode / _pack, awq_w4a16_sm89_kernel.cu:728-784; the execution layout plays the
 * role of sm89_awq_w4a16_interleaved_v1, awq_w4a16_decode_sm89.py:16-98).
 *   lane_weights  uint8 [ceil(N/128)][K/128][4 warps][2 row tiles][2 halves][32 lanes][16]   (prepack.py: lanes_w4)
 *                 unsigned codes; two's-complement nibbles are stored as code + 8 and announced by
 *                 nibble_signed = 1
 *   lane_scales   param_dtype [ceil(N/128)][K/128][128/group_size][4 warps][8][4]: the scales of the four
 *                 channels 32w + 16t + 8h + r (index 2t + h) a lane's accumulators belong to
 *   lane_zeros    zero points in the same order, or NULL for symmetric weights
 *   group_size in {64, 128}; K a multiple of 128; 1 <= M <= 16; any zero point (integer or not).
 *   output        [M, N] act_dtype, or fp32 (out_dtype = XQT_B200_FP32: unrounded partial sums of a
 *                 K-sharded layer, then no residual)
 *   residual      [M, N] act_dtype or NULL; it may be the output buffer itself (in-place residual += projection:
 *                 every element is read before it is written)
 *   epilogue_flags  bit 0: round the projection to act_dtype BEFORE adding the residual -- the numerics of the
 *                 unfused `residual + projection(x)` that AWQW4A16Linear.bind_residual keeps
 *                 (xqt/runtime/modules/awq_w4a16_linear.py:665-737); 0: one rounding after the add
 *                 (the GEMM contract, xqt/kernels/ops/gemm/reference.py:362-390)
 *                 bit 1: fused SwiGLU of a horizontally fused gate/up layer (the gate/up fusion with SiLU gating of
 *                 xqt/kernels/ops/_impl/cute/convrot_w8a8_sm89.py:664-917 at decode sizes): the layer's rows were laid
 *                 out so that every 128-row tile holds 64 gate rows followed by their 64 up rows; output is
 *                 [M, N/2] act_dtype = silu(gate) * up, each projection rounded to act_dtype first (the bits of the
 *                 unfused linear -> SwiGLU).  N a multiple of 128, no residual, no fp32 output; bias, if given, is in
 *                 the layer's (interleaved) row order.
 *   status        NULL, or a device word the kernel sets to 64 when the bounded wait for its
 *                 activation copy ran out (the result is then undefined; nothing hangs)
 * Needs no workspace: the K pieces of a tile are the CTAs of one thread-block cluster and reduce
 * through distributed shared memory in a fixed order (bit-reproducible). */
int xqt_b200_w4a16_decode_lanes_supported(int m, int n, int k, int group_size);
/* How the kernel would cut this problem: *warp_quads K pieces inside a CTA (1 or 2) times *cluster
 * CTAs per 128-channel tile (1..8).  set_plan forces one split for every later call of the process
 * (a tuning aid; (0, 0) returns to the automatic choice); a forced split is still shrunk to what the
 * problem's K allows.  No counterpart in the reference, whose decode kernel has one fixed shape
 * (awq_w4a16_sm89_kernel.cu:26-60). */
int xqt_b200_w4a16_decode_lanes_plan(int m, int n, int k, int group_size, int* warp_quads, int* cluster);
int xqt_b200_w4a16_decode_lanes_set_plan(int warp_quads, int cluster);
int xqt_b200_w4a16_decode_lanes(const void* activation, const void* lane_weights, const void* lane_scales,
                                const void* lane_zeros, const float* bias, const void* residual, void* output, int m, int n, int k,
                                int group_size, int nibble_signed, int act_dtype, int param_dtype,
                                int out_dtype, int epilogue_flags, unsigned int* status, xqt_b200_stream_t stream);
/* xqt_b200_w4a16_decode_lanes whose output slot is chosen on the device: with out_select != NULL the result is written
 * at output + ((*out_select + 1) & 1) * out_select_stride bytes (stride a multiple of 16; not with epilogue flag 2).
 * *out_select is the finished-call counter of xqt_b200_peer_allreduce_counted, read after the kernel's dependency on
 * the previous launch: a row-parallel decode layer writes its fp32 partial into the slot the next counted reduction
 * reads, with nothing in the launch arguments changing from call to call (CUDA-graph replay). */
int xqt_b200_w4a16_decode_lanes_select(const void* activation, const void* lane_weights, const void* lane_scales,
                                       const void* lane_zeros, const float* bias, const void* residual, void* output,
                                       int m, int n, int k, int group_size, int nibble_signed, int act_dtype,
                                       int param_dtype, int out_dtype, int epilogue_flags,
                                       const unsigned int* out_select, size_t out_select_stride,
                                       unsigned int* status, xqt_b200_stream_t stream);

/* W4A16 decode with the scratch built into the library: same operation, arguments and result as
 * xqt_b200_w4a16_decode_tiled, minus the workspace pair.  It has no counterpart in the reference.
 *
 * Who it is for: code that may launch kernels but must not allocate device memory at the point
 * of the call -- an inference server whose memory pool was handed out in full at start-up, a
 * plugin running inside a host application that owns the allocator, a real-time loop that
 * forbids allocator calls (they can synchronise the device or fail late).  Such callers pass
 * their pre-existing input and output buffers and nothing else.
 *
 * How: the tickets, partial sums and status word live in a file-scope __device__ array of
 * xqt_b200_w4a16_decode_static_scratch_bytes() bytes (about 2.6 MB) that every GPU using the
 * library holds until the process exits.  The entry point calls no cudaMalloc / cudaFree and no
 * allocating library routine; it enqueues one memset of its tickets and the kernel.
 *   - Limit: N <= xqt_b200_w4a16_decode_static_max_n() (131072); beyond it the call returns
 *     cudaErrorInvalidValue and launches nothing.
 *   - The first call on each device looks the array's device address up (with that device
 *     current) and caches it; make that first call before any stream capture begins.
 *   - All calls on a device share the one array: two calls that can overlap on the GPU (different
 *     streams without an ordering between them) race on it.  Serialise them.
 */
int xqt_b200_w4a16_decode_tiled_static(const void* activation, const void* tiled_weights,
                                       const void* tiled_params, const float* bias,
                                       const void* residual, void* output, int m, int n, int k,
                                       int group_size, int nibble_signed, int has_zero_point,
                                       int act_dtype, int param_dtype, xqt_b200_stream_t stream);
size_t xqt_b200_w4a16_decode_static_scratch_bytes(void);
int xqt_b200_w4a16_decode_static_max_n(void);
/* Copies the status word of the built-in scratch of the current device to *host_status (host pointer)
 * and synchronises `stream`; it describes the LAST call of xqt_b200_w4a16_decode_tiled_static on that
 * device (each call clears it first): 0 = every bounded wait completed.  Allocates nothing. */
int xqt_b200_w4a16_decode_static_status(unsigned int* host_status, xqt_b200_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Activation prologue shared by the W8A8 and W4A4 linears: block-diagonal Hadamard rotation,
 * one rounding to the activation dtype, dynamic symmetric quantisation.
 *
 * Replaces xqt_convrot_w8a8_sm89_quantize_rotated_act / _small_quantize
 * (convrot_w8a8_sm89_kernel.cu:57-504) and the rotate + quantise half of
 * quantize_w4a4_act_fuse_lora (svdq_w4a4_sm89_kernel.cu:24-328).
 *
 *   activation    [M, K] act_dtype
 *   rot_kind      0 none, 1 regular Hadamard (rot_block a power of 4), 2 Sylvester (power of 2)
 *   column_scale  [rot_block] fp32 = signs / sqrt(rot_block) (NULL when rot_kind == 0)
 *   quant_bits    8: per-token scale max(amax,1e-8)/127, codes in [-128,127], scales [M]
 *                 4: per (token, group_size) scale max(amax/7,1e-6), codes in [-8,7], scales [M, K/group_size];
 *                    group_size 0: one scale per token (ConvRotMixedPrecisionLinear's own activation form,
 *                    convrot_4bit.py:669-679), replicated into scales [M, K/64]
 *                 5: the scales and codes of 4, every code written as the byte sign << 7 | magnitude (read as
 *                    FP8 E4M3 that is code * 2^-9 exactly): the operand form xqt_b200_w4a4_gemm consumes
 *                 9: as 8 with the scale rounded to act_dtype, scale = act_dtype(amax/127), 0 and all-zero codes for an
 *                    all-zero token (the activation side of the SVDQuant W8A8 linear, gemm_w8a8.cuh:236-262)
 *                 6: as 5 (group_size 64 or 0) with the scales tile-major, [ceil(M/128)][K/64][128] floats (row r,
 *                    slot g at ((r/128)*K/64 + g)*128 + r%128): what xqt_b200_w4a4_gemm takes with flag 1
 *   codes         one byte per element [M, K] in every mode (int8 for 8 and 4);  rotated: [M, K] act_dtype or
 *                 NULL (the rotated, rounded activation, input of the W4A4 low-rank branch)
 */
int xqt_b200_rotate_quantize(const void* activation, const float* column_scale, void* codes,
                             float* scales, void* rotated, int m, int k, int rot_kind, int rot_block,
                             int quant_bits, int group_size, int act_dtype, xqt_b200_stream_t stream);

/* Per-tensor dynamic int8 quantisation, the activation side of xqt's reference W8A8 linear Int8MmaLinear
 * (xqt/contracts/int8_mma.py:135-149,308-319): scale = max(absmax(activation), eps) / 127,
 * codes = clamp(rint(x / scale), -127, 127).  codes int8 [M,K]; row_scales fp32 [M] receives the scale
 * once per row (the int8 GEMM below takes per-token scales); stats: two floats of caller scratch,
 * [0] = absmax, [1] = scale after the call.  K a multiple of 8. */
int xqt_b200_quantize_per_tensor(const void* activation, void* codes, float* row_scales, float* stats, int m,
                                 int k, int act_dtype, float eps, xqt_b200_stream_t stream);

/* W8A8 GEMM: output[m,n] = int32(sum_k a[m,k] w[n,k]) * act_scale[m] * weight_scale[n] (+ bias[n]).
 * Replaces xqt_convrot_w8a8_sm89_gemm / _small_gemm (convrot_w8a8_sm89_kernel.cu:506-755; the
 * Nunchaku main loop jit/include/nunchaku/gemm_w8a8.cuh:11-61).  act_codes int8 [M,K], weight_codes
 * int8 [N,K] (both K-major), K a multiple of 16, N a multiple of 8, output [M,N] out_dtype.
 * workspace: at least 256 bytes, zero before first use (status word). */
int xqt_b200_w8a8_gemm(const void* act_codes, const void* weight_codes, const float* act_scale,
                       const float* weight_scale, const float* bias, void* output, int m, int n,
                       int k, int out_dtype, void* workspace, size_t workspace_bytes,
                       xqt_b200_stream_t stream);

/* SVDQuant W8A8 (int8 x int8 GEMM with a low-rank branch; replaces quantize_act_lora / gemm_lora of
 * xqt/kernels/jit/csrc/quantization/svdq_w8a8_sm89_kernel.cu, called from _impl/cute/svdq_w8a8_sm89.py:258-312):
 *   xqt_b200_rotate_quantize(quant_bits = 9, rot_kind 0): per-token scale act_dtype(amax/127), int8 codes
 *   xqt_b200_lowrank_down:  la = x * down^T (fp32 [M,32])
 *   xqt_b200_lowrank_up:    low = la16 [M,R] * up16 [N,R]^T in fp32 [M,N]; both operands act_dtype, R (rank_padded) a
 *                           multiple of 64 with zero padding; dense tcgen05 GEMM
 *   xqt_b200_w8a8_gemm_addend: xqt_b200_w8a8_gemm with `addend` (fp32 [M,N], 16-byte aligned, or NULL) added to
 *                           acc * a_s * w_s + bias before the one rounding. */
int xqt_b200_w8a8_gemm_addend(const void* act_codes, const void* weight_codes, const float* act_scale,
                              const float* weight_scale, const float* bias, const float* addend,
                              void* output, int m, int n, int k, int out_dtype, void* workspace,
                              size_t workspace_bytes, xqt_b200_stream_t stream);
int xqt_b200_lowrank_up(const void* la, const void* up, float* output, int m, int n, int rank_padded,
                        int act_dtype, void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * W4A4 SVDQuant / ConvRot linear: after xqt_b200_rotate_quantize(quant_bits = 5, group 64)
 *   la     = rotated [M,K] * down[32,K]^T                              (xqt_b200_lowrank_down)
 *   output = sum_g a_s[m,g] w_s[n,g] int32(sum_{k in g} a_q w_q) + la * up^T + bias   (xqt_b200_w4a4_gemm)
 * Replaces xqt_svdq_w4a4_sm89_quantize_act_fuse_lora / _gemm_lora (svdq_w4a4_sm89_kernel.cu:330-572,
 * Nunchaku main loop gemm_w4a4.cuh:833-1101, low-rank branch lora.cuh:110-243); accumulation across
 * groups is fp32 here (half precision there).
 *   act_codes   [M,K] int4 codes in [-8,7] as sign-magnitude bytes (quant_bits 5 above): the tensor core takes
 *               them, and the weight nibbles widened the same way, as FP8 E4M3 values code * 2^-9, whose 64-K
 *               sums are exact in its fp32 accumulators;  act_scales fp32 [M, K/64]
 *   qweight     canonical signed-nibble storage uint8 [N, K/2] (the composite artifact's packed_residual)
 *   aux         per 128-channel tile t, xqt_b200_w4a4_aux_tile_bytes(K) bytes: fp32 [K/64][128] = w_scale * 2^18
 *               (transposed), then the tile's up factors as a 16 KiB tensor-core operand image: row n holds
 *               bf16 [hi(32) | lo(32)] with hi = bf16(up), lo = bf16(up - hi) (rank padded with zeros to 32), its
 *               eight 16-byte chunks stored at chunk index c ^ (n & 7) (the 128-byte swizzle).  The rank-R branch
 *               is la * up^T on the tensor core from such hi/lo pairs (fp32 sums, the lo x lo term dropped).
 *   down        act_dtype [32, K] (rows past the rank are zero);  la fp32 [ceil(M/128)*128, 32]
 *   K a multiple of 128, N a multiple of 8, rank <= 32.
 *   workspace   xqt_b200_w4a4_workspace_bytes(M, N, K) bytes, 256-byte aligned: the status word (zero before first
 *               use), then scratch the call fills itself: the la operand images and the weights widened to one
 *               sign-magnitude byte each ([N, K], converted once per call by a streaming pre-pass so that the GEMM
 *               takes both operands by TMA; the packed 4-bit storage stays the only persistent copy).
 *   flags       bit 0: act_scales is tile-major (quant_bits 6 above); bit 1: la points at the operand images
 *               xqt_b200_lowrank_down wrote through la_image (ceil(M/128) images of 16 KiB, 128-byte aligned: row r
 *               holds bf16 [hi(32) | lo(32)] of its 32 values, 16-byte chunk c at c ^ (r & 7)) instead of fp32 [M,32].
 *               With both set the call launches the GEMM alone (plus the weight widening unless weight_bytes is given).
 *   weight_bytes  null, or the [N, K] bytes xqt_b200_w4a4_expand_weight made of qweight once (16-byte aligned): an
 *               operand cache the caller chooses to hold (one byte per weight beside the packed half byte); the
 *               per-call widening pass is then skipped and qweight may be null.
 */
size_t xqt_b200_w4a4_workspace_bytes(int m, int n, int k);
int xqt_b200_lowrank_down(const void* rotated, const void* down, float* la, void* la_image, int m, int k, int act_dtype,
                          xqt_b200_stream_t stream);
size_t xqt_b200_w4a4_aux_tile_bytes(int k);
int xqt_b200_w4a4_supported(int m, int n, int k);
int xqt_b200_w4a4_expand_weight(const void* qweight, void* weight_bytes, int n, int k,
                                xqt_b200_stream_t stream);
int xqt_b200_w4a4_gemm(const void* act_codes, const float* act_scales, const void* qweight,
                       const void* weight_bytes, const void* aux, const float* la, const float* bias,
                       void* output, int m, int n, int k, int out_dtype, int flags, void* workspace,
                       size_t workspace_bytes, xqt_b200_stream_t stream);

/* The same linear in its operand-dequantised form, for M >= 256 (xqt_b200_w4a4_dense_preferred):
 * both operands are expanded once per call to fp16 -- code * scale, an exact fp32 product rounded
 * once -- the low-rank pair (la, up) is appended along K, and one dense tcgen05 fp16 GEMM with fp32
 * accumulation gives the output.  Same codes and scales as the integer form; it avoids that form's
 * per-group int32 drain and fp32 scaling, which bound it on the CUDA cores.  Accuracy: the fp16
 * rounding of both operands leaves about 4e-4 of relative error before the output rounding (1.2e-3
 * rel-L2 between bf16 outputs at K = 3072), against 1e-4 for the integer form; callers that need the
 * 1e-3 parity bar use the integer form.  No counterpart in xqt
 * (its sm_89 kernel has int4 tensor-core instructions, Blackwell has none).
 *   weight_scales fp32 [N, K/64] (the artifact's residual_scale);  up fp32 [N, 32] or NULL with la
 *   K a multiple of 64, N a multiple of 8; workspace >= xqt_b200_w4a4_dense_workspace_bytes(m, n, k),
 *   256-byte aligned.
 * xqt_b200_lowrank_down_tc is xqt_b200_lowrank_down on the dense tcgen05 GEMM (la rows >= M are not
 * written); workspace >= 256 bytes (status word). */
size_t xqt_b200_w4a4_dense_workspace_bytes(int m, int n, int k);
int xqt_b200_w4a4_dense_preferred(int m, int n, int k);
int xqt_b200_w4a4_dense(const void* act_codes, const float* act_scales, const void* qweight,
                        const float* weight_scales, const float* la, const float* up, const float* bias,
                        void* output, int m, int n, int k, int out_dtype, void* workspace,
                        size_t workspace_bytes, xqt_b200_stream_t stream);
int xqt_b200_lowrank_down_tc(const void* rotated, const void* down, float* la, int m, int k, int act_dtype,
                             void* workspace, size_t workspace_bytes, xqt_b200_stream_t stream);

/* Reduction step of a row-parallel (K-sharded) linear over NVLink peer memory, with the epilogue
 * fused in.  No counterpart in xqt (it has no multi-device execution; its metadata only records
 * where a shard would go, xqt/kernels/ops/gemm/contracts.py:379-402).
 *   partials[r]  device pointer, valid on THIS GPU, to rank r's fp32 partial [count] for this call
 *                (rank r's own GEMV wrote it; peers' buffers are mapped symmetric / IPC memory)
 *   flags[r]     device pointer to rank r's flag array, 8 x uint32, zero before the first call
 *   call         1, 2, 3, ... the same on every rank; a rank must alternate between two partial
 *                buffers from call to call (the hand-shake has no exit barrier)
 *   output[count] = round(sum over ranks in rank order + bias[i mod n]); count, n multiples of 4
 * Every rank launches it on its own GPU after its GEMV on the same stream.  The wait for the peers
 * is bounded: after spin_limit polls of a peer's flag (0 = the default, 2^22) the kernel stores 128
 * to *status, stops waiting and finishes normally; the output is then NOT the sum and the call must be
 * treated as failed.  status may be device memory or pinned host memory (then the host sees a timeout
 * without synchronising).  `call` comes from the host, so a launch must not be captured into a CUDA
 * graph: a replay would reuse the call number and its hand-shake would pass at once. */
int xqt_b200_peer_allreduce(const void* const* partials, void* const* flags, int rank, int world,
                            unsigned int call, long long count, int n, const float* bias, void* output,
                            int out_dtype, unsigned int spin_limit, unsigned int* status,
                            xqt_b200_stream_t stream);
/* The same reduction with the call number kept in device memory, so that the launch can be captured into a CUDA
 * graph and replayed: counter[0] (zero before the first call, this rank's own device memory, 2 x uint32) counts the
 * finished calls; the kernel works as call counter[0] + 1, reads slot (call & 1) of every rank's two-slot partial buffer
 * (partials[r] = slot 0, the slots slot_stride elements apart) and publishes the new count when its last block ends.
 * The kernel that writes this rank's partial selects the same slot from the same word
 * (xqt_b200_w4a16_decode_lanes_select).  Every rank must make the same sequence of calls. */
int xqt_b200_peer_allreduce_counted(const void* const* partials, void* const* flags, int rank, int world,
                                    unsigned int* counter, long long slot_stride, long long count, int n,
                                    const float* bias, void* output, int out_dtype,
                                    unsigned int spin_limit, unsigned int* status, xqt_b200_stream_t stream);

/* Concatenation step of column-parallel layers over NVLink peer memory, counted (graph-safe) like
 * xqt_b200_peer_allreduce_counted: sources[r] is slot 0 of rank r's two-slot byte buffer (the slots slot_stride_bytes
 * apart), into whose slot (counter + 1) & 1 rank r's kernels wrote `bytes` bytes (xqt_b200_w4a16_decode_lanes_select with
 * the same counter word); output [world][bytes] receives every rank's bytes in rank order (plain 16-byte peer loads).
 * bytes and slot_stride_bytes multiples of 16; same bounded wait and status as the reduction. */
int xqt_b200_peer_allgather_counted(const void* const* sources, void* const* flags, int rank, int world,
                                    unsigned int* counter, long long slot_stride_bytes, long long bytes,
                                    void* output, unsigned int spin_limit, unsigned int* status,
                                    xqt_b200_stream_t stream);

/* SwiGLU gating between the projections of an MLP: output[m, i] = silu(gate_up[m, i]) * gate_up[m, inter + i],
 * evaluated in fp32 and rounded once.  gate_up is [M, 2*inter] (the gate and up projections fused
 * horizontally into one linear), output [M, inter].  Replaces xqt_convrot_w8a8_sm89_fused_swiglu
 * (convrot_w8a8_sm89_kernel.cu:756-837). */
int xqt_b200_swiglu(const void* gate_up, void* output, int m, int inter, int dtype, xqt_b200_stream_t stream);

/* Copies the status word of `workspace` to *host_status (host pointer) and synchronises `stream`.
 * No counterpart in the reference, whose kernels have no device-side waits. */
int xqt_b200_workspace_status(const void* workspace, unsigned int* host_status,
                              xqt_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* XQT_B200_H_ */

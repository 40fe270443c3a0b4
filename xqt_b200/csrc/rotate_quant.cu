// Activation prologue of the W8A8 / W4A4 linears: block-diagonal Hadamard rotation followed by
// dynamic symmetric quantisation, one CTA per token.
//
// Rotation (xqt/compression/quant/quantizers/convrot_4bit.py:85-229, xqt/model/minicpm5_quarot.py:54-93):
// every `block` consecutive features are multiplied by H / sqrt(block) * signs, H the regular
// Hadamard matrix (orders 4^k) or the Sylvester matrix (orders 2^k).  It is evaluated as a fast
// Hadamard transform in fp32 with a FIXED butterfly order so the result is reproducible bit for
// bit on any machine: stages run from the smallest stride up; a regular stage maps (a,b,c,d) at
// distance `stride` to (p+t, p-t, q+r, r-q) with p=a+b, q=a-b, r=c+d, t=c-d; a Sylvester stage maps
// (a,b) to (a+b, a-b).  Then one multiply by column_scale[j] = signs[j]/sqrt(block) and one rounding
// to the activation dtype, the dtype every reference variant quantises the rotated activation in
// (convrot_int8.py:432-452, convrot_w8a8_sm89_kernel.cu:57-333).
//
// Quantisation, IEEE division and round-half-to-even throughout:
//   mode 8: per token,  scale = max(amax, 1e-8) / 127, q = clamp(rint(x/scale), -128, 127)
//           (xqt/kernels/ops/gemm/quantize.py:75-107)
//   mode 9: per token, the scale rounded to the activation dtype: scale = T(amax / 127) (0 for an all-zero token, whose
//           codes are 0), q = clamp(rint(x/scale), -128, 127) -- the activation side of the SVDQuant W8A8 linear
//           (jit/include/nunchaku/gemm_w8a8.cuh:236-262; the reference multiplies by an approximate reciprocal where
//           this divides)
//   mode 4: per (token, group), scale = max(amax/7, 1e-6), q = clamp(rint(x/scale), -8, 7)
//           (convrot_4bit.py:669-679 at the group granularity of gemm_w4a4.cuh:534-624);
//           group == 0 selects the artifact's own per-token form (one scale per token,
//           convrot_4bit.py:669-679), written to every 64-K slot of the scale row so that the
//           group-64 GEMM consumes it unchanged
//   mode 5: the codes and scales of mode 4, each code written as the byte sign << 7 | magnitude.  Read as
//           FP8 E4M3 that byte is the subnormal/first-binade value code * 2^-9 exactly (magnitudes 0..15
//           are linear there), the operand form of the W4A4 GEMM's tcgen05 kind::f8f6f4 MMA.
//   mode 6: mode 5 with the scales written tile-major, [ceil(M/128)][K/64][128] (the scale of row r and 64-K slot g at
//           ((r / 128) * K/64 + g) * 128 + r % 128): the order in which the W4A4 GEMM's producer fetches the two scale
//           rows of a 128-K stage with one 1 KiB copy.  Needs group 64 or 0.
// Codes are written as one byte each in every mode (Blackwell has no int4 MMA).
#include "common.cuh"

namespace xqt_b200 {

constexpr int kRqThreads = 256;

// flags: bit 0 sign-magnitude bytes, bit 1 tile-major scales (int4 modes); bit 2 the per-token int8 scale is rounded to T
__device__ __forceinline__ size_t rq_scale_index(int row, int g, int groups, int flags) {
  return (flags & 2) ? ((size_t)(row >> 7) * groups + g) * 128 + (row & 127) : (size_t)row * groups + g;
}
__device__ __forceinline__ int8_t rq_encode(float q, int signmag) {
  const int c = (int)q;
  return (int8_t)(signmag ? ((c < 0 ? 0x80 : 0) | (c < 0 ? -c : c)) : c);
}

template <typename T>
__global__ void __launch_bounds__(kRqThreads)
rotate_quant_kernel(const T* __restrict__ x, const float* __restrict__ column_scale, int8_t* __restrict__ codes,
                    float* __restrict__ scales, T* __restrict__ x_rot, int k, int rot_kind, int rot_block, int mode,
                    int group, int flags) {
  const int signmag = flags & 1;
  extern __shared__ float v[];  // [k]
  __shared__ float s_red[kRqThreads / 32];
  __shared__ float s_scale;
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* xr = x + (size_t)row * k;
  for (int i = tid; i < k; i += kRqThreads) v[i] = to_float<T>(xr[i]);
  __syncthreads();
  if (rot_kind == 1) {
    for (int stride = 1; stride < rot_block; stride *= 4) {
      for (int b = tid; b < k / 4; b += kRqThreads) {
        const int base = (b / stride) * 4 * stride + (b % stride);
        const float a = v[base], bb = v[base + stride], c = v[base + 2 * stride], d = v[base + 3 * stride];
        const float p = __fadd_rn(a, bb), q = __fsub_rn(a, bb), r = __fadd_rn(c, d), t = __fsub_rn(c, d);
        v[base] = __fadd_rn(p, t);
        v[base + stride] = __fsub_rn(p, t);
        v[base + 2 * stride] = __fadd_rn(q, r);
        v[base + 3 * stride] = __fsub_rn(r, q);
      }
      __syncthreads();
    }
  } else if (rot_kind == 2) {
    for (int stride = 1; stride < rot_block; stride *= 2) {
      for (int b = tid; b < k / 2; b += kRqThreads) {
        const int base = (b / stride) * 2 * stride + (b % stride);
        const float a = v[base], bb = v[base + stride];
        v[base] = __fadd_rn(a, bb);
        v[base + stride] = __fsub_rn(a, bb);
      }
      __syncthreads();
    }
  }
  // normalise, round once to T (kept in fp32 registers/shared memory as the rounded value)
  float amax = 0.f;
  for (int i = tid; i < k; i += kRqThreads) {
    float r = v[i];
    if (rot_kind != 0) r = __fmul_rn(r, column_scale[i % rot_block]);
    const T rounded = from_float<T>(r);
    if (x_rot != nullptr) x_rot[(size_t)row * k + i] = rounded;
    r = to_float<T>(rounded);
    v[i] = r;
    amax = fmaxf(amax, fabsf(r));
  }
  if (mode == 8) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
      float mx = 0.f;
      for (int w = 0; w < kRqThreads / 32; ++w) mx = fmaxf(mx, s_red[w]);
      const float sc = (flags & 4) ? to_float<T>(from_float<T>(__fdiv_rn(mx, 127.0f))) : __fdiv_rn(fmaxf(mx, 1e-8f), 127.0f);
      s_scale = sc;
      scales[row] = sc;
    }
    __syncthreads();
    const float sc = (flags & 4) ? (s_scale > 0.f ? s_scale : 1.f) : fmaxf(s_scale, 1e-8f);
    for (int i = tid; i < k; i += kRqThreads) {
      const float q = fminf(fmaxf(rintf(__fdiv_rn(v[i], sc)), -128.f), 127.f);
      codes[(size_t)row * k + i] = (int8_t)(int)q;
    }
  } else if (group == 0) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
      float mx = 0.f;
      for (int w = 0; w < kRqThreads / 32; ++w) mx = fmaxf(mx, s_red[w]);
      s_scale = fmaxf(__fdiv_rn(mx, 7.0f), 1e-6f);
    }
    __syncthreads();
    const float sc = s_scale;
    for (int gi = tid; gi < k / 64; gi += kRqThreads) scales[rq_scale_index(row, gi, k / 64, flags)] = sc;
    for (int i = tid; i < k; i += kRqThreads) {
      const float q = fminf(fmaxf(rintf(__fdiv_rn(v[i], sc)), -8.f), 7.f);
      codes[(size_t)row * k + i] = rq_encode(q, signmag);
    }
  } else {
    __syncthreads();
    const int groups = k / group;
    for (int gi = tid; gi < groups; gi += kRqThreads) {
      float mx = 0.f;
      for (int e = 0; e < group; ++e) mx = fmaxf(mx, fabsf(v[gi * group + e]));
      const float sc = fmaxf(__fdiv_rn(mx, 7.0f), 1e-6f);
      scales[rq_scale_index(row, gi, groups, flags)] = sc;
      for (int e = 0; e < group; ++e) {
        const float q = fminf(fmaxf(rintf(__fdiv_rn(v[gi * group + e], sc)), -8.f), 7.f);
        codes[(size_t)row * k + gi * group + e] = rq_encode(q, signmag);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Register-resident variant for K % 16 == 0, K <= 16384: thread t owns elements [16t, 16t+16) of the
// token (two 16-byte loads), the butterflies with stride < 16 stay in its registers and the wider
// ones go through warp shuffles (a rotation block of <= 256 elements spans <= 16 lanes).  Every
// output element is produced by exactly the additions and subtractions of the definition above, so
// the result is bit-identical to the shared-memory kernel and to the CPU oracle.
template <typename T>
__global__ void __launch_bounds__(1024)
rotate_quant_fast_kernel(const T* __restrict__ x, const float* __restrict__ column_scale, int8_t* __restrict__ codes,
                         float* __restrict__ scales, T* __restrict__ x_rot, int k, int rot_kind, int rot_block, int mode,
                         int group, int flags) {
  const int signmag = flags & 1;
  __shared__ float s_red[32];
  __shared__ float s_scale;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  const bool active = tid * 16 < k;
  float v[16];
  if (active) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * k + tid * 16);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    const T* a = reinterpret_cast<const T*>(&lo);
    const T* b = reinterpret_cast<const T*>(&hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = to_float<T>(a[i]);
      v[8 + i] = to_float<T>(b[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  if (rot_kind == 1) {
    // regular family: radix-4 stages, strides 1 and 4 in registers, 16 and 64 across lanes
#pragma unroll
    for (int st = 1; st <= 4; st *= 4) {
      if (st < rot_block) {
#pragma unroll
        for (int bfly = 0; bfly < 4; ++bfly) {
          const int base = (bfly / st) * 4 * st + (bfly % st);
          const float a = v[base], b = v[base + st], c = v[base + 2 * st], d = v[base + 3 * st];
          const float p = __fadd_rn(a, b), q = __fsub_rn(a, b), r = __fadd_rn(c, d), t = __fsub_rn(c, d);
          v[base] = __fadd_rn(p, t);
          v[base + st] = __fsub_rn(p, t);
          v[base + 2 * st] = __fadd_rn(q, r);
          v[base + 3 * st] = __fsub_rn(r, q);
        }
      }
    }
#pragma unroll
    for (int L = 1; L <= 4; L *= 4) {          // lane distance 1 <-> stride 16, 4 <-> stride 64
      if (16 * L < rot_block) {
        // The four inputs (a,b,c,d) of a butterfly sit in the lanes whose 2-bit digit is 0..3.
        // Exchange with the lane at distance L: digits {0,1} form p=a+b and q=a-b, digits {2,3} form
        // r=c+d and t=c-d (the odd digit computes the difference the other way round and negates
        // it, which is exact).  Exchange the difference at distance 2L: outputs p+t, p-t, q+r, r-q
        // are then sum +- received difference, minus on odd digits.  Same operations as the definition.
        const uint32_t flip = (lane & L) ? 0x80000000u : 0u;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float own = v[i];
          const float other = __shfl_xor_sync(0xffffffffu, own, L);
          const float sum = __fadd_rn(own, other);
          const float diff = __uint_as_float(__float_as_uint(__fsub_rn(own, other)) ^ flip);
          const float got = __shfl_xor_sync(0xffffffffu, diff, 2 * L);
          v[i] = __fadd_rn(sum, __uint_as_float(__float_as_uint(got) ^ flip));
        }
      }
    }
  } else if (rot_kind == 2) {
#pragma unroll
    for (int st = 1; st <= 8; st *= 2) {
      if (st < rot_block) {
#pragma unroll
        for (int bfly = 0; bfly < 8; ++bfly) {
          const int base = (bfly / st) * 2 * st + (bfly % st);
          const float a = v[base], b = v[base + st];
          v[base] = __fadd_rn(a, b);
          v[base + st] = __fsub_rn(a, b);
        }
      }
    }
#pragma unroll
    for (int L = 1; L <= 8; L *= 2) {          // lane distance L <-> stride 16 L
      if (16 * L < rot_block) {
        const bool upper = (lane & L) != 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, v[i], L);
          v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
        }
      }
    }
  }
  float amax = 0.f;
  {
    T rounded[16];
#pragma unroll
    // the 16 column factors of this thread are contiguous (a rotation block is a multiple of 16 here,
    // or the kernel is not chosen): four vector loads instead of sixteen indexed ones
    float cs[16];
    if (rot_kind != 0 && active) {
      const float4* c4 = reinterpret_cast<const float4*>(column_scale + ((tid * 16) % rot_block));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 c = __ldg(c4 + j);
        cs[4 * j] = c.x; cs[4 * j + 1] = c.y; cs[4 * j + 2] = c.z; cs[4 * j + 3] = c.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) cs[j] = 1.f;
    }
    for (int i = 0; i < 16; ++i) {
      float r = v[i];
      if (rot_kind != 0 && active) r = __fmul_rn(r, cs[i]);
      rounded[i] = from_float<T>(r);
      v[i] = to_float<T>(rounded[i]);
      amax = fmaxf(amax, fabsf(v[i]));
    }
    if (x_rot != nullptr && active) {
      uint4* dst = reinterpret_cast<uint4*>(x_rot + (size_t)row * k + tid * 16);
      dst[0] = *reinterpret_cast<const uint4*>(&rounded[0]);
      dst[1] = *reinterpret_cast<const uint4*>(&rounded[8]);
    }
  }
  float sc;
  float lo_clamp, hi_clamp;
  if (mode == 8) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
      float mx = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, s_red[w]);
      const float s0 = (flags & 4) ? to_float<T>(from_float<T>(__fdiv_rn(mx, 127.0f))) : __fdiv_rn(fmaxf(mx, 1e-8f), 127.0f);
      s_scale = s0;
      scales[row] = s0;
    }
    __syncthreads();
    sc = (flags & 4) ? (s_scale > 0.f ? s_scale : 1.f) : fmaxf(s_scale, 1e-8f);
    lo_clamp = -128.f; hi_clamp = 127.f;
  } else if (group == 0) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) s_red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
      float mx = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, s_red[w]);
      s_scale = fmaxf(__fdiv_rn(mx, 7.0f), 1e-6f);
    }
    __syncthreads();
    sc = s_scale;
    if (active && (tid & 3) == 0) scales[rq_scale_index(row, tid / 4, k / 64, flags)] = sc;     // one 64-K slot per four threads
    lo_clamp = -8.f; hi_clamp = 7.f;
  } else {
    // group of `group` elements = group/16 adjacent lanes (group is 16, 32, 64, ... <= 512)
    for (int off = 1; off < group / 16; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    sc = fmaxf(__fdiv_rn(amax, 7.0f), 1e-6f);
    if (active && (tid % (group / 16)) == 0) scales[rq_scale_index(row, (tid * 16) / group, k / group, flags)] = sc;
    lo_clamp = -8.f; hi_clamp = 7.f;
  }
  if (active) {
    int8_t q[16];
#pragma unroll
    // round(v / sc) with the IEEE quotient: a multiplication by the reciprocal gives the same integer
    // unless it lands within 2^-10 of a rounding boundary; only those elements pay for the division
    const float rcp = __frcp_rn(sc);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float quot = __fmul_rn(v[i], rcp);
      const float nearest = rintf(quot);
      const float dist = fabsf(fabsf(__fsub_rn(quot, nearest)) - 0.5f);   // distance from a half-integer
      float code = nearest;
      if (dist < 0x1p-10f && fabsf(quot) < 512.f) code = rintf(__fdiv_rn(v[i], sc));
      q[i] = rq_encode(fminf(fmaxf(code, lo_clamp), hi_clamp), signmag);
    }
    *reinterpret_cast<uint4*>(codes + (size_t)row * k + tid * 16) = *reinterpret_cast<const uint4*>(q);
  }
}

int rotate_quant_launch(const void* x, const float* column_scale, void* codes, float* scales, void* x_rot, int m, int k,
                        int rot_kind, int rot_block, int mode, int group, int act_dtype, cudaStream_t stream) {
  XQT_REQUIRE(m > 0 && k > 0 && (mode == 8 || mode == 9 || mode == 4 || mode == 5 || mode == 6));
  // modes 5, 6: the int4 codes of mode 4 written as sign-magnitude bytes; mode 6 also orders the scales tile-major;
  // mode 9: mode 8 with the scale rounded to the activation dtype
  const int signmag = mode == 5 ? 1 : (mode == 6 ? 3 : (mode == 9 ? 4 : 0));
  if (mode == 6) XQT_REQUIRE(group == 0 || group == 64);
  if (mode == 5 || mode == 6) mode = 4;
  if (mode == 9) mode = 8;
  XQT_REQUIRE(rot_kind >= 0 && rot_kind <= 2);
  if (rot_kind != 0) {
    XQT_REQUIRE(rot_block >= 1 && k % rot_block == 0 && column_scale != nullptr);
    int v = rot_block;
    const int base = rot_kind == 1 ? 4 : 2;
    while (v % base == 0) v /= base;
    XQT_REQUIRE(v == 1);
  }
  if (mode == 4) XQT_REQUIRE(group == 0 ? k % 64 == 0 : (group > 0 && k % group == 0));
  XQT_REQUIRE(act_dtype == XQT_B200_BF16 || act_dtype == XQT_B200_FP16);
  const bool group_ok = mode == 8 || group == 0 || (group >= 16 && group <= 512 && (group & (group - 1)) == 0);
  const bool block_ok = rot_kind == 0 || (rot_block >= 16 && ((uintptr_t)column_scale & 15) == 0);   // vector loads of the column factors
  if (k % 16 == 0 && k <= 16384 && group_ok && block_ok && ((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 15) == 0 &&
      (x_rot == nullptr || ((uintptr_t)x_rot & 15) == 0)) {
    const int threads = ceil_div(k / 16, 32) * 32;
    if (act_dtype == XQT_B200_BF16)
      rotate_quant_fast_kernel<__nv_bfloat16><<<m, threads, 0, stream>>>(
          (const __nv_bfloat16*)x, column_scale, (int8_t*)codes, scales, (__nv_bfloat16*)x_rot, k, rot_kind, rot_block, mode, group, signmag);
    else
      rotate_quant_fast_kernel<__half><<<m, threads, 0, stream>>>(
          (const __half*)x, column_scale, (int8_t*)codes, scales, (__half*)x_rot, k, rot_kind, rot_block, mode, group, signmag);
    return launch_status();
  }
  const size_t smem = (size_t)k * sizeof(float);
  XQT_REQUIRE(smem <= 200 * 1024);
#define XQT_RQ(TT)                                                                                               \
  do {                                                                                                           \
    auto kern = rotate_quant_kernel<TT>;                                                                         \
    XQT_SMEM_OPT_IN(kern, 200 * 1024);                                                                           \
    kern<<<m, kRqThreads, smem, stream>>>((const TT*)x, column_scale, (int8_t*)codes, scales, (TT*)x_rot, k,     \
                                          rot_kind, rot_block, mode, group, signmag);                            \
  } while (0)
  if (act_dtype == XQT_B200_BF16) XQT_RQ(__nv_bfloat16);
  else XQT_RQ(__half);
#undef XQT_RQ
  return launch_status();
}

}  // namespace xqt_b200

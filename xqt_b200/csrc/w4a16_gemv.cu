// W4A16 decode kernel for M <= 16 (group size 128): a split-K GEMV whose inner product runs on
// the tensor cores so that the instruction issue rate does not cap it below HBM bandwidth.
//
// Budget behind the design: at 6.5 TB/s a B200 streams 1.3e13 int4 weights per second while its
// 148 SMs issue 3.6e13 lane-instructions per second, i.e. under 3 instructions per weight.  A
// CUDA-core GEMV needs M FMAs per weight on top of the unpack, so anything beyond M = 1..2 must
// use MMA.  Here one warp-wide 16-byte load brings 8 output channels x 128 K (exactly one
// quantisation group per channel) straight from the canonical xqt_int4_nk_v1 rows (no repacked
// copy of the weights), the nibbles become exact bf16/fp16 integers with one lop3 + one sub per
// pair, eight mma.m16n8k16 accumulate the group in fp32, and the group scale / zero point are
// applied to the fp32 group sum:  y += s * (sum_k x*q  -  z * sum_k x).  The dequantised weight
// is therefore never rounded to 16 bits; the result matches the fp32 reference
// (xqt/kernels/ops/gemm/reference.py:263-271,527) to fp32 summation order.
//
// K order inside an MMA is free as long as A and B agree, so the lane that holds 32 consecutive
// K of one channel feeds them as K-slots {2t,2t+1,2t+8,2t+9} and the activation slice is staged
// in shared memory in that same order (pairs (k, k+4), the order lop3 extracts nibbles in).
//
// Split-K: CTA (tile, split) owns 64 channels x kc K.  Partials go to a scratch buffer; the last
// CTA to arrive for a tile (atomic ticket, no spinning) adds them in split order, applies bias and
// residual and writes the output, then re-arms the ticket.  The summation order is fixed, so
// results are reproducible run to run (the reference made the same choice for its split-K:
// w4a16_cutlass_fused_sm89.cu:241-248).
#include "common.cuh"

namespace xqt_b200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvRows = 64;          // output channels per CTA (8 n-tiles of 8)
constexpr int kGemvKBlock = 128;       // K per warp-wide load = one quantisation group
constexpr int kGemvMaxKc = 2048;
constexpr int kRedStride = 72;         // padded row of the cross-warp reduction buffer (floats)
constexpr int kGemvMaxCounters = 4096; // tickets at the head of the workspace

template <typename T>
struct Half2Of;
template <>
struct Half2Of<__half> {
  using type = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;        // 1024 + q
  static constexpr uint32_t kOffUnsigned = 0x64006400u;  // subtract 1024
  static constexpr uint32_t kOffSigned = 0x64086408u;    // subtract 1032 (codes were xor 8)
  static constexpr uint32_t kOne = 0x3C003C00u;
};
template <>
struct Half2Of<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;        // 128 + q
  static constexpr uint32_t kOffUnsigned = 0x43004300u;
  static constexpr uint32_t kOffSigned = 0x43084308u;
  static constexpr uint32_t kOne = 0x3F803F80u;
};

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// nibbles i and i+4 of `word` as an exact pair of T integers (K-slots k_i, k_{i+4})
template <typename T, bool SIGNED>
__device__ __forceinline__ uint32_t nibble_pair(uint32_t word, int i) {
  using H = Half2Of<T>;
  uint32_t r;
  const uint32_t shifted = word >> (4 * i);
  asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(shifted), "n"(0x000f000f), "r"(H::kMagic));
  typename H::type v = *reinterpret_cast<typename H::type*>(&r);
  const uint32_t offbits = SIGNED ? H::kOffSigned : H::kOffUnsigned;
  typename H::type off = *reinterpret_cast<const typename H::type*>(&offbits);
  v = __hsub2(v, off);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 8 consecutive T (k0..k7) -> (k0,k4),(k1,k5),(k2,k6),(k3,k7)
__device__ __forceinline__ uint4 pair_permute(uint4 v) {
  uint4 o;
  o.x = __byte_perm(v.x, v.z, 0x5410);
  o.y = __byte_perm(v.x, v.z, 0x7632);
  o.z = __byte_perm(v.y, v.w, 0x5410);
  o.w = __byte_perm(v.y, v.w, 0x7632);
  return o;
}

// KW: warps that split K inside the CTA (and n-tiles handled per warp); kc = K per CTA.
template <typename T, bool SIGNED, bool HAS_ZP, int KW>
__global__ void __launch_bounds__(kGemvThreads, 2)
w4a16_gemv_kernel(const T* __restrict__ x, const uint8_t* __restrict__ qw, const void* __restrict__ scales,
                  const void* __restrict__ zeros, const float* __restrict__ bias, const T* __restrict__ residual,
                  T* __restrict__ out, int m, int n, int k, int param_dtype, int kc, int splits,
                  float* __restrict__ partials, unsigned int* __restrict__ tickets) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x, split = blockIdx.y, ntiles = gridDim.x;
  const int n0 = tile * kGemvRows;
  const int kbase = split * kc;
  const int kblocks = min(kc, k - kbase) / kGemvKBlock;
  const int groups = k / kGemvKBlock;
  const int row_bytes = k / 2;

  // shared memory: [x slice | reduction buffer] (aliased) then per-(kblock,row) {scale, zero}
  const int xbytes = (kc / kGemvKBlock) * 4096;
  const int redbytes = KW * 16 * kRedStride * 4;
  uint4* sx = reinterpret_cast<uint4*>(smem_raw);
  float* sred = reinterpret_cast<float*>(smem_raw);
  float2* ssz = reinterpret_cast<float2*>(smem_raw + (xbytes > redbytes ? xbytes : redbytes));

  const int kb_lane = warp % KW;       // this warp takes kblocks kb_lane, kb_lane + KW, ...
  const int nt0 = (warp / KW) * KW;    // and n-tiles nt0 .. nt0 + KW - 1 of the CTA's eight

  // 1. get the first weight vectors in flight before anything else waits on memory
  uint4 wv[KW];
  auto load_weight = [&](int kb, int j) {
    int row = n0 + (nt0 + j) * 8 + g;
    row = row < n ? row : n - 1;
    return __ldg(reinterpret_cast<const uint4*>(qw + (size_t)row * row_bytes + (kbase + kb * kGemvKBlock) / 2) + t);
  };
  if (kb_lane < kblocks) {
#pragma unroll
    for (int j = 0; j < KW; ++j) wv[j] = load_weight(kb_lane, j);
  }

  // 2. stage the activation slice [16, kc] in MMA-fragment order, rows >= m as zeros
  {
    const int chunks_per_row = kblocks * 16;  // 16-byte chunks (8 K) per row of the slice
    for (int i = tid; i < 16 * chunks_per_row; i += kGemvThreads) {
      const int r = i / chunks_per_row, c = i % chunks_per_row;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < m) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * k + kbase) + c);
      const int kb = c >> 4, cc = c & 15;      // chunk cc covers k = 8*cc .. 8*cc+7 of the kblock
      const int tt = cc >> 2, w = cc & 3;      // lane tt reads word w of its 32-K run
      sx[kb * 256 + w * 64 + r * 4 + tt] = pair_permute(v);
    }
    for (int i = tid; i < kblocks * kGemvRows; i += kGemvThreads) {
      const int r = i / kblocks, kb = i % kblocks;
      int row = n0 + r;
      row = row < n ? row : n - 1;
      const size_t idx = (size_t)row * groups + kbase / kGemvKBlock + kb;
      float2 sz;
      sz.x = load_param(scales, param_dtype, idx);
      sz.y = HAS_ZP ? load_param(zeros, param_dtype, idx) : 0.f;
      ssz[kb * kGemvRows + r] = sz;
    }
  }
  __syncthreads();

  // 3. main loop
  float acc[KW][4];
#pragma unroll
  for (int j = 0; j < KW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  for (int kb = kb_lane; kb < kblocks; kb += KW) {
    uint4 alo[4], ahi[4];  // rows g and g+8, one vector per 8-K word
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      alo[w] = sx[kb * 256 + w * 64 + g * 4 + t];
      ahi[w] = sx[kb * 256 + w * 64 + (g + 8) * 4 + t];
    }
    float xs[4] = {0.f, 0.f, 0.f, 0.f};  // sum_k x over the group, rows g (xs[0]) and g+8 (xs[2])
    if (HAS_ZP) {
      const uint32_t one = Half2Of<T>::kOne;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mma16816<T>(xs, alo[w].x, ahi[w].x, alo[w].y, ahi[w].y, one, one);
        mma16816<T>(xs, alo[w].z, ahi[w].z, alo[w].w, ahi[w].w, one, one);
      }
    }
#pragma unroll
    for (int j = 0; j < KW; ++j) {
      float grp[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t words[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
      if (kb + KW < kblocks) wv[j] = load_weight(kb + KW, j);  // refill this slot for the next K block
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t word = SIGNED ? (words[w] ^ 0x88888888u) : words[w];
        const uint32_t p0 = nibble_pair<T, SIGNED>(word, 0), p1 = nibble_pair<T, SIGNED>(word, 1);
        const uint32_t p2 = nibble_pair<T, SIGNED>(word, 2), p3 = nibble_pair<T, SIGNED>(word, 3);
        mma16816<T>(grp, alo[w].x, ahi[w].x, alo[w].y, ahi[w].y, p0, p1);
        mma16816<T>(grp, alo[w].z, ahi[w].z, alo[w].w, ahi[w].w, p2, p3);
      }
      // C fragment: grp[0],grp[1] = (row g; channels 2t, 2t+1), grp[2],grp[3] = (row g+8; same)
      const float4 sz = *reinterpret_cast<const float4*>(&ssz[kb * kGemvRows + (nt0 + j) * 8 + 2 * t]);
      if (HAS_ZP) {
        acc[j][0] = fmaf(sz.x, fmaf(-sz.y, xs[0], grp[0]), acc[j][0]);
        acc[j][1] = fmaf(sz.z, fmaf(-sz.w, xs[0], grp[1]), acc[j][1]);
        acc[j][2] = fmaf(sz.x, fmaf(-sz.y, xs[2], grp[2]), acc[j][2]);
        acc[j][3] = fmaf(sz.z, fmaf(-sz.w, xs[2], grp[3]), acc[j][3]);
      } else {
        acc[j][0] = fmaf(sz.x, grp[0], acc[j][0]);
        acc[j][1] = fmaf(sz.z, grp[1], acc[j][1]);
        acc[j][2] = fmaf(sz.x, grp[2], acc[j][2]);
        acc[j][3] = fmaf(sz.z, grp[3], acc[j][3]);
      }
    }
  }
  __syncthreads();  // every warp is done with the activation slice; reuse it as reduction buffer

  // 4. reduce across the KW warps that split K: sred[kb_lane][16 rows][64 channels (padded)]
#pragma unroll
  for (int j = 0; j < KW; ++j) {
    const int ch = (nt0 + j) * 8 + 2 * t;
    float* base = sred + kb_lane * 16 * kRedStride;
    *reinterpret_cast<float2*>(base + g * kRedStride + ch) = make_float2(acc[j][0], acc[j][1]);
    *reinterpret_cast<float2*>(base + (g + 8) * kRedStride + ch) = make_float2(acc[j][2], acc[j][3]);
  }
  __syncthreads();
  const int om = tid >> 4, oc = (tid & 15) * 4;  // this thread: activation row om, channels oc..oc+3
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int w = 0; w < KW; ++w) {
    const float4 v = *reinterpret_cast<const float4*>(sred + w * 16 * kRedStride + om * kRedStride + oc);
    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
  }

  // 5. split-K: publish the partial, the last CTA of the tile finishes it
  if (splits > 1) {
    float4* mine = reinterpret_cast<float4*>(partials + ((size_t)split * ntiles + tile) * (16 * kGemvRows));
    mine[tid] = sum;
    __threadfence();
    __shared__ unsigned int s_ticket;
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(&tickets[tile], 1u);
    __syncthreads();
    if (s_ticket != (unsigned)(splits - 1)) return;
    __threadfence();
    sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(partials + ((size_t)s * ntiles + tile) * (16 * kGemvRows)) + tid);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    if (tid == 0) tickets[tile] = 0u;  // re-arm for the next launch
  }
  if (om < m) {
    float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int ch = n0 + oc + e;
      if (ch < n) {
        float v = vals[e];
        if (bias != nullptr) v += bias[ch];
        const size_t o = (size_t)om * n + ch;
        if (residual != nullptr) v += to_float<T>(residual[o]);
        out[o] = from_float<T>(v);
      }
    }
  }
}

struct GemvPlan {
  int kc, kw, splits, tiles;
  size_t smem;
};

static GemvPlan gemv_plan(int n, int k, int num_sms) {
  GemvPlan p;
  p.tiles = ceil_div(n, kGemvRows);
  int kc = kGemvMaxKc;
  // the largest K chunk that still yields about two CTAs per SM
  while (kc > kGemvKBlock && (long)p.tiles * ceil_div(k, kc) < 2L * num_sms) kc >>= 1;
  p.kc = kc;
  p.kw = kc / kGemvKBlock >= 8 ? 8 : kc / kGemvKBlock;
  p.splits = ceil_div(k, kc);
  const size_t xbytes = (size_t)(kc / kGemvKBlock) * 4096, redbytes = (size_t)p.kw * 16 * kRedStride * 4;
  p.smem = (xbytes > redbytes ? xbytes : redbytes) + (size_t)(kc / kGemvKBlock) * kGemvRows * sizeof(float2);
  return p;
}

static int cached_sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (counts[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    counts[dev] = v;
  }
  return counts[dev];
}

size_t w4a16_gemv_workspace_bytes(int n, int k) {
  // tickets, then one [16, 64] fp32 partial per (split, tile).  Sized for the split a device
  // with up to 256 SMs would choose, which bounds what any B200 launch needs.
  const GemvPlan p = gemv_plan(n, k, 256);
  return 256 + (size_t)kGemvMaxCounters * sizeof(unsigned int) +
         (size_t)p.splits * p.tiles * 16 * kGemvRows * sizeof(float);
}

bool w4a16_gemv_supported(int m, int n, int k, int padded_k, int group_size) {
  return m >= 1 && m <= 16 && group_size == kGemvKBlock && padded_k == k && k % kGemvKBlock == 0 && n >= 1 &&
         ceil_div(n, kGemvRows) <= kGemvMaxCounters;
}

template <typename T, bool SIGNED, bool HAS_ZP>
static int gemv_dispatch_kw(const GemvPlan& p, const void* x, const void* qw, const void* scales, const void* zeros,
                            const float* bias, const void* residual, void* out, int m, int n, int k, int param_dtype,
                            float* partials, unsigned int* tickets, cudaStream_t stream) {
  const dim3 grid(p.tiles, p.splits), block(kGemvThreads);
#define XQT_GEMV_LAUNCH(KWV)                                                                              \
  do {                                                                                                    \
    auto kern = w4a16_gemv_kernel<T, SIGNED, HAS_ZP, KWV>;                                                \
    XQT_SMEM_OPT_IN(kern, 96 * 1024); /* the largest dynamic shared memory any plan uses */               \
    kern<<<grid, block, p.smem, stream>>>((const T*)x, (const uint8_t*)qw, scales, zeros, bias,           \
                                          (const T*)residual, (T*)out, m, n, k, param_dtype, p.kc,        \
                                          p.splits, partials, tickets);                                   \
  } while (0)
  switch (p.kw) {
    case 8: XQT_GEMV_LAUNCH(8); break;
    case 4: XQT_GEMV_LAUNCH(4); break;
    case 2: XQT_GEMV_LAUNCH(2); break;
    default: XQT_GEMV_LAUNCH(1); break;
  }
#undef XQT_GEMV_LAUNCH
  return launch_status();
}

int w4a16_gemv_launch(const void* x, const void* qw, const void* scales, const void* zeros, const float* bias,
                      const void* residual, void* out, int m, int n, int k, int nibble_signed, int act_dtype,
                      int param_dtype, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const GemvPlan p = gemv_plan(n, k, cached_sm_count());
  // workspace: [0,256) status block, [256, 256+16 KiB) tickets (must stay zero between launches),
  // then partial sums (need not be zero; the tensor-core GEMM uses the same area as its scratch)
  const size_t need = 256 + (size_t)kGemvMaxCounters * sizeof(unsigned int) +
                      (p.splits > 1 ? (size_t)p.splits * p.tiles * 16 * kGemvRows * sizeof(float) : 0);
  if (p.splits > 1) XQT_REQUIRE(workspace != nullptr && workspace_bytes >= need);
  unsigned int* tickets = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(workspace) + 256);
  float* partials = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 256 + kGemvMaxCounters * sizeof(unsigned int));
  const bool zp = zeros != nullptr;
#define XQT_GEMV_T(TT)                                                                                             \
  do {                                                                                                             \
    if (nibble_signed) {                                                                                           \
      if (zp) return gemv_dispatch_kw<TT, true, true>(p, x, qw, scales, zeros, bias, residual, out, m, n, k, param_dtype, partials, tickets, stream);   \
      return gemv_dispatch_kw<TT, true, false>(p, x, qw, scales, zeros, bias, residual, out, m, n, k, param_dtype, partials, tickets, stream);          \
    }                                                                                                              \
    if (zp) return gemv_dispatch_kw<TT, false, true>(p, x, qw, scales, zeros, bias, residual, out, m, n, k, param_dtype, partials, tickets, stream);    \
    return gemv_dispatch_kw<TT, false, false>(p, x, qw, scales, zeros, bias, residual, out, m, n, k, param_dtype, partials, tickets, stream);           \
  } while (0)
  if (act_dtype == XQT_B200_BF16) XQT_GEMV_T(__nv_bfloat16);
  XQT_GEMV_T(__half);
#undef XQT_GEMV_T
}

}  // namespace xqt_b200

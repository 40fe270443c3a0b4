// W4A16 decode (M <= 16) as a cluster split-K GEMV on the lane-ordered execution layout
// b200_w4_lanes_v1.  No scratch memory in global memory, no tickets: the K pieces of one 128-channel
// tile are the CTAs of one thread-block cluster and meet in distributed shared memory.
//
// Work split.  A tile is 128 output channels.  Its K range is cut into `pieces` = KW x S runs of
// 128-K blocks: S CTAs (the cluster) times KW warp quads inside a CTA.  One warp owns 32 channels
// (two 16-row A tiles of mma.m16n8k16) of one piece; it streams its packed weights straight from
// global memory into registers with 16-byte loads (512 contiguous bytes per warp and request), three
// 64-K half blocks ahead of the arithmetic (a four-slot register ring), and asks for the rest of its
// piece into L2 with bulk prefetches on entry; nothing in the main loop waits on a barrier.
// Measured alternatives that lost: staging the activations with 16-byte loads by all threads and adding the group
// sums on the way, in place of the bulk copies and the tensor-core pass (slower at every M: each batch of loads is an
// L2 round trip, 0.2-0.5 us more at M = 1 and 2-3 us more at M = 16); staging the weights through per-warp shared-memory rings filled by
// bulk copies (64 registers, four CTAs per SM: 11.5 us against 9.4 us on the 31 MB layers), an
// 80-register build for three CTAs per SM (12.9 us: future kernels' CTAs crowd the SMs), and per-owner
// mbarrier arrivals in place of the closing cluster barrier (11.2 us).
//
// Arithmetic.  A nibble becomes the exact bf16/fp16 integer B + q with one shift and one lop3
// (B = 128 or 1024, the value of the exponent pattern it is or-ed into); eight MMAs accumulate one
// 128-K block in fp32; the group's scale and zero point are applied to the fp32 group sum:
//     y[m] += s * (sum_k x[m,k] (B + q[k])  -  (B + z) * sum_k x[m,k]).
// The dequantised weight is never rounded, the zero point may be any real number, and the result
// equals the contract reference (xqt/kernels/ops/gemm/reference.py:263-271,527) up to fp32
// summation order.  The activation group sums sum_k x[m,k] come from the tensor cores too (an MMA
// whose A operand is all ones), once per CTA, while the first weights are in flight.
//
// Activations.  The CTA's K slice of x is copied once into shared memory with one bulk copy per
// token row (rows are padded by 64 bytes so that the B-fragment loads are conflict-free).  K order
// inside an MMA is free as long as A and B agree: lane (r, c) feeds K-slots
// k = 32*(j/2) + 8*c + 4*(j%2) + {0,1,2,3} in step j, i.e. 16 contiguous bytes of x per two steps.
//
// Reduction (fixed order, bit-reproducible): warp quads of a CTA add through shared memory; the
// CTAs of a cluster scatter their sums by token to the CTA that owns the token (token mod S) with
// plain st.shared::cluster stores, one cluster barrier, and every CTA finishes its own tokens:
// sum over the pieces in rank order, bias, residual, one rounding.
//
// Programmatic dependent launch: the weights never depend on an earlier kernel, so their first
// loads are issued before griddepcontrol.wait; activations, residual and output are touched after it.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace xqt_b200 {

using namespace sm100;

namespace dcl {
constexpr int kTileRows = 128;
constexpr int kKB = 128;              // K per block: one 32-byte load per (lane, A tile)
constexpr int kMaxCluster = 8;        // portable cluster size
constexpr int kMaxKW = 2;             // warp quads (K pieces) per CTA
#ifndef XQT_DCL_MIN_CTAS
#define XQT_DCL_MIN_CTAS 2
#endif
constexpr int kMinCtasSmallM = XQT_DCL_MIN_CTAS;   // resident 8-warp CTAs per SM the M <= 8 kernels are compiled for
constexpr int kMaxThreads = 128 * kMaxKW;
constexpr int kRedStride = 132;       // floats per token row of the reduction buffers (conflict-free)
constexpr int kXPad = 64;             // bytes added to a shared-memory row of x
constexpr int kMaxSliceBlocks8 = 48;  // longest K slice of a CTA, in blocks, for M <= 8 ...
constexpr int kMaxSliceBlocks16 = 24; // ... and for M <= 16 (about 100 KiB of activations)
enum Status : unsigned int { kTimeout = 64 };
}  // namespace dcl

struct DecodeClParams {
  const uint8_t* wt;    // [tiles][kblocks][4 warps][2 A tiles][32 lanes][32 B]
  const uint8_t* scl;   // scales      [tiles][kblocks][128/g][4 warps][8 rows][4] P
  const uint8_t* zer;   // zero points, same shape, or null (symmetric weights)
  const void* x;        // [M][K]
  const float* bias;
  const void* residual;
  void* out;
  unsigned int* status; // may be null
  int m, n, k, out_f32;
  int round_first;      // 1: round the projection to T before the residual is added (unfused `residual + proj` numerics)
  const unsigned int* out_select;   // null, or a device word w: the output goes to out + ((w + 1) & 1) * out_select_stride bytes
  long long out_select_stride;      // (the slot of a two-slot buffer that the counted peer reduction will read next)
  int glu;              // 1: a tile is 64 gate channels followed by their 64 up channels; out[M, N/2] = silu(gate) * up
  int kblocks, pieces, kw;
  int per, rem;         // kblocks = pieces * per + rem: piece i starts at i * per + min(i, rem)
  int xrow_bytes;       // shared-memory row stride of x
  int off_xsum, off_redl, off_redc;   // byte offsets inside dynamic shared memory
  int own_max;          // tokens a CTA can own: ceil(8*NT / S)
  int prefetch;         // 1: request each warp's whole piece into L2 at kernel start
  float base_off;       // B (+ 8 when the stored nibbles were two's complement)
};

template <typename T>
struct ClTraits;
template <>
struct ClTraits<__half> {
  static constexpr uint32_t kMagic = 0x64006400u;
  static constexpr uint32_t kOnes = 0x3C003C00u;
};
template <>
struct ClTraits<__nv_bfloat16> {
  static constexpr uint32_t kMagic = 0x43004300u;
  static constexpr uint32_t kOnes = 0x3F803F80u;
};

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cl_lds128(uint32_t (&v)[4], uint32_t addr) {
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
__device__ __forceinline__ float2 cl_lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float cl_lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void cl_sts32f(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cl_sts128z(uint32_t addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr), "r"(0u) : "memory");
}

// element `hi` (0 or 1) of two 16-bit parameters packed in one register
template <typename P>
__device__ __forceinline__ float unpack_half(uint32_t v, int hi);
template <>
__device__ __forceinline__ float unpack_half<__nv_bfloat16>(uint32_t v, int hi) {
  return __uint_as_float(hi ? (v & 0xffff0000u) : (v << 16));
}
template <>
__device__ __forceinline__ float unpack_half<__half>(uint32_t v, int hi) {
  const __half2 h = *reinterpret_cast<const __half2*>(&v);
  return hi ? __high2float(h) : __low2float(h);
}

// T: activation / output type; P: type of the stored (scale, zero point) pairs; GK: quantisation
// group (64 or 128); NT: 8-token MMA tiles (1 for M <= 8, 2 for M <= 16)
template <typename T, typename P, int GK, int NT>
__global__ void __launch_bounds__(dcl::kMaxThreads, NT == 1 ? dcl::kMinCtasSmallM : 2)
w4a16_decode_cl_kernel(const DecodeClParams p) {
  using namespace dcl;
  using Tr = ClTraits<T>;
  constexpr int SUB = kKB / GK;           // groups per block
  constexpr int STEPS = 8 / SUB;          // MMA K-steps per group
  constexpr int MP = 8 * NT;              // token rows held in shared memory
  constexpr bool P32 = sizeof(P) == 4;
  constexpr int PR = P32 ? 2 : 4;         // parameter registers per (slot, group)
  constexpr int kPrmBlockBytes = SUB * 128 * (int)sizeof(P);   // scales (or zero points) of one tile and 128-K block

  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_s = smem_addr(smem);
  const uint32_t xbar = smem_s;                       // mbarrier of the activation copy
  const uint32_t zero_s = smem_s + 128;               // 256 bytes of zeros: the activation row of tokens >= M
  const uint32_t xs_s = smem_s + 384;                 // x rows 0..M-1
  const uint32_t xsum_s = smem_s + p.off_xsum;        // [slice blocks][SUB][16] fp32
  const uint32_t redl_s = smem_s + p.off_redl;        // [KW-1][MP][kRedStride] fp32
  const uint32_t redc_s = smem_s + p.off_redc;        // [S][own_max][kRedStride] fp32

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int w = warp & 3, kwi = warp >> 2;
  const int r = lane >> 2, c = lane & 3;
  const int nthreads = blockDim.x;
  const uint32_t S = cluster_nctarank(), rank = cluster_ctarank();
  const int tile = (int)cluster_id_x();

  auto piece_start = [&](int piece) { return piece * p.per + min(piece, p.rem); };
  const int piece = (int)rank * p.kw + kwi;
  const int kb0 = piece_start(piece), kb1 = piece_start(piece + 1);
  const int cta_kb0 = piece_start((int)rank * p.kw), cta_kb1 = piece_start(((int)rank + 1) * p.kw);
  const int nkb = kb1 - kb0;

  const uint8_t* wp = p.wt + (((size_t)tile * p.kblocks + kb0) * 4 + w) * 2048 + lane * 16;   // next block to request
  // a lane's four channels (32w + 16t + 8h + r, index 2t + h) are adjacent: one 8-byte load of 16-bit
  // parameters; with fp32 parameters lane c loads entry c and the quad exchanges them by shuffle
  const size_t poff = ((size_t)tile * p.kblocks + kb0) * kPrmBlockBytes + (P32 ? ((w * 8 + r) * 4 + c) * 4 : (w * 8 + r) * 8);
  const uint8_t* sp = p.scl + poff;
  const uint8_t* zp = p.zer != nullptr ? p.zer + poff : nullptr;

  // register ring of four 64-K half blocks: [slot][row tile][word of K-step]; slot parity = half.
  // Parameters travel with the second half of their block (group 128: one set per block, two sets
  // held) or with every half (group 64: one set per half, four held).
  constexpr int NPR = GK == 64 ? 4 : 2;
  uint32_t wq[4][2][4];
  uint32_t pr[NPR][PR];
  auto load = [&](auto slot_c) {
    constexpr int slot = decltype(slot_c)::value;
    constexpr int half = slot & 1;
    ldg128_stream(wq[slot][0], wp + half * 512);
    ldg128_stream(wq[slot][1], wp + 1024 + half * 512);
    if constexpr (GK == 64 || half == 1) {
      constexpr int set = GK == 64 ? slot : (slot >> 1);
      constexpr int sub_off = GK == 64 ? half * (kPrmBlockBytes / 2) : 0;
      if constexpr (P32) {
        pr[set][0] = ldg32_stream(sp + sub_off);
        pr[set][1] = zp != nullptr ? ldg32_stream(zp + sub_off) : 0u;
      } else {
        ldg64_stream(*reinterpret_cast<uint32_t(*)[2]>(&pr[set][0]), sp + sub_off);
        if (zp != nullptr) ldg64_stream(*reinterpret_cast<uint32_t(*)[2]>(&pr[set][2]), zp + sub_off);
        else pr[set][2] = pr[set][3] = 0u;
      }
    }
    if constexpr (half == 1) {
      wp += 8192;
      sp += kPrmBlockBytes;
      if (zp != nullptr) zp += kPrmBlockBytes;
    }
  };
  using I0 = std::integral_constant<int, 0>;
  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, 2>;
  using I3 = std::integral_constant<int, 3>;
  const int halves = 2 * nkb;

  // the first weights are on their way before anything else happens
  if (halves > 0) {
    load(I0{});
    load(I1{});
  }
  if (halves > 2) load(I2{});
  // ... and the rest of this warp's piece is requested into L2 right away (one bulk prefetch per
  // block and lane: the warp's 2 KiB of a block are contiguous), so that the whole layer is in
  // flight from HBM from the first microsecond and the register ring only has to cover L2 latency
  for (int i = 1 + lane; i < nkb && p.prefetch; i += 32) {
    bulk_prefetch_l2(p.wt + (((size_t)tile * p.kblocks + kb0 + i) * 4 + w) * 2048, 2048);
    bulk_prefetch_l2(p.scl + ((size_t)tile * p.kblocks + kb0 + i) * kPrmBlockBytes + w * (kPrmBlockBytes / 4), kPrmBlockBytes / 4);
    if (p.zer != nullptr)
      bulk_prefetch_l2(p.zer + ((size_t)tile * p.kblocks + kb0 + i) * kPrmBlockBytes + w * (kPrmBlockBytes / 4), kPrmBlockBytes / 4);
  }

  if (tid == 0) {
    mbar_init(xbar, 1);
    fence_barrier_init();
  }
  if (S > 1) cluster_arrive_relaxed();   // phase 0: "this CTA runs"; waited for before the first remote store

  const int slice_kb = cta_kb1 - cta_kb0;
  const int slice_bytes = slice_kb * 256;
  if (tid < 16) cl_sts128z(zero_s + tid * 16);
  __syncthreads();                        // barrier initialised, zero row written
  grid_dependency_wait();                 // x, residual and out may belong to the kernel before this one
  if (tid == 0) {
    mbar_expect_tx(xbar, (uint32_t)(p.m * slice_bytes));
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.x) + (size_t)cta_kb0 * 256;
    for (int row = 0; row < p.m; ++row)
      bulk_g2s(xs_s + row * p.xrow_bytes, src + (size_t)row * p.k * 2, (uint32_t)slice_bytes, xbar);
  }
  if (!mbar_wait(xbar, 0)) {
    if (p.status != nullptr) atomicExch(p.status, (unsigned int)kTimeout);
  }

  // The next kernel of the stream may become resident from here on (measured: triggering it at entry
  // instead lets several future kernels pile up on the SMs and costs the small layers 0.2 us each).
  grid_launch_dependents();
  // activation group sums on the tensor cores: A = ones, so every row of the result is sum_k x[m,k]
  {
    const int nwarps = nthreads >> 5;
    uint32_t ones[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) asm volatile("mov.b32 %0, %1;\n" : "=r"(ones[i]) : "n"(Tr::kOnes));
    for (int item = warp; item < slice_kb * NT; item += nwarps) {
      const int kbl = item / NT, nt = item - kbl * NT;
      const int row = nt * 8 + r;
      const uint32_t xrow = (row < p.m ? xs_s + row * p.xrow_bytes + kbl * 256 : zero_s) + c * 16;
#pragma unroll
      for (int sub = 0; sub < SUB; ++sub) {
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int jj = 0; jj < STEPS; jj += 2) {
          uint32_t xb[4];
          cl_lds128(xb, xrow + ((sub * STEPS + jj) >> 1) * 64);
          mma_16816<T>(sum, ones, xb[0], xb[1]);
          mma_16816<T>(sum, ones, xb[2], xb[3]);
        }
        if (r == 0) {
          const uint32_t a = xsum_s + (((kbl * SUB + sub) * 16) + nt * 8 + 2 * c) * 4;
          cl_sts32f(a, sum[0]);
          cl_sts32f(a + 4, sum[1]);
        }
      }
    }
  }
  __syncthreads();

  float acc[2][NT][4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][nt][i] = 0.f;

  uint32_t magic;
  asm volatile("mov.b32 %0, %1;\n" : "=r"(magic) : "n"(Tr::kMagic));
  const float base_off = p.base_off;

  // this lane's activation row per n-tile (token 8*nt + r) and its advance per block: rows of
  // tokens >= M all read the zero row and do not advance
  uint32_t xrow[NT], xstep[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int row = nt * 8 + r;
    xrow[nt] = (row < p.m ? xs_s + row * p.xrow_bytes + (kb0 - cta_kb0) * 256 : zero_s) + c * 16;
    xstep[nt] = row < p.m ? 256u : 0u;
  }
  uint32_t xsum_a = xsum_s + ((kb0 - cta_kb0) * SUB * 16 + 2 * c) * 4;

  float tmp[2][NT][4];
  auto compute = [&](auto slot_c) {
    constexpr int slot = decltype(slot_c)::value;
    constexpr int half = slot & 1;
    if constexpr (GK == 64 || half == 0) {
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int v = 0; v < 4; ++v) tmp[t][nt][v] = 0.f;
    }
    uint32_t xb[NT][4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      if ((jj & 1) == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) cl_lds128(xb[nt], xrow[nt] + (half * 2 + (jj >> 1)) * 64);
      }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t word = wq[slot][t][jj];
        uint32_t a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(a[i]) : "r"(word >> (4 * i)), "n"(0x000f000f), "r"(magic));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_16816<T>(tmp[t][nt], a, xb[nt][(jj & 1) * 2], xb[nt][(jj & 1) * 2 + 1]);
      }
    }
    if constexpr (GK == 64 || half == 1) {
      // y += s * (group sum - (B + z) * sum_k x)
      constexpr int sub = GK == 64 ? half : 0;
      constexpr int set = GK == 64 ? slot : (slot >> 1);
      float2 xs2[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) xs2[nt] = cl_lds64f(xsum_a + (sub * 16 + nt * 8) * 4);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float sc, z;
          if constexpr (P32) {
            const int from = (lane & ~3) | (t * 2 + h);
            sc = __uint_as_float(__shfl_sync(0xffffffffu, pr[set][0], from));
            z = __uint_as_float(__shfl_sync(0xffffffffu, pr[set][1], from));
          } else {
            sc = unpack_half<P>(pr[set][t], h);
            z = unpack_half<P>(pr[set][2 + t], h);
          }
          const float nzb = -(z + base_off);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            acc[t][nt][h * 2 + 0] = fmaf(sc, fmaf(nzb, xs2[nt].x, tmp[t][nt][h * 2 + 0]), acc[t][nt][h * 2 + 0]);
            acc[t][nt][h * 2 + 1] = fmaf(sc, fmaf(nzb, xs2[nt].y, tmp[t][nt][h * 2 + 1]), acc[t][nt][h * 2 + 1]);
          }
        }
      }
    }
    if constexpr (half == 1) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) xrow[nt] += xstep[nt];
      xsum_a += SUB * 16 * 4;
    }
  };

  // slots 0, 1, 2 hold halves h, h+1, h+2 at the top of an iteration
  int h = 0;
#pragma unroll 1
  for (; h + 4 <= halves; h += 4) {
    load(I3{});
    compute(I0{});
    if (h + 4 < halves) load(I0{});
    compute(I1{});
    if (h + 5 < halves) load(I1{});
    compute(I2{});
    if (h + 6 < halves) load(I2{});
    compute(I3{});
  }
  if (h < halves) {
    compute(I0{});
    compute(I1{});
  }

  // ------------------------------------------------------------------ reduction
  // this thread holds channel 32w + 16t + 8h + r, tokens 8nt + 2c + {0,1}
  if (kwi > 0) {
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int ch = 32 * w + 16 * t + 8 * (v >> 1) + r, token = 8 * nt + 2 * c + (v & 1);
          cl_sts32f(redl_s + (((kwi - 1) * MP + token) * kRedStride + ch) * 4, acc[t][nt][v]);
        }
  }
  __syncthreads();
  if (kwi == 0) {
    for (int q = 0; q + 1 < p.kw; ++q) {
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int ch = 32 * w + 16 * t + 8 * (v >> 1) + r, token = 8 * nt + 2 * c + (v & 1);
            acc[t][nt][v] += cl_lds32f(redl_s + ((q * MP + token) * kRedStride + ch) * 4);
          }
    }
  }
  if (S > 1) cluster_wait_acquire();      // phase 0 complete: every CTA of the cluster is running
  if (kwi == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int token = 8 * nt + 2 * c + e;
        if (token < p.m) {
          const uint32_t dest = (uint32_t)token % S, li = (uint32_t)token / S;
          const uint32_t local = redc_s + ((rank * p.own_max + li) * kRedStride) * 4;
          const uint32_t remote = S > 1 ? cluster_map(local, dest) : local;
#pragma unroll
          for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int ch = 32 * w + 16 * t + 8 * h + r;
              if (S > 1) st_cluster_f32(remote + ch * 4, acc[t][nt][h * 2 + e]);
              else cl_sts32f(remote + ch * 4, acc[t][nt][h * 2 + e]);
            }
        }
      }
  }
  if (S > 1) {
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    __syncthreads();
  }
  // this CTA finishes tokens rank, rank + S, ...
  if (p.glu) {
    // SwiGLU of a horizontally fused gate/up layer whose rows were interleaved per tile: channel ch < 64 of the tile is
    // gate row 64 tile + ch, channel 64 + ch its up row.  Both sums are rounded to T first, as the unfused form stores
    // them, and gated with the arithmetic of swiglu_kernel: the result has the same bits as linear -> swiglu.
    const int own = p.m > (int)rank ? (p.m - (int)rank + (int)S - 1) / (int)S : 0;
    const int half_n = p.n >> 1;
    for (int idx = tid; idx < own * (kTileRows / 2); idx += nthreads) {
      const int li = idx >> 6, ch = idx & 63;
      const int token = li * (int)S + (int)rank;
      float g = 0.f, u = 0.f;
      for (uint32_t src = 0; src < S; ++src) {
        const uint32_t a = redc_s + ((src * p.own_max + li) * kRedStride + ch) * 4;
        g += cl_lds32f(a);
        u += cl_lds32f(a + 64 * 4);
      }
      if (p.bias != nullptr) {
        g += p.bias[tile * kTileRows + ch];
        u += p.bias[tile * kTileRows + 64 + ch];
      }
      const float gx = to_float<T>(from_float<T>(g)), ux = to_float<T>(from_float<T>(u));
      reinterpret_cast<T*>(p.out)[(size_t)token * half_n + tile * (kTileRows / 2) + ch] = from_float<T>(gx / (1.0f + expf(-gx)) * ux);
    }
  } else {
    const int own = p.m > (int)rank ? (p.m - (int)rank + (int)S - 1) / (int)S : 0;
    unsigned char* out_base = reinterpret_cast<unsigned char*>(p.out);
    if (p.out_select != nullptr && ((*reinterpret_cast<const volatile unsigned int*>(p.out_select) + 1u) & 1u)) out_base += p.out_select_stride;
    for (int idx = tid; idx < own * kTileRows; idx += nthreads) {
      const int li = idx >> 7, ch = idx & 127;
      const int token = li * (int)S + (int)rank;
      const int chn = tile * kTileRows + ch;
      float sum = 0.f;
      for (uint32_t src = 0; src < S; ++src) sum += cl_lds32f(redc_s + ((src * p.own_max + li) * kRedStride + ch) * 4);
      if (chn < p.n) {
        if (p.bias != nullptr) sum += p.bias[chn];
        const size_t o = (size_t)token * p.n + chn;
        if (p.residual != nullptr) {
          if (p.round_first) sum = to_float<T>(from_float<T>(sum));
          sum += to_float<T>(reinterpret_cast<const T*>(p.residual)[o]);     // may alias out: read before the store below
        }
        if (p.out_f32) reinterpret_cast<float*>(out_base)[o] = sum;
        else reinterpret_cast<T*>(out_base)[o] = from_float<T>(sum);
      }
    }
  }
}

// --------------------------------------------------------------------------------------- host side

namespace {

struct ClPlan {
  int kw, s;
};

int cl_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev] = v;
  }
  return cached[dev];
}

// A plan forced through w4a16_decode_cl_set_plan (tuning runs); kw == 0 means automatic.
int g_forced_kw = 0, g_forced_s = 0;

bool cl_plan_override(ClPlan& plan) {
  if (g_forced_kw <= 0 || g_forced_s <= 0) return false;
  plan.kw = g_forced_kw;
  plan.s = g_forced_s;
  return true;
}

// How many K pieces a tile is cut into.  Measured on B200: the launch must fit one wave (16 warps
// per SM at 128 registers), power-of-two clusters place better than odd ones, and 8-warp CTAs (two K
// pieces per CTA, two CTAs per SM) beat both smaller and larger ones.  So: the largest power of two
// P with tiles * 4 * P warps inside one wave and at least two 128-K blocks per piece, cut as
// 2 x P/2 (1 x 1 when P is 1, 4 x 8 when P is 32).
ClPlan cl_plan(int tiles, int kblocks, int m) {
  using namespace dcl;
  ClPlan plan;
  const int max_slice = m > 8 ? kMaxSliceBlocks16 : kMaxSliceBlocks8;
  if (!cl_plan_override(plan)) {
    const int wave_warps = cl_sm_count() * 16;
    int pieces = 1;
    while (pieces < kMaxKW * kMaxCluster && (long long)tiles * 4 * (pieces * 2) <= wave_warps && pieces * 2 * 2 <= kblocks)
      pieces *= 2;
    plan.kw = pieces == 1 ? 1 : 2;
    plan.s = pieces / plan.kw;
    // a CTA's K slice (kblocks / s) must fit its shared memory: trade warp quads for CTAs
    while ((kblocks + plan.s - 1) / plan.s + 1 > max_slice + 1 && plan.s < kMaxCluster) {
      plan.s *= 2;
      if (plan.kw > 1) plan.kw /= 2;
    }
  }
  if (plan.kw < 1) plan.kw = 1;
  if (plan.kw > kMaxKW) plan.kw = kMaxKW;
  if (plan.s < 1) plan.s = 1;
  if (plan.s > kMaxCluster) plan.s = kMaxCluster;
  while (plan.kw * plan.s > kblocks && plan.kw > 1) plan.kw >>= 1;
  while (plan.kw * plan.s > kblocks && plan.s > 1) --plan.s;
  while ((kblocks + plan.s - 1) / plan.s + 1 > max_slice + 1 && plan.s < kMaxCluster) ++plan.s;
  return plan;
}

}  // namespace

void w4a16_decode_cl_set_plan(int kw, int s) {
  g_forced_kw = kw;
  g_forced_s = s;
}

void w4a16_decode_cl_get_plan(int m, int n, int k, int* kw, int* s) {
  const ClPlan plan = cl_plan(ceil_div(n, dcl::kTileRows), k / dcl::kKB, m);
  *kw = plan.kw;
  *s = plan.s;
}

bool w4a16_decode_cl_supported(int m, int n, int k, int group_size) {
  using namespace dcl;
  if (!(m >= 1 && m <= 16 && n >= 1 && k >= kKB && k % kKB == 0 && (group_size == 64 || group_size == 128))) return false;
  const int max_slice = m > 8 ? kMaxSliceBlocks16 : kMaxSliceBlocks8;
  const int kblocks = k / kKB;
  return (kblocks + kMaxCluster - 1) / kMaxCluster + 1 <= max_slice + 1;
}

template <typename T, typename P, int GK, int NT>
static int dcl_launch(const DecodeClParams& p, int grid, int threads, int cluster, size_t smem_bytes, cudaStream_t stream) {
  auto kern = w4a16_decode_cl_kernel<T, P, GK, NT>;
  XQT_SMEM_OPT_IN(kern, 200 * 1024);
  static int pdl = -1;
  if (pdl < 0) {
    const char* v = getenv("XQT_B200_PDL");
    pdl = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl == 1) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  XQT_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return launch_status();
}

template <typename T, typename P>
static int dcl_dispatch(const DecodeClParams& p, int group_size, int nt, int grid, int threads, int cluster, size_t smem,
                        cudaStream_t stream) {
  if (group_size == 128) {
    return nt == 1 ? dcl_launch<T, P, 128, 1>(p, grid, threads, cluster, smem, stream)
                   : dcl_launch<T, P, 128, 2>(p, grid, threads, cluster, smem, stream);
  }
  return nt == 1 ? dcl_launch<T, P, 64, 1>(p, grid, threads, cluster, smem, stream)
                 : dcl_launch<T, P, 64, 2>(p, grid, threads, cluster, smem, stream);
}

int w4a16_decode_cl_launch(const void* x, const void* wt, const void* scl, const void* zer, const float* bias, const void* residual,
                           void* out, int m, int n, int k, int group_size, int nibble_signed, int act_dtype,
                           int param_dtype, int out_f32, int epilogue_flags, const unsigned int* out_select,
                           long long out_select_stride, unsigned int* status, cudaStream_t stream) {
  using namespace dcl;
  XQT_REQUIRE(w4a16_decode_cl_supported(m, n, k, group_size));
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)wt & 31) == 0 && ((uintptr_t)scl & 15) == 0 && ((uintptr_t)zer & 15) == 0);
  XQT_REQUIRE(!out_f32 || residual == nullptr);
  const int tiles = ceil_div(n, kTileRows), kblocks = k / kKB;
  const int nt = m > 8 ? 2 : 1, mp = 8 * nt, sub = kKB / group_size;
  const ClPlan plan = cl_plan(tiles, kblocks, m);
  DecodeClParams p;
  p.wt = (const uint8_t*)wt; p.scl = (const uint8_t*)scl; p.zer = (const uint8_t*)zer; p.x = x; p.bias = bias; p.residual = residual; p.out = out;
  p.status = status;
  p.m = m; p.n = n; p.k = k; p.out_f32 = out_f32;
  p.round_first = (epilogue_flags & 1) != 0;
  XQT_REQUIRE(!(p.round_first && out_f32));
  p.out_select = out_select; p.out_select_stride = out_select_stride;
  XQT_REQUIRE(out_select == nullptr || (out_select_stride % 16 == 0 && (epilogue_flags & 2) == 0));
  p.glu = (epilogue_flags & 2) != 0;
  XQT_REQUIRE(!p.glu || (n % kTileRows == 0 && !out_f32 && residual == nullptr));
  p.kblocks = kblocks; p.kw = plan.kw; p.pieces = plan.kw * plan.s;
  XQT_REQUIRE(p.pieces >= 1 && p.pieces <= kblocks);
  const int slice_max = (kblocks * plan.kw + p.pieces - 1) / p.pieces + 1;   // upper bound of any CTA's slice
  XQT_REQUIRE(slice_max <= (m > 8 ? kMaxSliceBlocks16 : kMaxSliceBlocks8) + 1);
  p.xrow_bytes = slice_max * 256 + kXPad;
  p.own_max = (mp + plan.s - 1) / plan.s;
  p.per = kblocks / p.pieces;
  p.rem = kblocks % p.pieces;
  int off = 384 + m * p.xrow_bytes;
  p.off_xsum = off; off += slice_max * sub * 16 * 4;
  p.off_redl = off; off += (plan.kw - 1) * mp * kRedStride * 4;
  p.off_redc = off; off += plan.s * p.own_max * kRedStride * 4;
  XQT_REQUIRE(off <= 200 * 1024);
  p.base_off = (act_dtype == XQT_B200_BF16 ? 128.f : 1024.f) + (nibble_signed ? 8.f : 0.f);
  {
    // XQT_B200_DECODE_PREFETCH=0 turns the start-of-kernel L2 prefetch off (A/B measurements)
    static int prefetch = -1;
    if (prefetch < 0) {
      const char* v = getenv("XQT_B200_DECODE_PREFETCH");
      prefetch = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    p.prefetch = prefetch;
  }
  const int grid = tiles * plan.s, threads = 128 * plan.kw;
  if (act_dtype == XQT_B200_BF16) {
    if (param_dtype == XQT_B200_BF16) return dcl_dispatch<__nv_bfloat16, __nv_bfloat16>(p, group_size, nt, grid, threads, plan.s, off, stream);
    if (param_dtype == XQT_B200_FP16) return dcl_dispatch<__nv_bfloat16, __half>(p, group_size, nt, grid, threads, plan.s, off, stream);
    return dcl_dispatch<__nv_bfloat16, float>(p, group_size, nt, grid, threads, plan.s, off, stream);
  }
  if (param_dtype == XQT_B200_BF16) return dcl_dispatch<__half, __nv_bfloat16>(p, group_size, nt, grid, threads, plan.s, off, stream);
  if (param_dtype == XQT_B200_FP16) return dcl_dispatch<__half, __half>(p, group_size, nt, grid, threads, plan.s, off, stream);
  return dcl_dispatch<__half, float>(p, group_size, nt, grid, threads, plan.s, off, stream);
}

}  // namespace xqt_b200

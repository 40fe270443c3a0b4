// W4A16 decode (M <= 16) on the tile-ordered execution layout: a persistent, TMA-fed, stream-K
// kernel that is meant to run at HBM speed.
//
// Why this shape.  A decode linear is a pure weight stream: 0.5 byte per weight, touched once.
// To keep 6.5 TB/s busy an SM must have ~40 KB in flight at all times, and at that rate it may
// spend fewer than three instructions per weight.  Hence:
//   * one CTA per SM, alive for the whole launch, with a ring of shared-memory stages that a
//     single producer warp fills with bulk async copies (cp.async.bulk + mbarrier tx counts): one
//     16 KiB copy for the weights of (128 channels x 256 K), one for their scales/zero points and
//     one 512-byte copy per activation row.  No thread ever waits on a global load;
//   * the work list is the sequence of all (tile, K-stage) pairs cut into gridDim equal runs
//     (stream-K), so every SM streams the same number of bytes whatever N and K are.  A tile that
//     spans two or more CTAs is finished by the last of them to arrive: partial sums go to a
//     scratch buffer, an atomic ticket picks the finisher (nobody spins), the finisher adds the
//     partials in CTA order (bit-reproducible) and re-arms the ticket;
//   * eight consumer warps turn nibbles into exact bf16/fp16 integers (one lop3 + one sub per
//     pair), feed mma.m16n8k16 with the 16 activation rows as the M side, and apply the group
//     scale and zero point to the fp32 sum of each quantisation group:
//        y += s * (sum_k x q  -  z * sum_k x)
//     so the weight is never rounded to 16 bits and the result equals the fp32 contract reference
//     (xqt/kernels/ops/gemm/reference.py:263-271,527) up to fp32 summation order.
// Every mbarrier wait is bounded; on expiry the kernel records a status word and drains.
#include "common.cuh"

namespace xqt_b200 {

namespace decode {
constexpr int kTileRows = 128;
constexpr int kKBlock = 128;
constexpr int kKS = 2;                      // K blocks per pipeline stage
constexpr int kStageK = kKS * kKBlock;      // 256
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kWBytes = kKS * 8192;         // 128 channels x 256 K x 4 bit
constexpr int kXRowBytes = kStageK * 2 + 64;  // +64: rows land on different banks for the LDS.128 pattern
constexpr int kXBytes = 16 * kXRowBytes;
constexpr int kRedBytes = 4 * 32 * 16 * 4;  // four n-groups x 32 lanes x 16 floats
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kPartialFloats = 16 * kTileRows;
constexpr int kMaxTiles = 8192;             // tickets at the head of the workspace
constexpr int kMaxGrid = 256;
constexpr uint32_t kSpinLimit = 1u << 22;

enum Status : unsigned int { kOk = 0, kProducerTimeout = 1, kConsumerTimeout = 2 };
}  // namespace decode

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait: false when the limit ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < decode::kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

template <typename T>
struct DecTraits;
template <>
struct DecTraits<__half> {
  using h2 = __half2;
  static constexpr uint32_t kMagic = 0x64006400u, kOffU = 0x64006400u, kOffS = 0x64086408u, kOne = 0x3C003C00u;
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <>
struct DecTraits<__nv_bfloat16> {
  using h2 = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u, kOffU = 0x43004300u, kOffS = 0x43084308u, kOne = 0x3F803F80u;
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// nibble positions i and i+4 of `word` (adjacent K in the tiled layout) -> exact pair of T integers
template <typename T, bool SIGNED>
__device__ __forceinline__ uint32_t dq_pair(uint32_t word, int i) {
  using Tr = DecTraits<T>;
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(word >> (4 * i)), "n"(0x000f000f), "r"(Tr::kMagic));
  typename Tr::h2 v = *reinterpret_cast<typename Tr::h2*>(&r);
  const uint32_t ob = SIGNED ? Tr::kOffS : Tr::kOffU;
  v = __hsub2(v, *reinterpret_cast<const typename Tr::h2*>(&ob));
  return *reinterpret_cast<uint32_t*>(&v);
}

struct DecodeParams {
  const void* x;
  const uint8_t* wt;
  const uint8_t* sz;
  const float* bias;
  const void* residual;
  void* out;
  int m, n, k;
  int tiles, spt;            // stages per tile = k / 256
  long long total;           // tiles * spt
  int nstages, stage_bytes, sz_stage_bytes;
  float* partials;           // [grid][2][16*128]
  unsigned int* tickets;     // [tiles]
  unsigned int* status;
};

// cta that owns global stage index x when `total` stages are cut into `grid` equal runs
__device__ __forceinline__ int cta_of(long long x, long long total, int grid) {
  return (int)(((x + 1) * grid - 1) / total);
}

template <typename T, typename P, bool SIGNED, bool HAS_ZP, int GP>
__global__ void __launch_bounds__(decode::kThreads, 1) w4a16_decode_kernel(const DecodeParams p) {
  using namespace decode;
  using Tr = DecTraits<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages];
  __shared__ unsigned int s_flag;
  __shared__ volatile unsigned int s_abort;  // set by the first wait that ran out; later waits are skipped

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long s_begin = (long long)cta * p.total / grid, s_end = (long long)(cta + 1) * p.total / grid;
  const int ns = p.nstages;
  unsigned char* red = smem + (size_t)ns * p.stage_bytes;

  if (tid == 0) {
    s_abort = 0u;
    for (int i = 0; i < ns; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);                          // full: one expect_tx arrival
      mbar_init(smem_u32(&bars[kMaxStages + i]), kConsumerWarps);  // empty: one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // activation rows >= m are never copied: they must read as zero
  for (int i = tid; i < ns * (kXBytes / 16); i += kThreads) {
    const int st = i / (kXBytes / 16), o = i % (kXBytes / 16);
    reinterpret_cast<uint4*>(smem + (size_t)st * p.stage_bytes + kWBytes)[o] = make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ producer warp
    const uint32_t tx = kWBytes + p.sz_stage_bytes + p.m * (kStageK * 2);
    uint32_t it = 0;
    bool alive = true;
    for (long long s = s_begin; s < s_end && alive; ++s, ++it) {
      const int slot = it % ns;
      const uint32_t full = smem_u32(&bars[slot]), empty = smem_u32(&bars[kMaxStages + slot]);
      if (lane == 0) alive = (s_abort == 0u) && mbar_wait(empty, ((it / ns) & 1) ^ 1);
      alive = __shfl_sync(0xffffffffu, alive, 0);
      if (!alive) break;
      const long long tile = s / p.spt;
      const int ks = (int)(s % p.spt);
      unsigned char* st = smem + (size_t)slot * p.stage_bytes;
      const long long unit = tile * (long long)(p.k / kKBlock) + (long long)ks * kKS;  // first (tile, kblock) unit
      if (lane == 0) {
        mbar_expect_tx(full, tx);
        bulk_g2s(smem_u32(st), p.wt + unit * 8192, kWBytes, full);
      } else if (lane == 1) {
        bulk_g2s(smem_u32(st + kWBytes + kXBytes), p.sz + unit * (p.sz_stage_bytes / kKS), p.sz_stage_bytes, full);
      } else if (lane - 2 < p.m) {
        const int r = lane - 2;
        bulk_g2s(smem_u32(st + kWBytes + r * kXRowBytes),
                 reinterpret_cast<const T*>(p.x) + (size_t)r * p.k + (size_t)ks * kStageK, kStageK * 2, full);
      }
      __syncwarp();
    }
    if (!alive && lane == 0) {
      if (s_abort == 0u) atomicExch(p.status, (unsigned int)kProducerTimeout);
      s_abort = 1u;
    }
    // the copies still in flight target this CTA's shared memory: see them land before leaving
    if (lane == 0) {
      const uint32_t issued = it;
      const uint32_t first = issued > (uint32_t)ns ? issued - ns : 0;
      for (uint32_t j = first; j < issued; ++j) (void)mbar_wait(smem_u32(&bars[j % ns]), (j / ns) & 1);
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int g = lane >> 2, t = lane & 3;
  const int kb = warp % kKS;   // K block of the stage this warp multiplies
  const int ng = warp / kKS;   // its four n-tiles: channels 32*ng .. 32*ng+31 of the tile
  constexpr int WPS = 4 / GP;  // 32-K words per quantisation group
  const bool hi_rows = p.m > 8;

  float acc[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  uint32_t it = 0;
  for (long long s = s_begin; s < s_end; ++s, ++it) {
    const int slot = it % ns;
    const long long tile = s / p.spt;
    const int ks = (int)(s % p.spt);
    unsigned char* st = smem + (size_t)slot * p.stage_bytes;
    // A wait that runs out marks the launch as failed and stops waiting; the warp still walks the
    // same control flow as the others (their named barriers count it), the output is then garbage
    // and the status word says so.
    if (s_abort == 0u && !mbar_wait(smem_u32(&bars[slot]), (it / ns) & 1)) {
      s_abort = 1u;
      if (lane == 0) atomicExch(p.status, (unsigned int)kConsumerTimeout);
    }
    // A fragments: rows g and g+8, word w covers k = 128*kb + 32*w + 8*t .. +7
    uint4 alo[4], ahi[4];
    const unsigned char* xs = st + kWBytes + (kb * kKBlock + 8 * t) * 2;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      alo[w] = *reinterpret_cast<const uint4*>(xs + g * kXRowBytes + w * 64);
      ahi[w] = hi_rows ? *reinterpret_cast<const uint4*>(xs + (g + 8) * kXRowBytes + w * 64) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 wv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      wv[j] = *reinterpret_cast<const uint4*>(st + ((kb * 16 + ng * 4 + j) * 32 + lane) * 16);
    const P* szs = reinterpret_cast<const P*>(st + kWBytes + kXBytes) + (size_t)kb * GP * kTileRows * 2;

#pragma unroll
    for (int u = 0; u < GP; ++u) {
      float xs_sum[4] = {0.f, 0.f, 0.f, 0.f};
      float grp[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) grp[j][0] = grp[j][1] = grp[j][2] = grp[j][3] = 0.f;
#pragma unroll
      for (int ww = 0; ww < WPS; ++ww) {
        const int w = u * WPS + ww;
        if (HAS_ZP) {
          Tr::mma(xs_sum, alo[w].x, ahi[w].x, alo[w].y, ahi[w].y, Tr::kOne, Tr::kOne);
          Tr::mma(xs_sum, alo[w].z, ahi[w].z, alo[w].w, ahi[w].w, Tr::kOne, Tr::kOne);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t word = w == 0 ? wv[j].x : (w == 1 ? wv[j].y : (w == 2 ? wv[j].z : wv[j].w));
          if (SIGNED) word ^= 0x88888888u;
          const uint32_t b0 = dq_pair<T, SIGNED>(word, 0), b1 = dq_pair<T, SIGNED>(word, 1);
          const uint32_t b2 = dq_pair<T, SIGNED>(word, 2), b3 = dq_pair<T, SIGNED>(word, 3);
          Tr::mma(grp[j], alo[w].x, ahi[w].x, alo[w].y, ahi[w].y, b0, b1);
          Tr::mma(grp[j], alo[w].z, ahi[w].z, alo[w].w, ahi[w].w, b2, b3);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // (scale, zero) of channels 2t and 2t+1 of n-tile j for this group
        const P* q = szs + ((size_t)u * kTileRows + ng * 32 + j * 8 + 2 * t) * 2;
        const float s0 = to_float<P>(q[0]), z0 = to_float<P>(q[1]), s1 = to_float<P>(q[2]), z1 = to_float<P>(q[3]);
        if (HAS_ZP) {
          acc[j][0] = fmaf(s0, fmaf(-z0, xs_sum[0], grp[j][0]), acc[j][0]);
          acc[j][1] = fmaf(s1, fmaf(-z1, xs_sum[0], grp[j][1]), acc[j][1]);
          acc[j][2] = fmaf(s0, fmaf(-z0, xs_sum[2], grp[j][2]), acc[j][2]);
          acc[j][3] = fmaf(s1, fmaf(-z1, xs_sum[2], grp[j][3]), acc[j][3]);
        } else {
          acc[j][0] = fmaf(s0, grp[j][0], acc[j][0]);
          acc[j][1] = fmaf(s1, grp[j][1], acc[j][1]);
          acc[j][2] = fmaf(s0, grp[j][2], acc[j][2]);
          acc[j][3] = fmaf(s1, grp[j][3], acc[j][3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars[kMaxStages + slot]));

    if (ks != p.spt - 1 && s != s_end - 1) continue;

    // ---------------------------------------------------------------- end of this CTA's run in `tile`
    // 1. add the two K-block warps of each n-group (warp kb==1 hands over through shared memory)
    float* rbuf = reinterpret_cast<float*>(red) + (ng * 32 + lane) * 16;
    if (kb == 1) {
#pragma unroll
      for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(rbuf + 4 * j) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    }
    consumer_sync();
    if (kb == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(rbuf + 4 * j);
        acc[j][0] += v.x; acc[j][1] += v.y; acc[j][2] += v.z; acc[j][3] += v.w;
      }
    }
    // 2. who else works on this tile?
    const long long t_first = tile * p.spt, t_last = t_first + p.spt - 1;
    const int c_first = cta_of(t_first, p.total, grid), c_last = cta_of(t_last, p.total, grid);
    bool finish = true;
    if (c_first != c_last) {
      const int seg = (s_begin / p.spt == tile) ? 0 : 1;
      float* slot_out = p.partials + ((size_t)cta * 2 + seg) * kPartialFloats + (ng * 32 + lane) * 16;
      if (kb == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(slot_out + 4 * j) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        __threadfence();
      }
      consumer_sync();
      if (tid == 0) s_flag = atomicAdd(&p.tickets[tile], 1u);
      consumer_sync();
      finish = (s_flag == (unsigned int)(c_last - c_first));
      if (finish) {
        __threadfence();
        if (kb == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {
            const int cseg = (((long long)c * p.total / grid) / p.spt == tile) ? 0 : 1;
            const float* src = p.partials + ((size_t)c * 2 + cseg) * kPartialFloats + (ng * 32 + lane) * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 v = __ldcg(reinterpret_cast<const float4*>(src + 4 * j));
              acc[j][0] += v.x; acc[j][1] += v.y; acc[j][2] += v.z; acc[j][3] += v.w;
            }
          }
        }
        if (tid == 0) p.tickets[tile] = 0u;  // re-arm for the next launch
      }
    }
    // 3. bias, residual, cast, store (C fragment: rows g / g+8, channels 2t / 2t+1 of each n-tile)
    if (finish && kb == 0) {
      T* out = reinterpret_cast<T*>(p.out);
      const T* res = reinterpret_cast<const T*>(p.residual);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = g + (e >> 1) * 8;
          const long long ch = tile * kTileRows + ng * 32 + j * 8 + 2 * t + (e & 1);
          if (row < p.m && ch < p.n) {
            float v = acc[j][e];
            if (p.bias != nullptr) v += p.bias[ch];
            const size_t o = (size_t)row * p.n + ch;
            if (res != nullptr) v += to_float<T>(res[o]);
            out[o] = from_float<T>(v);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  }
}

// --------------------------------------------------------------------------------------- host side

static int decode_sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  return v;
}

size_t w4a16_decode_workspace_bytes() {
  using namespace decode;
  return 256 + (size_t)kMaxTiles * sizeof(unsigned int) + (size_t)kMaxGrid * 2 * kPartialFloats * sizeof(float);
}

bool w4a16_decode_supported(int m, int n, int k, int group_size) {
  using namespace decode;
  return m >= 1 && m <= 16 && n >= 1 && k >= kStageK && k % kStageK == 0 &&
         (group_size == 32 || group_size == 64 || group_size == 128) && ceil_div(n, kTileRows) <= kMaxTiles;
}

template <typename T, typename P, bool SIGNED, bool HAS_ZP>
static int decode_launch_gp(const DecodeParams& p, int gp, int grid, size_t smem_bytes, cudaStream_t stream) {
#define XQT_DEC_LAUNCH(GPV)                                                                              \
  do {                                                                                                   \
    auto kern = w4a16_decode_kernel<T, P, SIGNED, HAS_ZP, GPV>;                                          \
    XQT_SMEM_OPT_IN(kern, decode::kSmemBudget);                                                          \
    kern<<<grid, decode::kThreads, smem_bytes, stream>>>(p);                                             \
  } while (0)
  if (gp == 1) XQT_DEC_LAUNCH(1);
  else if (gp == 2) XQT_DEC_LAUNCH(2);
  else XQT_DEC_LAUNCH(4);
#undef XQT_DEC_LAUNCH
  return launch_status();
}

template <typename T, typename P>
static int decode_launch_tp(const DecodeParams& p, int gp, int grid, size_t smem_bytes, bool is_signed, bool zp,
                            cudaStream_t stream) {
  if (is_signed) {
    if (zp) return decode_launch_gp<T, P, true, true>(p, gp, grid, smem_bytes, stream);
    return decode_launch_gp<T, P, true, false>(p, gp, grid, smem_bytes, stream);
  }
  if (zp) return decode_launch_gp<T, P, false, true>(p, gp, grid, smem_bytes, stream);
  return decode_launch_gp<T, P, false, false>(p, gp, grid, smem_bytes, stream);
}

int w4a16_decode_launch(const void* x, const void* wt, const void* sz, const float* bias, const void* residual,
                        void* out, int m, int n, int k, int group_size, int nibble_signed, int has_zp, int act_dtype,
                        int param_dtype, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  using namespace decode;
  XQT_REQUIRE(w4a16_decode_supported(m, n, k, group_size));
  XQT_REQUIRE(workspace != nullptr && workspace_bytes >= w4a16_decode_workspace_bytes());
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)wt & 15) == 0 && ((uintptr_t)sz & 15) == 0);
  const int gp = kKBlock / group_size;
  const int psize = param_dtype == XQT_B200_FP32 ? 4 : 2;
  DecodeParams p;
  p.x = x; p.wt = (const uint8_t*)wt; p.sz = (const uint8_t*)sz; p.bias = bias; p.residual = residual; p.out = out;
  p.m = m; p.n = n; p.k = k;
  p.tiles = ceil_div(n, kTileRows);
  p.spt = k / kStageK;
  p.total = (long long)p.tiles * p.spt;
  p.sz_stage_bytes = kKS * gp * kTileRows * 2 * psize;
  p.stage_bytes = (kWBytes + kXBytes + p.sz_stage_bytes + 127) / 128 * 128;
  int ns = (kSmemBudget - kRedBytes) / p.stage_bytes;
  p.nstages = ns > kMaxStages ? kMaxStages : ns;
  XQT_REQUIRE(p.nstages >= 2);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<unsigned int*>(ws);
  p.tickets = reinterpret_cast<unsigned int*>(ws + 256);
  p.partials = reinterpret_cast<float*>(ws + 256 + (size_t)kMaxTiles * sizeof(unsigned int));
  long long grid = decode_sm_count();
  if (grid > kMaxGrid) grid = kMaxGrid;
  if (grid > p.total) grid = p.total;
  const size_t smem_bytes = (size_t)p.nstages * p.stage_bytes + kRedBytes;
  const bool sg = nibble_signed != 0, zp = has_zp != 0;
  if (act_dtype == XQT_B200_BF16) {
    if (param_dtype == XQT_B200_BF16) return decode_launch_tp<__nv_bfloat16, __nv_bfloat16>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
    if (param_dtype == XQT_B200_FP16) return decode_launch_tp<__nv_bfloat16, __half>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
    return decode_launch_tp<__nv_bfloat16, float>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  }
  if (param_dtype == XQT_B200_BF16) return decode_launch_tp<__half, __nv_bfloat16>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  if (param_dtype == XQT_B200_FP16) return decode_launch_tp<__half, __half>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  return decode_launch_tp<__half, float>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
}

// ------------------------------------------------------------------------- allocation-free variant
//
// Scratch for callers that cannot allocate device memory (see xqt_b200_w4a16_decode_tiled_static in
// include/xqt_b200.h).  The array lives in the library image: every GPU that loads the library holds
// these bytes until the process exits.  Layout: status word @0, tickets @256, partials after them.
namespace decode_static {
constexpr int kMaxTiles = 1024;   // N <= 131072 output channels
constexpr int kMaxGrid = 160;     // CTAs (a B200 has 148 SMs)
constexpr size_t kTicketBytes = (size_t)kMaxTiles * sizeof(unsigned int);
constexpr size_t kBytes = 256 + kTicketBytes + (size_t)kMaxGrid * 2 * decode::kPartialFloats * sizeof(float);
}  // namespace decode_static

static __device__ __align__(256) unsigned char g_decode_static_scratch[decode_static::kBytes];

// In host code the array's name is only a stand-in for the symbol, not a device address: the
// address is asked for once per device, with that device current, and cached.
static int decode_static_scratch(unsigned char** out) {
  static unsigned char* cache[64] = {nullptr};
  int dev = 0;
  XQT_CUDA(cudaGetDevice(&dev));
  XQT_REQUIRE(dev >= 0 && dev < 64);
  if (cache[dev] == nullptr) {
    void* ptr = nullptr;
    XQT_CUDA(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
    cache[dev] = reinterpret_cast<unsigned char*>(ptr);
  }
  *out = cache[dev];
  return 0;
}

size_t w4a16_decode_static_scratch_bytes() { return decode_static::kBytes; }

// status word of the built-in scratch of the current device (the last call's: every call clears it)
int w4a16_decode_static_status(unsigned int* host_status, cudaStream_t stream) {
  unsigned char* ws = nullptr;
  {
    const int rc = decode_static_scratch(&ws);
    if (rc != 0) return rc;
  }
  XQT_CUDA(cudaMemcpyAsync(host_status, ws, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
  XQT_CUDA(cudaStreamSynchronize(stream));
  return 0;
}
int w4a16_decode_static_max_n() { return decode_static::kMaxTiles * decode::kTileRows; }

int w4a16_decode_launch_static(const void* x, const void* wt, const void* sz, const float* bias, const void* residual,
                               void* out, int m, int n, int k, int group_size, int nibble_signed, int has_zp,
                               int act_dtype, int param_dtype, cudaStream_t stream) {
  using namespace decode;
  XQT_REQUIRE(w4a16_decode_supported(m, n, k, group_size));
  XQT_REQUIRE(ceil_div(n, kTileRows) <= decode_static::kMaxTiles);   // beyond the scratch built into the library
  XQT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)wt & 15) == 0 && ((uintptr_t)sz & 15) == 0);
  unsigned char* ws = nullptr;
  {
    const int rc = decode_static_scratch(&ws);
    if (rc != 0) return rc;
  }
  const int gp = kKBlock / group_size;
  const int psize = param_dtype == XQT_B200_FP32 ? 4 : 2;
  DecodeParams p;
  p.x = x; p.wt = (const uint8_t*)wt; p.sz = (const uint8_t*)sz; p.bias = bias; p.residual = residual; p.out = out;
  p.m = m; p.n = n; p.k = k;
  p.tiles = ceil_div(n, kTileRows);
  p.spt = k / kStageK;
  p.total = (long long)p.tiles * p.spt;
  p.sz_stage_bytes = kKS * gp * kTileRows * 2 * psize;
  p.stage_bytes = (kWBytes + kXBytes + p.sz_stage_bytes + 127) / 128 * 128;
  int ns = (kSmemBudget - kRedBytes) / p.stage_bytes;
  p.nstages = ns > kMaxStages ? kMaxStages : ns;
  XQT_REQUIRE(p.nstages >= 2);
  p.status = reinterpret_cast<unsigned int*>(ws);
  p.tickets = reinterpret_cast<unsigned int*>(ws + 256);
  p.partials = reinterpret_cast<float*>(ws + 256 + decode_static::kTicketBytes);
  // Every call shares the array and finds what the last one left: the tickets and the status word
  // must start at zero (a memset on the stream allocates nothing); partials are overwritten before use.
  XQT_CUDA(cudaMemsetAsync(ws, 0, 256 + (size_t)p.tiles * sizeof(unsigned int), stream));
  long long grid = decode_sm_count();
  if (grid > decode_static::kMaxGrid) grid = decode_static::kMaxGrid;
  if (grid > p.total) grid = p.total;
  const size_t smem_bytes = (size_t)p.nstages * p.stage_bytes + kRedBytes;
  const bool sg = nibble_signed != 0, zp = has_zp != 0;
  if (act_dtype == XQT_B200_BF16) {
    if (param_dtype == XQT_B200_BF16) return decode_launch_tp<__nv_bfloat16, __nv_bfloat16>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
    if (param_dtype == XQT_B200_FP16) return decode_launch_tp<__nv_bfloat16, __half>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
    return decode_launch_tp<__nv_bfloat16, float>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  }
  if (param_dtype == XQT_B200_BF16) return decode_launch_tp<__half, __nv_bfloat16>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  if (param_dtype == XQT_B200_FP16) return decode_launch_tp<__half, __half>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
  return decode_launch_tp<__half, float>(p, gp, (int)grid, smem_bytes, sg, zp, stream);
}

}  // namespace xqt_b200

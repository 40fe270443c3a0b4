// One-shot all-reduce over NVLink peer memory with the linear's epilogue fused in: the reduction step
// of a row-parallel (K-sharded) quantized linear at decode sizes.
//
// Every rank's GEMV writes its fp32 partial [count] into its own slot of a buffer that all ranks of
// the node have mapped (symmetric memory: plain peer pointers).  This kernel, launched
// by every rank on its own GPU, (1) tells every peer that this rank's partial is complete and waits
// until every peer has said the same, (2) reads the `world` partials straight from their owners'
// memory, adds them in rank order -- the same order on every rank, so all ranks produce identical
// bits -- adds the bias, rounds once and writes the rank's own full output.  For a few hundred KiB
// this is one NVLink round trip instead of the launch and protocol latency of a library all-reduce.
//
// Hand-shake: flags[r] on rank q holds the last call number in which rank r signalled q.  Call
// numbers only grow; partial buffers are used alternately (call e uses slot e & 1), so a rank can
// only overwrite a slot two calls later, after every peer has signalled the call in between, which
// a peer does only after its own kernel of the earlier call has finished reading.  No exit barrier
// is needed.  The wait is bounded: after `spin_limit` polls (kSpin when the caller passes 0) the kernel
// records kTimeout in the status word -- which may live in pinned host memory, so that the host sees
// it without a synchronisation -- skips the wait and finishes through its normal path; the output is
// then not the sum and the caller must treat the call as failed.
//
// Counted form (graph-safe): the call number lives in device memory instead of a launch argument.  `counter[0]` holds
// the number of finished calls; every block reads it on entry, works as call counter[0] + 1 on slot (call & 1) of the
// two-slot partial buffers, and the block that finishes last (ticket in counter[1]) publishes the new count.  The
// kernel that wrote the partial picked its slot from the same word (the decode kernel's out_select), so a captured
// graph replays correctly: nothing in the launch arguments changes from call to call.
#include "common.cuh"

namespace xqt_b200 {

namespace par {
constexpr int kMaxWorld = 8;
constexpr unsigned int kSpin = 1u << 22;
enum Status : unsigned int { kTimeout = 128 };
}  // namespace par

struct PeerReduceParams {
  const float* partial[par::kMaxWorld];   // rank r's partial for this call (peer pointers)
  unsigned int* flags[par::kMaxWorld];    // rank r's flag array [kMaxWorld] (peer pointers)
  int rank, world;
  unsigned int call;                      // this call's number (> 0, same on every rank)
  long long count;                        // elements, a multiple of 4
  int n;                                  // row length (bias period)
  const float* bias;                      // [n] or null
  void* out;                              // [count] in T
  unsigned int* status;
  unsigned int spin_limit;                // polls before the wait for a peer gives up
  unsigned int* counter;                  // counted form: [0] finished calls, [1] block tickets; null otherwise
  long long slot_stride;                  // counted form: elements between the two slots of every partial buffer
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) peer_allreduce_kernel(const PeerReduceParams p) {
  using namespace par;
  unsigned int call = p.call;
  long long slot_off = 0;
  if (p.counter != nullptr) {
    call = *reinterpret_cast<volatile unsigned int*>(p.counter) + 1u;
    slot_off = (call & 1u) ? p.slot_stride : 0;
  }
  // (1) signal and wait.  Block 0 signals (the partial was written by the kernel before this one on
  // the same stream, so it is complete); every block waits on this rank's own flag array.
  if (blockIdx.x == 0 && threadIdx.x < p.world && (int)threadIdx.x != p.rank)
    st_release_sys(p.flags[threadIdx.x] + p.rank, call);
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    const unsigned int* f = p.flags[p.rank] + threadIdx.x;
    unsigned int spins = 0;
    // call numbers only grow: "signalled this call or a later one"
    while ((int)(ld_acquire_sys(f) - call) < 0) {
      if (++spins >= p.spin_limit) {
        st_release_sys(p.status, (unsigned int)kTimeout);   // device or pinned host memory
        break;
      }
    }
  }
  __syncthreads();
  // (2) reduce in rank order, epilogue, store
  const long long vecs = p.count / 4;
  T* out = reinterpret_cast<T*>(p.out);
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < vecs; v += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 part[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < p.world) part[r] = __ldcg(reinterpret_cast<const float4*>(p.partial[r] + slot_off) + v);   // all loads in flight
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < p.world) {
        acc.x += part[r].x; acc.y += part[r].y; acc.z += part[r].z; acc.w += part[r].w;
      }
    if (p.bias != nullptr) {
      const int col = (int)((v * 4) % p.n);   // n is a multiple of 4: the four elements share a row
      const float4 b = *reinterpret_cast<const float4*>(p.bias + col);
      acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    T o[4] = {from_float<T>(acc.x), from_float<T>(acc.y), from_float<T>(acc.z), from_float<T>(acc.w)};
    *reinterpret_cast<uint2*>(out + v * 4) = *reinterpret_cast<const uint2*>(o);
  }
  if (p.counter != nullptr) {
    // every block has read counter[0] before it takes its ticket; the last one publishes the finished call
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.counter + 1, 1u) == gridDim.x - 1) {
        p.counter[1] = 0u;
        __threadfence();
        *reinterpret_cast<volatile unsigned int*>(p.counter) = call;
      }
    }
  }
}

// counter == nullptr: `call` is this call's number and partials[r] the slot in use; else the counted form: partials[r]
// is slot 0 of rank r's two-slot buffer, the slots slot_stride elements apart, and `call` is ignored
// All-gather over peer memory, counted form only: after the same hand-shake every rank copies slot (call & 1) of every
// rank's buffer (its own included) into out[r * vecs ...] with 16-byte peer loads.  The concatenation step of
// column-parallel layers whose outputs the ranks wrote into their own two-slot buffers (decode kernels with out_select).
struct PeerGatherParams {
  const uint4* source[par::kMaxWorld];    // slot 0 of rank r's buffer (peer pointers)
  unsigned int* flags[par::kMaxWorld];
  int rank, world;
  long long vecs;                         // 16-byte pieces per rank
  long long slot_stride;                  // 16-byte pieces between the two slots
  uint4* out;                             // [world][vecs]
  unsigned int* status;
  unsigned int spin_limit;
  unsigned int* counter;                  // [0] finished calls, [1] block tickets
};

__global__ void __launch_bounds__(256) peer_allgather_kernel(const PeerGatherParams p) {
  using namespace par;
  const unsigned int call = *reinterpret_cast<volatile unsigned int*>(p.counter) + 1u;
  const long long slot_off = (call & 1u) ? p.slot_stride : 0;
  if (blockIdx.x == 0 && threadIdx.x < p.world && (int)threadIdx.x != p.rank)
    st_release_sys(p.flags[threadIdx.x] + p.rank, call);
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    const unsigned int* f = p.flags[p.rank] + threadIdx.x;
    unsigned int spins = 0;
    while ((int)(ld_acquire_sys(f) - call) < 0) {
      if (++spins >= p.spin_limit) {
        st_release_sys(p.status, (unsigned int)kTimeout);
        break;
      }
    }
  }
  __syncthreads();
  const long long total = p.vecs * p.world;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / p.vecs);
    const long long v = i - (long long)r * p.vecs;
    p.out[i] = __ldcg(p.source[r] + slot_off + v);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.counter + 1, 1u) == gridDim.x - 1) {
      p.counter[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(p.counter) = call;
    }
  }
}

int peer_allgather_launch(const void* const* sources, void* const* flags, int rank, int world, unsigned int* counter,
                          long long slot_stride_bytes, long long bytes, void* out, unsigned int spin_limit,
                          unsigned int* status, cudaStream_t stream) {
  using namespace par;
  XQT_REQUIRE(world >= 2 && world <= kMaxWorld && rank >= 0 && rank < world && counter != nullptr);
  XQT_REQUIRE(bytes > 0 && bytes % 16 == 0 && slot_stride_bytes >= bytes && slot_stride_bytes % 16 == 0);
  XQT_REQUIRE(sources != nullptr && flags != nullptr && out != nullptr && status != nullptr && ((uintptr_t)out & 15) == 0);
  PeerGatherParams p{};
  for (int r = 0; r < world; ++r) {
    XQT_REQUIRE(sources[r] != nullptr && flags[r] != nullptr && ((uintptr_t)sources[r] & 15) == 0);
    p.source[r] = reinterpret_cast<const uint4*>(sources[r]);
    p.flags[r] = reinterpret_cast<unsigned int*>(flags[r]);
  }
  p.rank = rank; p.world = world; p.vecs = bytes / 16; p.slot_stride = slot_stride_bytes / 16;
  p.out = reinterpret_cast<uint4*>(out); p.status = status; p.counter = counter;
  p.spin_limit = spin_limit == 0 ? kSpin : spin_limit;
  long long blocks = (p.vecs * world + 255) / 256;
  if (blocks > 148) blocks = 148;
  peer_allgather_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return launch_status();
}

int peer_allreduce_launch(const void* const* partials, void* const* flags, int rank, int world, unsigned int call,
                          long long count, int n, const float* bias, void* out, int out_dtype, unsigned int spin_limit,
                          unsigned int* status, unsigned int* counter, long long slot_stride, cudaStream_t stream) {
  using namespace par;
  XQT_REQUIRE(world >= 2 && world <= kMaxWorld && rank >= 0 && rank < world && (call > 0 || counter != nullptr));
  XQT_REQUIRE(counter == nullptr || (slot_stride >= count && slot_stride % 4 == 0));
  XQT_REQUIRE(count > 0 && count % 4 == 0 && n > 0 && n % 4 == 0 && count % n == 0);
  XQT_REQUIRE(partials != nullptr && flags != nullptr && out != nullptr && status != nullptr);
  XQT_REQUIRE(out_dtype == XQT_B200_BF16 || out_dtype == XQT_B200_FP16);
  XQT_REQUIRE(((uintptr_t)out & 7) == 0 && (bias == nullptr || ((uintptr_t)bias & 15) == 0));
  PeerReduceParams p{};
  for (int r = 0; r < world; ++r) {
    XQT_REQUIRE(partials[r] != nullptr && flags[r] != nullptr && ((uintptr_t)partials[r] & 15) == 0);
    p.partial[r] = reinterpret_cast<const float*>(partials[r]);
    p.flags[r] = reinterpret_cast<unsigned int*>(flags[r]);
  }
  p.rank = rank; p.world = world; p.call = call; p.count = count; p.n = n; p.bias = bias; p.out = out; p.status = status;
  p.spin_limit = spin_limit == 0 ? kSpin : spin_limit;
  p.counter = counter; p.slot_stride = slot_stride;
  const long long vecs = count / 4;
  long long blocks = (vecs + 255) / 256;
  if (blocks > 148) blocks = 148;
  if (out_dtype == XQT_B200_BF16) peer_allreduce_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(p);
  else peer_allreduce_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(p);
  return launch_status();
}

}  // namespace xqt_b200

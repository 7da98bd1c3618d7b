// One-shot all-reduce (sum, fp32) for the tensor-parallel decoder: the message after a row-sharded
// projection is 10 KB .. 650 KB, far below the size where ring or tree algorithms pay, and it
// happens 52 times per token, so latency is everything.  Every rank pushes its vector straight
// into a slot of every peer's buffer with plain stores over NVLink (peer-mapped symmetric memory,
// no TMA, no multicast), raises a per-chunk flag on the peer, waits for the flags of all ranks in
// its own buffer and adds the slots in rank order, so all ranks get bit-identical sums.
//
// Buffer of one rank (the same layout on every rank):
//   slots  [2 sets][world ranks][max_count floats]   written by the peers (slot r by rank r)
//   flags  [2 sets][world ranks][kChunks] uint32     written by the peers, value = sequence number
//   seq    [kChunks] uint32                          private: last finished sequence number per chunk
// Consecutive calls alternate between the two sets; a rank can be at most one call ahead of the
// slowest rank (it needs that rank's flag to finish), so a set is never overwritten while a peer
// still reads it.  The sequence number lives in device memory, which keeps a captured CUDA graph
// replayable.  Waits are bounded: after kSpinLimit probes the kernel writes NB_ERR_TIMEOUT to the
// status word and returns with whatever has arrived.
#include <cuda_runtime.h>

#include <algorithm>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

constexpr int kArChunks = 32;            // most CTAs per all-reduce (8 for decode-sized vectors, more for long ones)
constexpr int kArMaxWorld = 8;
constexpr uint32_t kArSpinLimit = 1u << 24;

struct ArParams {
  uint8_t* peers[kArMaxWorld];  // base of every rank's buffer as mapped into this process
  const float* in;
  float* out;
  int count, max_count, world, rank;
  uint32_t spin_limit;
  int* status;
};

__host__ __device__ inline size_t ar_slots_bytes(int world, int max_count) { return (size_t)2 * world * max_count * sizeof(float); }
__host__ __device__ inline size_t ar_flags_bytes(int world) { return (size_t)2 * world * kArChunks * sizeof(uint32_t); }

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(const ArParams p) {
  const int c = blockIdx.x, tid = threadIdx.x;
  uint8_t* self = p.peers[p.rank];
  uint32_t* seq_ptr = reinterpret_cast<uint32_t*>(self + ar_slots_bytes(p.world, p.max_count) + ar_flags_bytes(p.world)) + c;
  const uint32_t seq = *seq_ptr + 1;
  const int set = seq & 1;
  // this CTA's share of the vector, in float4 units
  const int n4 = p.count >> 2;
  const int per = (n4 + (int)gridDim.x - 1) / (int)gridDim.x;
  const int i0 = c * per, i1 = min(n4, i0 + per);
  const size_t slot_off = ((size_t)set * p.world + p.rank) * p.max_count;

  const float4* in4 = reinterpret_cast<const float4*>(p.in);
  for (int i = i0 + tid; i < i1; i += blockDim.x) {
    const float4 v = in4[i];
#pragma unroll
    for (int q = 0; q < kArMaxWorld; ++q)
      if (q < p.world) reinterpret_cast<float4*>(reinterpret_cast<float*>(p.peers[q]) + slot_off)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_timeout;
  if (tid == 0) s_timeout = 0;
  __syncthreads();
  if (tid < p.world) {
    // tell rank `tid` that this rank's chunk c of call `seq` is in place ...
    uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers[tid] + ar_slots_bytes(p.world, p.max_count)) +
                       ((size_t)set * p.world + p.rank) * kArChunks + c;
    st_release_sys(remote, seq);
    // ... and wait for rank `tid`'s chunk c in this rank's buffer
    const uint32_t* local = reinterpret_cast<const uint32_t*>(self + ar_slots_bytes(p.world, p.max_count)) +
                            ((size_t)set * p.world + tid) * kArChunks + c;
    uint32_t spins = 0;
    while (ld_acquire_sys(local) != seq) {
      if (++spins > p.spin_limit) {
        s_timeout = 1;
        if (p.status) atomicExch(p.status, (int)NB_ERR_TIMEOUT);
        break;
      }
      if (spins > 64) __nanosleep(32);   // a late peer: stop hammering the NVLink-mapped flag
    }
  }
  __syncthreads();
  const float* slots = reinterpret_cast<const float*>(self) + (size_t)set * p.world * p.max_count;
  float4* out4 = reinterpret_cast<float4*>(p.out);
  for (int i = i0 + tid; i < i1; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kArMaxWorld; ++q) {
      if (q < p.world) {
        const float4 v = __ldcv(reinterpret_cast<const float4*>(slots + (size_t)q * p.max_count) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    out4[i] = acc;
  }
  __syncthreads();
  if (tid == 0) *seq_ptr = seq;
}

}  // namespace nb

using namespace nb;

extern "C" size_t nb_allreduce_buffer_bytes(int world, int max_count) {
  if (world < 1 || world > kArMaxWorld || max_count < 4 || (max_count & 3)) return 0;
  return ar_slots_bytes(world, max_count) + ar_flags_bytes(world) + kArChunks * sizeof(uint32_t);
}

extern "C" int nb_allreduce(const float* in, float* out, int count, const uint64_t* peer_bufs, int world, int rank,
                            int max_count, uint32_t spin_limit, int* status, void* stream) {
  if (!in || !out || !peer_bufs || world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return NB_ERR_ARG;
  if (count < 4 || (count & 3) || count > max_count || (max_count & 3)) return NB_ERR_SHAPE;
  if ((uintptr_t)in % 16 || (uintptr_t)out % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  ArParams p{};
  for (int q = 0; q < world; ++q) {
    if (!peer_bufs[q] || peer_bufs[q] % 16) return NB_ERR_ALIGN;
    p.peers[q] = reinterpret_cast<uint8_t*>(peer_bufs[q]);
  }
  p.in = in; p.out = out; p.count = count; p.max_count = max_count; p.world = world; p.rank = rank;
  p.spin_limit = spin_limit ? spin_limit : kArSpinLimit;
  p.status = status;
  // A plain, fully stream-ordered launch.  Programmatic dependent launch was measured on two GPUs (2.2B decoder,
  // batch 1): releasing the next kernel at this kernel's start 1.94 ms/token, after its dependency wait 1.66 ms,
  // plain launch 1.56 ms — the kernels that start early crowd out the GEMV that is still computing.
  // every rank derives the same number of CTAs from the count: 8 up to 4096 floats per CTA, then more, up to kArChunks
  const int ctas = std::min(kArChunks, std::max(8, count / 2048));
  allreduce_oneshot_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(p);
  return check_launch();
}

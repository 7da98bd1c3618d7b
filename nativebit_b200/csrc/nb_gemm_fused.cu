// Fused prefill GEMM for NativeBit packed linears on sm_100a: Y (M, N) = X (M, K) . W (N, K)^T for many
// activation rows, with the dequantisation INSIDE the tensor-core kernel: producer warps turn packed
// indices + codebooks into fp16 tiles in shared memory and tcgen05.mma consumes them, so the weight never
// exists in global memory as a dense matrix.  The reference materialises the whole weight on every
// forward (unpack + gather + matmul, inference/triton_kernel.py:258-275); its tiled TPU kernel
// dequantises a tile and contracts it (nativebit_jax/packed_kernel.py:135-178), which is the semantics
// kept here with one difference: the weights enter as the fp16 codebook entries themselves (exact).
//
// Operands.  The WEIGHT tile is the M = 128 operand of the MMA (128 output features x 64 k), the
// ACTIVATION tile the N operand (BN = 16..256 tokens x 64 k), the accumulator D[feature][token] lives in
// tensor memory.  A weight tile is therefore dequantised once per BN tokens; at BN = 256 that is 8192
// lookups per 512 tensor-core clocks, a quarter of the SM's byte-permute throughput.
//
// Weights are read in the stream layout (nb_stream_pack: per 16 rows x 128 weights, every lane-group's
// indices as nibbles in position order + the rows' byte-plane lookup tables), straight from L2 into
// registers.  Persistent kernel, one CTA per SM, 704 threads:
//   warp 0       one lane issues the TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast)
//                of the BN x 64 activation slab of every k-step into a ring of stages;
//   warp 1       allocates tensor memory; one lane waits on the stage's "full" barrier (eight producer warps'
//                arrivals + the TMA bytes) and issues four tcgen05.mma (128 x BN x 16, fp16 x fp16 -> fp32)
//                per stage, then tcgen05.commit on the stage's "empty" barrier;
//   warps 2-5    epilogue: each warp owns one 32-lane quadrant of tensor memory (32 output features),
//                reads a finished accumulator with tcgen05.ld and stores Y (transposed: lanes run along
//                N, so a warp's store of one token covers 32 consecutive outputs);
//   warps 6-21   dequant producers, two groups of 8 warps that take turns at the k-steps (filling a stage is
//                a chain of dependent steps, so two stages are filled at a time): thread (row, half) of the
//                128 x 64 weight tile loads four selector words and the row's table (prefetched one of its
//                k-steps ahead), looks 32 weights up with byte permutes and writes them as four 16-byte
//                chunks into the 128-byte-swizzled stage.
// Two accumulators in tensor memory let the epilogue of one tile overlap the MMAs of the next.  Every
// mbarrier wait is bounded; on a timeout the waiter raises a shared abort flag, writes NB_ERR_TIMEOUT
// to the status word and all roles fall through to the exit, where tensor memory is freed.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdio>

#include "nb_common.cuh"
#include "nb_device.cuh"
#include "nb_host.h"
#include "nb_umma.cuh"

namespace nb {

constexpr int kFM = 128;                  // output features per tile (the MMA's M)
constexpr int kFK = 64;                   // k per stage
constexpr int kFProducerWarp0 = 6, kFProducerWarps = 8;   // warps per producer group
constexpr int kFGroups = 2;                                // groups take turns at the k-steps
constexpr int kFThreads = (kFProducerWarp0 + kFGroups * kFProducerWarps) * 32;
constexpr int kFABytes = kFM * kFK * 2;   // 16 KB of weights per stage
constexpr int kFRing = 192 * 1024;
constexpr int kFMaxStages = 8;
constexpr int kFSmem = kFRing + 1024 + 512;

__host__ __device__ constexpr int fused_stages(int bn) {
  return kFRing / (kFABytes + bn * kFK * 2) < kFMaxStages ? kFRing / (kFABytes + bn * kFK * 2) : kFMaxStages;
}

#ifdef NB_FUSED_TRACE
__device__ long long g_ftrace[8][512];
#define FTRACE(role, kt) do { if (blockIdx.x == 0 && (kt) < 512) g_ftrace[role][kt] = clock64(); } while (0)
#else
#define FTRACE(role, kt) do {} while (0)
#endif

template <int BITS> struct FusedFmt {
  static constexpr int kTabBytes = BITS == 4 ? 32 : 16;
  static constexpr int kUnitBytes = 1024 + 16 * kTabBytes;   // the stream layout's unit (nb_stream.cu)
};

template <int BITS>
__global__ void __launch_bounds__(kFThreads, 1)
gemm_fused_kernel(const __grid_constant__ CUtensorMap map_x, const uint8_t* __restrict__ w_stream, void* __restrict__ y, int y_dtype,
                  int M, int N, int K, int BN, int m_tiles, int w_tiles, int pair, int ks, float* __restrict__ partial, int* status) {
  using F = FusedFmt<BITS>;
  constexpr int kT = BITS == 4 ? 8 : 4;
  const int S = fused_stages(BN);
  const int b_bytes = BN * kFK * 2;           // multiple of 1024 because BN is a multiple of 16
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                         // weights
  uint8_t* sB = smem + S * kFABytes;          // activations
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kFRing);   // a stage's weights (8 producer warps) AND activations (TMA bytes)
  uint64_t* empty = full + kFMaxStages;
  uint64_t* acc_full = empty + kFMaxStages;   // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;         // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KT = K / kFK, bpr = K / kBlock;
  const int KTs = (KT + ks - 1) / ks;           // k-steps per k split (the last split may be shorter, never empty)
  const int n_total = m_tiles * w_tiles * ks;   // work item t: k split t % ks of output tile t / ks
  const int rows_padded = ((N + 15) >> 4) << 4;   // rows the stream layout holds (zero rows past N)

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(&full[s], kFProducerWarps + 1); bar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { bar_init(&acc_full[b], 1); bar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // output tile o = t / ks: features 128 * (o / m_tiles), tokens BN * (o % m_tiles): CTAs running together share a
  // weight tile; with ks > 1 the k range of an output tile is cut into ks parts whose fp32 results go to
  // `partial` and are added in k order by a second kernel (short inputs would otherwise leave most SMs idle
  // behind a long serial chain of k-steps)
  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer of the activation slabs
      int s = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
        const int m0 = ((t / ks) % m_tiles) * BN;
        const int k_lo = (t % ks) * KTs, k_hi = min(KT, k_lo + KTs);
        bool ok = true;
        for (int kt = k_lo; kt < k_hi; ++kt) {
          ok = bar_wait(&empty[s], phase ^ 1, abort_flag, status);
          if (!ok) break;
          FTRACE(0, kt);
          bar_expect_tx(&full[s], (uint32_t)b_bytes);
          tma_load_2d(sB + s * b_bytes, &map_x, &full[s], kt * kFK, m0);
          if (++s == S) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      // instruction descriptor: fp32 accumulate (bit 4), A and B fp16 (format 0 at bits 7 and 10), both K-major,
      // N = BN (tokens), M = 128 (features)
      const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kFM >> 4) << 24);
      const uint64_t desc_a0 = smem_desc_sw128(sA), desc_b0 = smem_desc_sw128(sB);
      int s = 0, local = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x, ++local) {
        const int buf = local & 1;
        bool ok = bar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * 256);
        const int k_lo = (t % ks) * KTs, k_hi = min(KT, k_lo + KTs);
        for (int kt = k_lo; kt < k_hi && ok; ++kt) {
          ok = bar_wait(&full[s], phase, abort_flag, status);
          if (!ok) break;
          FTRACE(2, kt);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          // the stage's descriptors: the start-address field counts 16-byte units, so a stage further on is an add
          const uint64_t da = desc_a0 + (uint64_t)(s * (kFABytes >> 4)), db = desc_b0 + (uint64_t)(s * (b_bytes >> 4));
          umma_f16(tmem_d, da, db, idesc, kt > k_lo ? 1u : 0u);
#pragma unroll
          for (int k4 = 1; k4 < kFK / 16; ++k4)  // 16 fp16 = 32 bytes = 2 descriptor address units per step
            umma_f16(tmem_d, da + 2 * k4, db + 2 * k4, idesc, 1u);
          umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
          if (++s == S) { s = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[buf]);
        if (!ok) break;
      }
    }
  } else if (warp < kFProducerWarp0) {
    // ---- epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +31 = features n0 + 32*(w%4) + lane
    const int q = warp & 3;
    int local = 0;
    for (int t = blockIdx.x; t < n_total; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const int o = t / ks;
      const int m0 = (o % m_tiles) * BN, n0 = (o / m_tiles) * kFM;
      // with k splits the tile's fp32 sums go to this split's slab of `partial` ((M >> pair) x N floats each)
      void* const y_t = ks > 1 ? (void*)(partial + (size_t)(t % ks) * (size_t)(M >> pair) * N) : y;
      const int y_dt = ks > 1 ? (int)NB_F32 : y_dtype;
      const bool ok = bar_wait<200>(&acc_full[buf], (local >> 1) & 1, abort_flag, status) && !*abort_flag;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = n0 + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t r[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + c * 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (n < N && pair) {
          // rows 2i and 2i+1 of the operand are the two fp16 terms of activation row i: their results are added
          const int mb = (m0 + c * 16) >> 1;
          const int m_out = M >> 1;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (mb + j < m_out) {
              const float v = __uint_as_float(r[2 * j]) + __uint_as_float(r[2 * j + 1]);
              if (y_dt == NB_BF16) reinterpret_cast<__nv_bfloat16*>(y_t)[(size_t)(mb + j) * N + n] = __float2bfloat16_rn(v);
              else reinterpret_cast<float*>(y_t)[(size_t)(mb + j) * N + n] = v;
            }
          }
        } else if (n < N) {
          const int mb = m0 + c * 16;
          if (y_dt == NB_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(y_t) + (size_t)mb * N + n;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (mb + j < M) dst[(size_t)j * N] = __float2bfloat16_rn(__uint_as_float(r[j]));
          } else {
            float* dst = reinterpret_cast<float*>(y_t) + (size_t)mb * N + n;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (mb + j < M) dst[(size_t)j * N] = __uint_as_float(r[j]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s2u(&acc_empty[buf])) : "memory");
    }
  } else {
    // ---- dequant producers: thread (row, half) writes 32 weights = 64 bytes of row `row` of the stage
    const int p = threadIdx.x - kFProducerWarp0 * 32;
    const int grp = p >> 8, pp = p & 255;                // group `grp` fills the k-steps kt with kt % kFGroups == grp
    const int row = pp & 127, q2 = pp >> 7;
    const int r16 = row & 15, g = r16 & 7, hrow = r16 >> 3;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint32_t step0 = 0;                                  // k-steps of all earlier work items: stage = step % S, phase = (step / S) & 1
    for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
      const int n0 = ((t / ks) / m_tiles) * kFM;
      const int k_lo = (t % ks) * KTs, k_hi = min(KT, k_lo + KTs);
      const int grow = n0 + row;
      const bool valid = grow < rows_padded;
      const uint8_t* urow = w_stream + (size_t)(grow >> 4) * bpr * F::kUnitBytes;   // the row tile's units
      // k-step kt covers positions 64*(kt&1) .. +63 of k-block kt>>1: this thread's lane group is t = 2*(kt&1) + q2
      auto load = [&](int kt, uint4& sel, uint4 (&tab)[kT / 4]) {
        sel = zero4;
#pragma unroll
        for (int j = 0; j < kT / 4; ++j) tab[j] = zero4;
        if (valid && kt < k_hi) {
          const uint8_t* u = urow + (size_t)(kt >> 1) * F::kUnitBytes;
          const int lane_u = g * 4 + 2 * (kt & 1) + q2;
          sel = __ldg(reinterpret_cast<const uint4*>(u + hrow * 512 + lane_u * 16));
#pragma unroll
          for (int j = 0; j < kT / 4; ++j) tab[j] = __ldg(reinterpret_cast<const uint4*>(u + 1024 + r16 * F::kTabBytes + 16 * j));
        }
      };
      uint4 sel, tab[kT / 4];
      load(k_lo + grp, sel, tab);
      bool ok = true;
      for (int kt = k_lo + grp; kt < k_hi; kt += kFGroups) {
        uint4 sel_n, tab_n[kT / 4];
        load(kt + kFGroups, sel_n, tab_n);               // this group's next k-step, in flight while this one is unpacked
        const uint32_t step = step0 + (uint32_t)(kt - k_lo);
        const int s = (int)(step % (uint32_t)S);
        const uint32_t phase = (step / (uint32_t)S) & 1u;
        if (pp == 0) FTRACE(3, kt);
        ok = bar_wait<20>(&empty[s], phase ^ 1, abort_flag, status);
        if (!ok) break;
        if (pp == 0) FTRACE(4, kt);
        uint32_t T[kT];
#pragma unroll
        for (int j = 0; j < kT / 4; ++j) { T[4 * j] = tab[j].x; T[4 * j + 1] = tab[j].y; T[4 * j + 2] = tab[j].z; T[4 * j + 3] = tab[j].w; }
        const uint32_t words[4] = {sel.x, sel.y, sel.z, sel.w};
        // row `row` of a K-major tile with 128-byte swizzle: 16-byte chunk c sits at chunk c ^ (row & 7)
        uint8_t* rbase = sA + s * kFABytes + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a, b, c, d;
          lookup4<BITS>(words[j], T, a, b);              // positions 8j .. 8j+3
          lookup4<BITS>(words[j] >> 16, T, c, d);        // positions 8j+4 .. 8j+7
          const int chunk = (4 * q2 + j) ^ (row & 7);
          *reinterpret_cast<uint4*>(rbase + chunk * 16) = make_uint4(a, b, c, d);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s2u(&full[s])) : "memory");
        if (pp == 0) FTRACE(5, kt);
        sel = sel_n;
#pragma unroll
        for (int j = 0; j < kT / 4; ++j) tab[j] = tab_n[j];
      }
      if (!ok) break;
      step0 += (uint32_t)(k_hi - k_lo);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// bf16 -> fp16, eight elements per thread, saturating to +-65504 (exact for magnitudes 6.1e-5 .. 65504).
__global__ void __launch_bounds__(256) bf16_to_f16_kernel2(const uint4* __restrict__ in, uint4* __restrict__ out, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 v = in[i];
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) r[j] = f32x2_to_f16x2_sat(__uint_as_float(u[j] << 16), __uint_as_float(u[j] & 0xFFFF0000u));
  out[i] = make_uint4(r[0], r[1], r[2], r[3]);
}

// Tile plan of one call: token-tile width BN (a multiple of 16 up to 256) and number of k splits.  A k-step of a work
// item costs the longer of the tensor-core time, 2 * BN clocks, and the time the producers need to fill a stage, which
// does not depend on BN (measured: about kProducerClocks); a work item is one k split of one 128 x BN output tile, the
// items run in waves of one per SM.  The plan with the fewest estimated clocks wins: waves * k-steps per item * clocks
// per k-step, plus a charge for the second kernel that adds the splits' results (fixed part + its reads).  Splits keep at least four
// k-steps each and none is empty; inputs of up to 256 operand rows take one token tile.
constexpr int kProducerClocks = 340;
constexpr int kSplitCharge = 3000;
struct FusedPlan { int bn, ks; };
static FusedPlan plan_fused(int rows, int N, int K, int sms) {
  const int KT = K / kFK;
  const int w_tiles = (N + kFM - 1) / kFM;
  FusedPlan best{256, 1};
  double best_cost = 1e30;
  const int bn_hi = rows <= 256 ? std::min(256, (rows + 15) / 16 * 16) : 256;
  const int bn_lo = rows <= 256 ? bn_hi : 96;
  for (int bn = bn_hi; bn >= bn_lo; bn -= 16) {
    const long tiles = (long)w_tiles * ((rows + bn - 1) / bn);
    for (int ks = 1; ks <= 8; ++ks) {
      const int kts = (KT + ks - 1) / ks;
      if (ks > 1 && (kts < 4 || (long)(ks - 1) * kts >= KT)) continue;
      const long waves = (tiles * ks + sms - 1) / sms;
      // the second kernel reads ks slabs of rows x N floats at roughly 3 KB per clock
      const double sum_cost = ks > 1 ? kSplitCharge + (double)ks * rows * N * 4.0 / 3000.0 : 0.0;
      const double cost = (double)waves * kts * std::max(2 * bn, kProducerClocks) + sum_cost;
      if (cost < best_cost * 0.98) { best_cost = cost; best = FusedPlan{bn, ks}; }
    }
  }
  return best;
}

// y (rows x N) = sum over the k splits' fp32 slabs, in split order; four outputs per thread.
__global__ void __launch_bounds__(256) splitk_sum_kernel(const float* __restrict__ partial, int ks, size_t slab, void* __restrict__ y,
                                                         int y_dtype, size_t n4) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 acc = reinterpret_cast<const float4*>(partial)[i];
  for (int z = 1; z < ks; ++z) {
    const float4 v = reinterpret_cast<const float4*>(partial + (size_t)z * slab)[i];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (y_dtype == NB_BF16) {
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(y) + 2 * i;
    dst[0] = __floats2bfloat162_rn(acc.x, acc.y);
    dst[1] = __floats2bfloat162_rn(acc.z, acc.w);
  } else {
    reinterpret_cast<float4*>(y)[i] = acc;
  }
}

// (rows, cols) row-major 16-bit matrix -> tensor map with a (box_rows x 64) box and 128-byte swizzle.
static int make_map_f16(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
  return make_map(map, base, rows, cols, box_rows);   // element size and swizzle are those of the bf16 maps
}

}  // namespace nb

using namespace nb;

#ifdef NB_FUSED_TRACE
extern "C" int nb_fused_trace_read(long long* host) { return (int)cudaMemcpyFromSymbol(host, g_ftrace, sizeof(g_ftrace)); }
#endif

// Workspace: [256 B status][fp16 operand rows x K][k-split slabs: ks x (M x N) floats]; sized for the worse of the
// one-term (bf16 / fp16) and two-term (fp32) forms of M activation rows.
static size_t fused_partial_bytes(int rows, int M, int N, int K) {
  const int ks = plan_fused(rows, N, K, sm_count()).ks;
  return ks > 1 ? (size_t)ks * M * N * sizeof(float) : 0;
}

extern "C" size_t nb_prefill_fused_workspace_bytes(int M, int N, int K) {
  if (M < 1 || N < 1 || K < kFK) return 0;
  const size_t x_bytes = ((size_t)2 * M * K * 2 + 255) / 256 * 256;
  return 256 + x_bytes + std::max(fused_partial_bytes(M, M, N, K), fused_partial_bytes(2 * M, M, N, K));
}

extern "C" int nb_gemm_prefill_fused(const void* x, int x_dtype, int M, const uint8_t* w_stream, int bits, int N, int K, void* y,
                                     int y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !w_stream || !y || M < 1 || N < 1 || K < 1) return NB_ERR_ARG;
  if (x_dtype != NB_BF16 && x_dtype != NB_F16 && x_dtype != NB_F32) return NB_ERR_ARG;
  if (y_dtype != NB_BF16 && y_dtype != NB_F32) return NB_ERR_ARG;
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_SHAPE;
  if (K % kBlock != 0) return NB_ERR_SHAPE;
  if (!workspace || workspace_bytes < nb_prefill_fused_workspace_bytes(M, N, K)) return NB_ERR_WORKSPACE;
  if ((uintptr_t)workspace % 256 || (uintptr_t)x % 16 || (uintptr_t)w_stream % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const void* xh = x;
  const int pair = x_dtype == NB_F32 ? 1 : 0;
  const int rows = pair ? 2 * M : M;              // rows of the fp16 operand
  uint8_t* dst = reinterpret_cast<uint8_t*>(workspace) + 256;
  if (x_dtype == NB_BF16) {
    const size_t n8 = (size_t)M * K / 8;
    bf16_to_f16_kernel2<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(dst), n8);
    if (int rc = check_launch()) return rc;
    xh = dst;
  } else if (x_dtype == NB_F32) {
    const size_t n8 = (size_t)M * K / 8;
    f32_to_f16_pair_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<uint4*>(dst), M, K);
    if (int rc = check_launch()) return rc;
    xh = dst;
  }
  const int sms = sm_count();
  const FusedPlan plan = plan_fused(rows, N, K, sms);
  const int bn = plan.bn;
  CUtensorMap mx;
  if (int rc = make_map_f16(&mx, xh, rows, K, bn)) return rc;
  const int m_tiles = (rows + bn - 1) / bn, w_tiles = (N + kFM - 1) / kFM;
  int ks = plan.ks;
  if (ks > 1 && (N % 4 != 0 || (uintptr_t)y % 16)) ks = 1;       // the summing kernel writes four outputs at a time
  float* partial = reinterpret_cast<float*>(dst + ((size_t)2 * M * K * 2 + 255) / 256 * 256);
  const int grid = std::min(sms, m_tiles * w_tiles * ks);
  int* status = reinterpret_cast<int*>(workspace);
  static bool attr_done[64][5] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const void* fn = bits == 3 ? (const void*)gemm_fused_kernel<3> : bits == 2 ? (const void*)gemm_fused_kernel<2> : (const void*)gemm_fused_kernel<4>;
  if (!attr_done[dev & 63][bits]) {
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem)) return record_cuda_error(e);
    attr_done[dev & 63][bits] = true;
  }
  if (bits == 3) gemm_fused_kernel<3><<<grid, kFThreads, kFSmem, st>>>(mx, w_stream, y, y_dtype, rows, N, K, bn, m_tiles, w_tiles, pair, ks, partial, status);
  else if (bits == 2) gemm_fused_kernel<2><<<grid, kFThreads, kFSmem, st>>>(mx, w_stream, y, y_dtype, rows, N, K, bn, m_tiles, w_tiles, pair, ks, partial, status);
  else gemm_fused_kernel<4><<<grid, kFThreads, kFSmem, st>>>(mx, w_stream, y, y_dtype, rows, N, K, bn, m_tiles, w_tiles, pair, ks, partial, status);
  if (int rc = check_launch()) return rc;
  if (ks > 1) {
    const size_t n4 = (size_t)M * N / 4;
    splitk_sum_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(partial, ks, (size_t)M * N, y, y_dtype, n4);
    return check_launch();
  }
  return NB_OK;
}

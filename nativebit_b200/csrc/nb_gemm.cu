// Prefill GEMM for NativeBit packed linears on sm_100a: Y (M, N) = X (M, K) . W (N, K)^T for many
// activation rows, on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// nb_gemm_prefill dequantises the packed weight once into an fp16 (N, K) scratch matrix (35 MB for
// 6912 x 2560: it stays in the 126 MB L2) with the gather kernel of nb_unpack.cu, then runs the
// kernel below on X and that matrix.  W enters as fp16 (the codebook entries themselves, so the
// weights are exact; the reference's any-M kernel rounds them to bf16,
// nativebit_jax/packed_kernel.py:151-159).  The tensor-core instruction wants both operands in one
// 16-bit format (a bf16 A with an fp16 B is an illegal instruction on sm_100a), so bf16 activations
// are first converted to fp16 (exact for magnitudes 6.1e-5..65504, saturating above, as in the
// GEMV).  Products are accumulated in fp32.
//
// Kernel: persistent, one CTA per SM walking 128 x BN output tiles (BN = a multiple of 16 in
// [128, 256] chosen to fill the last wave), two accumulator buffers in tensor memory, 192 threads:
//   warp 0   one lane issues TMA tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//            128 x 64 slab of X and a BN x 64 slab of W per k-step into a ring of shared-memory
//            stages, each completing on the stage's "full" mbarrier;
//   warp 1   allocates the 512 columns of tensor memory; one lane waits for a full stage and issues
//            four tcgen05.mma (M=128, N=BN, K=16) per stage from shared-memory descriptors, then
//            tcgen05.commit on the stage's "empty" barrier (and on the accumulator barrier at the end);
//   warps 2-5  epilogue: each warp owns one 32-lane quadrant of tensor memory, reads the finished
//            buffer with tcgen05.ld (16 columns at a time), converts and stores its 32 rows of Y,
//            then hands the buffer back, while the MMA warp already fills the other buffer.
// Every mbarrier wait is bounded: after kSpinLimit probes the waiter raises a shared abort flag,
// writes NB_ERR_TIMEOUT to the status word and all roles fall through to the common exit, where
// tensor memory is freed.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "nb_common.cuh"
#include "nb_host.h"
#include "nb_umma.cuh"

namespace nb {

struct GemmCfg {
  static constexpr int kMaxStages = 8;
  static constexpr int kMaxBN = 256;
  static constexpr int kABytes = kBM * kBK * 2;          // 16 KB
  static constexpr int kRing = 4 * (kABytes + kMaxBN * kBK * 2);  // 192 KB of operand stages
  static constexpr int kSmem = kRing + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // number of stages that fit the ring for a tile width (4 at BN = 256, 5 at 144, 6 at 128)
  __host__ __device__ static constexpr int stages(int bn) {
    return kRing / (kABytes + bn * kBK * 2) < kMaxStages ? kRing / (kABytes + bn * kBK * 2) : kMaxStages;
  }
  static constexpr int kTmemCols = 512;                  // two accumulator buffers of up to 256 columns
};

// Persistent kernel: CTA b works on output tiles b, b + gridDim.x, ...; tile t covers rows
// 128*(t % m_tiles) and columns BN*(t / m_tiles), so CTAs running together share a W slab in L2.
// Two accumulator buffers in tensor memory let the epilogue of one tile overlap the MMAs of the next.
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, void* __restrict__ y,
                 int y_dtype, int M, int N, int K, int BN, int m_tiles, int n_tiles, int f16, int pair, int* status) {
  using Cfg = GemmCfg;
  const int S = Cfg::stages(BN);
  const int b_bytes = BN * kBK * 2;   // multiple of 1024 because BN is a multiple of 16
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + S * Cfg::kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::kRing);
  uint64_t* empty = full + Cfg::kMaxStages;
  uint64_t* acc_full = empty + Cfg::kMaxStages;     // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2; // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KT = K / kBK;
  const int n_total = m_tiles * n_tiles;
  const uint32_t stage_bytes = (uint32_t)(Cfg::kABytes + b_bytes);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(&full[s], 1); bar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { bar_init(&acc_full[b], 1); bar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer
      int s = 0;           // ring position and its phase bit, carried across tiles
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
        const int m0 = (t % m_tiles) * kBM, n0 = (t / m_tiles) * BN;
        bool ok = true;
        for (int kt = 0; kt < KT; ++kt) {
          ok = bar_wait(&empty[s], phase ^ 1, abort_flag, status);
          if (!ok) break;
          bar_expect_tx(&full[s], stage_bytes);
          tma_load_2d(sA + s * Cfg::kABytes, &map_x, &full[s], kt * kBK, m0);
          tma_load_2d(sB + s * b_bytes, &map_w, &full[s], kt * kBK, n0);
          if (++s == S) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      // instruction descriptor: fp32 accumulate (bit 4), A = X and B = W both bf16 (format 1) or both
      // fp16 (format 0) at bits 7 and 10, both K-major, N = BN, M = 128
      const uint32_t fmt = f16 ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      const uint64_t desc_a0 = smem_desc_sw128(sA), desc_b0 = smem_desc_sw128(sB);
      int s = 0, local = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x, ++local) {
        const int buf = local & 1;
        // wait until the epilogue has drained this accumulator buffer (first use passes at once)
        bool ok = bar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * Cfg::kMaxBN);
        for (int kt = 0; kt < KT && ok; ++kt) {
          ok = bar_wait(&full[s], phase, abort_flag, status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          // the stage's descriptors: the start-address field counts 16-byte units, so a stage further on is an add
          const uint64_t da = desc_a0 + (uint64_t)(s * (Cfg::kABytes >> 4)), db = desc_b0 + (uint64_t)(s * (b_bytes >> 4));
          umma_f16(tmem_d, da, db, idesc, kt > 0 ? 1u : 0u);
#pragma unroll
          for (int k4 = 1; k4 < kBK / 16; ++k4)  // 16 bf16 = 32 bytes = 2 descriptor address units per step
            umma_f16(tmem_d, da + 2 * k4, db + 2 * k4, idesc, 1u);
          umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
          if (++s == S) { s = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[buf]);  // accumulator complete (or aborted: the epilogue checks the flag)
        if (!ok) break;
      }
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +31 = rows m0 + 32*(w%4) + lane
    const int q = warp & 3;
    int local = 0;
    for (int t = blockIdx.x; t < n_total; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (t % m_tiles) * kBM, n0 = (t / m_tiles) * BN;
      const bool ok = bar_wait<200>(&acc_full[buf], (local >> 1) & 1, abort_flag, status) && !*abort_flag;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t r[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::kMaxBN + c * 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int n = n0 + c * 16;
        int m_st = m, rows_st = M;
        if (pair) {
          // operand rows 2i and 2i+1 are the two fp16 terms of activation row i: adjacent lanes add their results
          // (every lane takes part in the shuffles), the even lane stores output row i
#pragma unroll
          for (int j = 0; j < 16; ++j)
            r[j] = __float_as_uint(__uint_as_float(r[j]) + __shfl_xor_sync(0xffffffffu, __uint_as_float(r[j]), 1));
          m_st = m >> 1;
          rows_st = M >> 1;
        }
        if ((!pair || !(lane & 1)) && m_st < rows_st && n < N) {
          const bool whole = n + 16 <= N;
          if (y_dtype == NB_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(y) + (size_t)m_st * N + n;
            if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
              uint32_t pk[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                pk[j] = *reinterpret_cast<const uint32_t*>(&h);
              }
              reinterpret_cast<uint4*>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              reinterpret_cast<uint4*>(dst)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* dst = reinterpret_cast<float*>(y) + (size_t)m_st * N + n;
            if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n + j < N) dst[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
      // this warp is done with the buffer: one arrival per warp (4 in total) hands it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s2u(&acc_empty[buf])) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
  }
}

// Tile width: the multiple of 16 in [128, 256] that wastes the least of the last wave of CTAs
// (ties go to the wider tile, which reads X fewer times).
static int pick_bn(int M, int N, int sms) {
  const int m_tiles = (M + kBM - 1) / kBM;
  int best = 256;
  double best_eff = -1.0;
  for (int bn = 256; bn >= 128; bn -= 16) {
    const long tiles = (long)m_tiles * ((N + bn - 1) / bn);
    const long waves = (tiles + sms - 1) / sms;
    const double eff = (double)M * N / ((double)waves * sms * kBM * bn);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = bn; }
  }
  return best;
}

static int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, void* y, int y_dtype, int M, int N, int K, int bn,
                       int f16, int pair, int* status, cudaStream_t st) {
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    if (cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg::kSmem))
      return record_cuda_error(e);
    attr_done[dev & 63] = true;
  }
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + bn - 1) / bn;
  const int grid = std::min(sm_count(), m_tiles * n_tiles);
  gemm_bf16_kernel<<<grid, 192, GemmCfg::kSmem, st>>>(mx, mw, y, y_dtype, M, N, K, bn, m_tiles, n_tiles, f16, pair, status);
  return check_launch();
}

}  // namespace nb

using namespace nb;

extern "C" size_t nb_prefill_workspace_bytes(int M, int N, int K) {
  if (M < 1 || N < 1 || K < 1) return 0;
  // status word (first 256 bytes) + fp16 weight + fp16 copy of the activations (two terms per element for fp32)
  return 256 + (((size_t)N * K * 2 + 255) & ~(size_t)255) + (size_t)2 * M * K * 2;
}

namespace nb {
// bf16 -> fp16, eight elements per thread, saturating to +-65504.
__global__ void __launch_bounds__(256) bf16_to_f16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 v = in[i];
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = __uint_as_float(u[j] << 16), b = __uint_as_float(u[j] & 0xFFFF0000u);
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r[j]) : "f"(b), "f"(a));
  }
  out[i] = make_uint4(r[0], r[1], r[2], r[3]);
}
}  // namespace nb

// x (M, K) times w (N, K), both bf16 or both fp16 (f16).  The tensor maps copy 2-byte elements either way.  pair: rows
// 2i and 2i+1 of x are the two fp16 terms of one activation row; y then has M / 2 rows.
static int gemm_16bit(const void* x, const void* w, int f16, int M, int N, int K, void* y, int y_dtype, int* status, void* stream,
                      int pair = 0) {
  if (!x || !w || !y || M < 1 || N < 1 || K < 1) return NB_ERR_ARG;
  if (y_dtype != NB_BF16 && y_dtype != NB_F32) return NB_ERR_ARG;
  if (K % kBK != 0) return NB_ERR_SHAPE;
  if ((uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 4) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const int bn = pick_bn(M, N, sm_count());
  CUtensorMap mx, mw;
  if (int rc = make_map(&mx, x, M, K, kBM)) return rc;
  if (int rc = make_map(&mw, w, N, K, bn)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  return launch_gemm(mx, mw, y, y_dtype, M, N, K, bn, f16, pair, status, st);
}

extern "C" int nb_gemm_bf16(const void* x, const void* w, int M, int N, int K, void* y, int y_dtype, int* status, void* stream) {
  return gemm_16bit(x, w, 0, M, N, K, y, y_dtype, status, stream);
}

extern "C" int nb_gemm_prefill(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype, int bits,
                               int block_size, int N, int K, void* y, int y_dtype, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if (!x || !packed || !codebook || !y) return NB_ERR_ARG;
  if (x_dtype != NB_BF16 && x_dtype != NB_F16 && x_dtype != NB_F32) return NB_ERR_ARG;
  if (!workspace || workspace_bytes < nb_prefill_workspace_bytes(M, N, K)) return NB_ERR_WORKSPACE;
  if ((uintptr_t)workspace % 256) return NB_ERR_ALIGN;
  if (K % kBK != 0 || K % block_size != 0) return NB_ERR_SHAPE;
  if ((uintptr_t)x % 16) return NB_ERR_ALIGN;
  uint8_t* w = reinterpret_cast<uint8_t*>(workspace) + 256;
  uint8_t* xh = w + (((size_t)N * K * 2 + 255) & ~(size_t)255);
  if (int rc = nb_dequant(packed, codebook, cb_dtype, bits, block_size, N, K, w, NB_F16, stream)) return rc;
  if (x_dtype == NB_F16) return gemm_16bit(x, w, 1, M, N, K, y, y_dtype, reinterpret_cast<int*>(workspace), stream);
  const size_t n8 = (size_t)M * K / 8;  // K % 64 == 0
  if (x_dtype == NB_F32) {  // two fp16 terms per element as operand rows 2i, 2i+1; the epilogue adds their results
    f32_to_f16_pair_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const float4*>(x),
                                                                                          reinterpret_cast<uint4*>(xh), M, K);
    if (int rc = check_launch()) return rc;
    return gemm_16bit(xh, w, 1, 2 * M, N, K, y, y_dtype, reinterpret_cast<int*>(workspace), stream, 1);
  }
  bf16_to_f16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint4*>(x),
                                                                                    reinterpret_cast<uint4*>(xh), n8);
  if (int rc = check_launch()) return rc;
  return gemm_16bit(xh, w, 1, M, N, K, y, y_dtype, reinterpret_cast<int*>(workspace), stream);
}

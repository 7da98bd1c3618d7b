// Prefill GEMM for NativeBit packed linears on sm_100a: Y (M, N) = X (M, K) . W (N, K)^T for many
// activation rows, on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
//
// nb_gemm_prefill dequantises the packed weight once into a bf16 (N, K) scratch matrix (35 MB for
// 6912 x 2560: it stays in the 126 MB L2) with the gather kernel of nb_unpack.cu, then runs the
// kernel below on X and that matrix.  Operands are bf16 (weights are the fp16 codebook entries
// rounded to bf16, as in the reference's any-M kernel, nativebit_jax/packed_kernel.py:151-159),
// products are accumulated in fp32.
//
// Kernel: one CTA per 128 x BN output tile (BN = 256 or 128), 192 threads:
//   warp 0   one lane issues TMA tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//            128 x 64 slab of X and a BN x 64 slab of W per k-step into a ring of shared-memory
//            stages, each completing on the stage's "full" mbarrier;
//   warp 1   allocates BN columns of tensor memory; one lane waits for a full stage and issues
//            four tcgen05.mma (M=128, N=BN, K=16) per stage from shared-memory descriptors, then
//            tcgen05.commit on the stage's "empty" barrier (and on the accumulator barrier at the end);
//   warps 2-5  epilogue: each warp owns one 32-lane quadrant of tensor memory, reads it with
//            tcgen05.ld (32 columns at a time), converts and stores its 32 rows of Y.
// Every mbarrier wait is bounded: after kSpinLimit probes the waiter raises a shared abort flag,
// writes NB_ERR_TIMEOUT to the status word and all roles fall through to the common exit, where
// tensor memory is freed.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <mutex>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

constexpr int kBM = 128, kBK = 64;
constexpr uint32_t kGemmSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s2u(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s2u(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(s2u(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and raises the abort flag) when it gives up or someone else did.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  for (uint32_t i = 0; i < kGemmSpinLimit; ++i) {
    if (bar_test(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicExch(status, (int)NB_ERR_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(s2u(dst)), "l"(map), "r"(s2u(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* p) {
  return (uint64_t)((s2u(p) & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s2u(bar)) : "memory");
}

template <int BN> struct GemmCfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kSmem = kStages * (kABytes + kBBytes) + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, void* __restrict__ y,
                 int y_dtype, int M, int N, int K, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + S * Cfg::kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + S * Cfg::kBBytes);
  uint64_t* empty = full + S;
  uint64_t* accum = empty + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * BN;
  const int KT = K / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { bar_init(&full[s], 1); bar_init(&empty[s], 1); }
    bar_init(accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (!bar_wait(&empty[s], ((kt / S) & 1) ^ 1, abort_flag, status)) break;
        bar_expect_tx(&full[s], Cfg::kABytes + Cfg::kBBytes);
        tma_load_2d(sA + s * Cfg::kABytes, &map_x, &full[s], kt * kBK, m0);
        tma_load_2d(sB + s * Cfg::kBBytes, &map_w, &full[s], kt * kBK, n0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      // instruction descriptor: fp32 accumulate, A and B bf16, both K-major, N = BN, M = 128
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      bool ok = true;
      for (int kt = 0; kt < KT && ok; ++kt) {
        const int s = kt % S;
        ok = bar_wait(&full[s], (kt / S) & 1, abort_flag, status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = smem_desc_sw128(sA + s * Cfg::kABytes), db = smem_desc_sw128(sB + s * Cfg::kBBytes);
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4)  // 16 bf16 = 32 bytes = 2 descriptor address units per step
          umma_bf16(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
        umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
      }
      umma_commit(accum);        // accumulator complete (or pipeline aborted: the epilogue checks the flag)
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +31 = rows m0 + 32*(w%4) + lane
    const int q = warp & 3;
    const bool ok = bar_wait(accum, 0, abort_flag, status) && !*abort_flag;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int m = m0 + q * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int n = n0 + c * 32;
        if (m < M && n < N) {
          if (y_dtype == NB_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(y) + (size_t)m * N + n;
            if (n + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                pk[j] = *reinterpret_cast<const uint32_t*>(&h);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            } else {
              for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* dst = reinterpret_cast<float*>(y) + (size_t)m * N + n;
            for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __uint_as_float(r[j]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// (rows, cols) row-major bf16 matrix -> tensor map with a (box_rows x 64) box and 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_last_error("cuTensorMapEncodeTiled is not available from the driver"); return NB_ERR_LAUNCH; }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[96];
    std::snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    set_last_error(msg);
    return NB_ERR_LAUNCH;
  }
  return NB_OK;
}

template <int BN>
static int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, void* y, int y_dtype, int M, int N, int K, int* status,
                       cudaStream_t st) {
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    if (cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmem))
      return record_cuda_error(e);
    attr_done[dev & 63] = true;
  }
  const dim3 grid((N + BN - 1) / BN, (M + kBM - 1) / kBM);
  gemm_bf16_kernel<BN><<<grid, 192, GemmCfg<BN>::kSmem, st>>>(mx, mw, y, y_dtype, M, N, K, status);
  return check_launch();
}

}  // namespace nb

using namespace nb;

extern "C" size_t nb_prefill_workspace_bytes(int M, int N, int K) {
  if (M < 1 || N < 1 || K < 1) return 0;
  return (size_t)N * K * 2 + 256;  // bf16 weight + status word
}

extern "C" int nb_gemm_bf16(const void* x, const void* w, int M, int N, int K, void* y, int y_dtype, int* status, void* stream) {
  if (!x || !w || !y || M < 1 || N < 1 || K < 1) return NB_ERR_ARG;
  if (y_dtype != NB_BF16 && y_dtype != NB_F32) return NB_ERR_ARG;
  if (K % kBK != 0) return NB_ERR_SHAPE;
  if ((uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 4) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const int bn = (N % 256 == 0 && (long)(N / 256) * ((M + kBM - 1) / kBM) >= sm_count()) ? 256 : 128;
  CUtensorMap mx, mw;
  if (int rc = make_map(&mx, x, M, K, kBM)) return rc;
  if (int rc = make_map(&mw, w, N, K, bn)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  return bn == 256 ? launch_gemm<256>(mx, mw, y, y_dtype, M, N, K, status, st)
                   : launch_gemm<128>(mx, mw, y, y_dtype, M, N, K, status, st);
}

extern "C" int nb_gemm_prefill(const void* x, int M, const uint8_t* packed, const void* codebook, int cb_dtype, int bits,
                               int block_size, int N, int K, void* y, int y_dtype, void* workspace, size_t workspace_bytes,
                               void* stream) {
  if (!x || !packed || !codebook || !y) return NB_ERR_ARG;
  if (!workspace || workspace_bytes < nb_prefill_workspace_bytes(M, N, K)) return NB_ERR_WORKSPACE;
  if ((uintptr_t)workspace % 256) return NB_ERR_ALIGN;
  if (K % kBK != 0 || K % block_size != 0) return NB_ERR_SHAPE;
  if (int rc = nb_dequant(packed, codebook, cb_dtype, bits, block_size, N, K, workspace, NB_BF16, stream)) return rc;
  int* status = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(workspace) + (size_t)N * K * 2);
  return nb_gemm_bf16(x, workspace, M, N, K, y, y_dtype, status, stream);
}

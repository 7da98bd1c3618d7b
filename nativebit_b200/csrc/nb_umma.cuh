// Building blocks of the tcgen05 / tensor-memory GEMM kernels (nb_gemm.cu, nb_gemm_fused.cu): mbarrier
// waits with a bound, TMA tile loads, shared-memory matrix descriptors, the MMA and commit wrappers, and
// the host-side tensor-map encoder.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <mutex>

#include "nb_common.cuh"
#include "nb_device.cuh"
#include "nb_host.h"

namespace nb {

constexpr int kBM = 128, kBK = 64;
constexpr uint32_t kGemmSpinLimit = 1u << 21;

__device__ __forceinline__ uint32_t s2u(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s2u(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s2u(bar)), "r"(bytes) : "memory");
}
// One probe of a barrier phase that may suspend the thread in hardware for up to about kBarSuspendNs
// before it answers: a waiting thread takes no issue slots and no shared-memory bandwidth from the threads
// that issue the copies and the MMAs.  (Probing with test_wait in a loop was measured to slow the single
// TMA and MMA lanes of a 704-thread CTA by a factor of five.)
constexpr uint32_t kBarSuspendNs = 1000;
__device__ __forceinline__ bool bar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(s2u(bar)), "r"(parity), "r"(kBarSuspendNs) : "memory");
  return ok != 0;
}

// Bounded wait; returns false (and raises the abort flag) when it gives up or someone else did.  The bound is
// kGemmSpinLimit probes: between 0.1 s (every probe answers at once) and a few seconds (every probe suspends
// for its full time), far beyond any kernel of this library.  kSleep > 0 adds a back-off between probes.
template <int kSleep = 0>
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  for (uint32_t i = 0; i < kGemmSpinLimit; ++i) {
    if (bar_test(bar, parity)) return true;
    if (kSleep > 0) __nanosleep(kSleep);
    if ((i & 63u) == 63u && *abort_flag) return false;
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

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s2u(bar)) : "memory");
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
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
inline int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
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

// fp32 -> two fp16 terms per element, hi = fp16(x) (saturating) and lo = fp16(x - hi), written as rows 2i and
// 2i+1 of a (2M, K) fp16 matrix: x = hi + lo to about 22 significant bits.  Eight elements per thread.
static __global__ void __launch_bounds__(256) f32_to_f16_pair_kernel(const float4* __restrict__ in, uint4* __restrict__ out, int M, int K) {
  const int k8 = K >> 3;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * k8) return;
  const int row = (int)(i / k8), c = (int)(i - (size_t)row * k8);
  const float4 a = in[2 * i], b = in[2 * i + 1];
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  uint32_t hi[4], lo[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    hi[j] = f32x2_to_f16x2_sat(v[2 * j], v[2 * j + 1]);
    const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&hi[j]));
    lo[j] = f32x2_to_f16x2_sat(v[2 * j] - h.x, v[2 * j + 1] - h.y);
  }
  out[(size_t)(2 * row) * k8 + c] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  out[(size_t)(2 * row + 1) * k8 + c] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}


}  // namespace nb

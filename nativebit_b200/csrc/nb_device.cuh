// Device-side building blocks shared by the decode kernels (nb_gemv.cu, nb_stream.cu): byte-permute
// table lookups, mbarrier and bulk-copy wrappers, the m16n8k16 tensor-core MMA, scoped loads and
// stores for flags, and dtype conversions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "nb_common.cuh"

namespace nb {

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Non-blocking probe of a barrier phase.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 16-byte asynchronous copy global -> shared (L2 only), and a deferred barrier arrival that fires
// once all earlier asynchronous copies of the executing thread have completed.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four table lookups: selector nibbles 0..3 of `sel` -> two registers of two fp16 weights.
// Up to 8 entries: T = {low-byte plane lo, low-byte plane hi, high-byte plane lo, high-byte plane hi}.
// 16 entries (4-bit): T[0..3] as above for entries 0..7, T[4..7] for entries 8..15; bit 3 of a nibble
// selects between the two halves through a byte mask (0xFF where the index is >= 8) that a permute
// of {0x00000000, 0xFFFFFFFF} produces from index >> 1.
template <int BITS>
__device__ __forceinline__ void lookup4(uint32_t sel, const uint32_t (&T)[BITS == 4 ? 8 : 4], uint32_t& r01, uint32_t& r23) {
  uint32_t lo, hi;
  if (BITS == 4) {
    const uint32_t s7 = sel & 0x7777u;
    const uint32_t m = prmt(0u, 0xFFFFFFFFu, (sel >> 1) & 0x7777u);
    const uint32_t lo0 = prmt(T[0], T[1], s7), lo1 = prmt(T[4], T[5], s7);
    const uint32_t hi0 = prmt(T[2], T[3], s7), hi1 = prmt(T[6], T[7], s7);
    lo = (lo0 & ~m) | (lo1 & m);
    hi = (hi0 & ~m) | (hi1 & m);
  } else {
    lo = prmt(T[0], T[1], sel);
    hi = prmt(T[2], T[3], sel);
  }
  r01 = prmt(lo, hi, 0x5140);
  r23 = prmt(lo, hi, 0x7362);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// One block's codebook (in shared memory) -> byte planes for lookup4; zero table if !valid.
template <int BITS>
__device__ __forceinline__ void make_table(const uint8_t* cb, int cb_dtype, bool valid, uint32_t (&T)[BITS == 4 ? 8 : 4]) {
  constexpr int kRegs = BITS == 4 ? 8 : 4;
  uint32_t e[kRegs];  // 2^BITS fp16 entries, two per register
#pragma unroll
  for (int i = 0; i < kRegs; ++i) e[i] = 0u;
  if (valid) {
    constexpr int kEntries = 1 << BITS;
    if (cb_dtype == NB_F16) {
      if (BITS == 2) {
        const uint2 v = *reinterpret_cast<const uint2*>(cb);
        e[0] = v.x; e[1] = v.y;
      } else {
#pragma unroll
        for (int i = 0; i < kEntries / 8; ++i) {
          const uint4 v = *reinterpret_cast<const uint4*>(cb + 16 * i);
          e[4 * i] = v.x; e[4 * i + 1] = v.y; e[4 * i + 2] = v.z; e[4 * i + 3] = v.w;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < kEntries / 4; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(cb + 16 * i);
        e[2 * i] = pack_half2(a.x, a.y); e[2 * i + 1] = pack_half2(a.z, a.w);
      }
    }
  }
  if (BITS == 2) {  // 4 entries: selector values 0..3 pick from the first operand
    T[0] = prmt(e[0], e[1], 0x6420); T[2] = prmt(e[0], e[1], 0x7531);
    T[1] = T[2]; T[3] = T[0];
  } else {
#pragma unroll
    for (int h = 0; h < kRegs / 4; ++h) {
      T[4 * h + 0] = prmt(e[4 * h], e[4 * h + 1], 0x6420); T[4 * h + 1] = prmt(e[4 * h + 2], e[4 * h + 3], 0x6420);
      T[4 * h + 2] = prmt(e[4 * h], e[4 * h + 1], 0x7531); T[4 * h + 3] = prmt(e[4 * h + 2], e[4 * h + 3], 0x7531);
    }
  }
}

template <int BITS>
__device__ __forceinline__ void read_block(const uint8_t* blk, uint32_t (&w)[Fmt<BITS>::kWords]) {
#pragma unroll
  for (int i = 0; i < Fmt<BITS>::kWords / 4; ++i) {
    const uint4 v = *reinterpret_cast<const uint4*>(blk + 16 * i);
    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
  }
}

__device__ __forceinline__ float load_x(const void* x, int dtype, size_t i) {
  if (dtype == NB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
  if (dtype == NB_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
  return reinterpret_cast<const float*>(x)[i];
}

// Eight consecutive activations (index i is a multiple of 8, pointer 16-byte aligned) as floats.
__device__ __forceinline__ void load_x8(const void* x, int dtype, size_t i, float (&v)[8]) {
  if (dtype == NB_F32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + i);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + i + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + i);
    const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dtype == NB_BF16) {
        v[2 * j] = __uint_as_float(u[j] << 16);
        v[2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[j]));
        v[2 * j] = f.x; v[2 * j + 1] = f.y;
      }
    }
  }
}

__device__ __forceinline__ void store_y(void* y, int dtype, size_t i, float v) {
  if (dtype == NB_BF16) reinterpret_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
  else if (dtype == NB_F16) reinterpret_cast<__half*>(y)[i] = __float2half_rn(v);
  else reinterpret_cast<float*>(y)[i] = v;
}

// {a, b} -> packed fp16 pair (a in the low half), round to nearest, saturating to +-65504.
__device__ __forceinline__ uint32_t f32x2_to_f16x2_sat(float a, float b) {
  uint32_t d;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}

__device__ __forceinline__ __half to_half_clamped(float v) {
  return __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
}

}  // namespace nb

// Fused decode GEMV / skinny GEMM for NativeBit packed linears on sm_100a (M = 1..16 rows).
//
// Work decomposition.  A "unit" is 16 output rows x 4 codebook blocks (512 input columns):
// lane (g, t) of a warp (g = lane/4, t = lane%4) owns the block of row g and the block of row
// g+8 at k-block 4*kgroup+t.  It loads the packed indices of its two blocks with 16-byte
// loads (48 bytes per 3-bit block) plus the two 16-byte codebooks, turns them into nibble
// selectors with a handful of mask operations (nb_common.cuh), and gathers four fp16 weights
// per byte-permute pair from a low-byte / high-byte plane of the codebook held in registers.
// Four weights of row g and four of row g+8 form the A fragment of one m16n8k16 tensor-core
// MMA whose B fragment is the matching four activations of up to 8 batch rows, so the
// multiply-accumulate (fp16 x fp16 products are exact, fp32 accumulation) costs one
// instruction per 256 weights and all remaining issue slots go to the unpack.  Because the
// weights are consumed in "slot" order rather than position order, the activation tile is
// staged into shared memory once per CTA in the same slot order (and as fp16).
//
// A CTA owns `tr` row tiles x one contiguous range of k-groups; its warps take units round
// robin and add their 16 x 8 partial tiles into a shared fp32 accumulator.  When the k range
// is split over several CTAs (grid.y > 1) each CTA writes its partial tile to scratch, takes a
// ticket, and the CTA that takes the last ticket adds the partials in fixed order, writes y and
// resets the ticket counter, so results are deterministic and the scratch needs no per-launch
// clearing.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kXBlockBytes = 32 * 8 * 8 + 32;  // one k-block of one 8-row activation tile, +32 B skew
constexpr int kMaxSmem = 200 * 1024;

struct GemvPlan {
  int tr;           // row tiles (of 16 rows) per CTA
  int parts;        // k partitions = grid.y
  int kg_per_part;  // k-groups (of 4 blocks) per partition
  int grid_x;
  size_t smem;
};

struct GemvParams {
  const void* x;
  const uint8_t* packed;
  const void* codebook;
  void* y;
  float* scratch;
  int* counters;
  int M, N, bpr, row_tiles, kgroups;
  int tr, kg_per_part;
  int x_dtype, y_dtype, cb_dtype;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four table lookups: selector nibbles 0..3 of `sel` -> two registers of two fp16 weights.
// T = {low-byte plane lo, low-byte plane hi, high-byte plane lo, high-byte plane hi}.
__device__ __forceinline__ void lookup4(uint32_t sel, const uint32_t (&T)[4], uint32_t& r01, uint32_t& r23) {
  const uint32_t lo = prmt(T[0], T[1], sel), hi = prmt(T[2], T[3], sel);
  r01 = prmt(lo, hi, 0x5140);
  r23 = prmt(lo, hi, 0x7362);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Loads one block's codebook and splits it into byte planes.  Invalid blocks get a zero table.
template <int BITS>
__device__ __forceinline__ void load_table(const void* codebook, int cb_dtype, size_t block, bool valid, uint32_t (&T)[4]) {
  uint32_t e0 = 0, e1 = 0, e2 = 0, e3 = 0;  // 2^BITS fp16 entries, two per register
  if (valid) {
    if (BITS == 3) {
      if (cb_dtype == NB_F16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(codebook) + block);
        e0 = v.x; e1 = v.y; e2 = v.z; e3 = v.w;
      } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>(codebook) + 2 * block);
        const float4 b = __ldg(reinterpret_cast<const float4*>(codebook) + 2 * block + 1);
        e0 = pack_half2(a.x, a.y); e1 = pack_half2(a.z, a.w); e2 = pack_half2(b.x, b.y); e3 = pack_half2(b.z, b.w);
      }
    } else {
      if (cb_dtype == NB_F16) {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(codebook) + block);
        e0 = v.x; e1 = v.y;
      } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>(codebook) + block);
        e0 = pack_half2(a.x, a.y); e1 = pack_half2(a.z, a.w);
      }
    }
  }
  if (BITS == 3) {
    T[0] = prmt(e0, e1, 0x6420); T[1] = prmt(e2, e3, 0x6420);
    T[2] = prmt(e0, e1, 0x7531); T[3] = prmt(e2, e3, 0x7531);
  } else {  // 4 entries: selector values 0..3 pick from the first operand
    T[0] = prmt(e0, e1, 0x6420); T[2] = prmt(e0, e1, 0x7531);
    T[1] = T[2]; T[3] = T[0];
  }
}

template <int BITS>
__device__ __forceinline__ void load_block(const uint8_t* packed, size_t block, bool valid, uint32_t (&w)[Fmt<BITS>::kWords]) {
  constexpr int kVec = Fmt<BITS>::kWords / 4;
  if (valid) {
    const uint4* p = reinterpret_cast<const uint4*>(packed + block * (size_t)(16 * BITS));
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const uint4 v = ldg_stream(p + i);
      w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < Fmt<BITS>::kWords; ++i) w[i] = 0;
  }
}

__device__ __forceinline__ float load_x(const void* x, int dtype, size_t i) {
  if (dtype == NB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
  if (dtype == NB_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
  return reinterpret_cast<const float*>(x)[i];
}

__device__ __forceinline__ void store_y(void* y, int dtype, size_t i, float v) {
  if (dtype == NB_BF16) reinterpret_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
  else if (dtype == NB_F16) reinterpret_cast<__half*>(y)[i] = __float2half_rn(v);
  else reinterpret_cast<float*>(y)[i] = v;
}

template <int BITS, int NT>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int kWords = Fmt<BITS>::kWords;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

  const int rt0 = blockIdx.x * p.tr;
  const int rt_n = min(p.tr, p.row_tiles - rt0);
  const int kg0 = blockIdx.y * p.kg_per_part;
  const int kg_n = min(p.kg_per_part, p.kgroups - kg0);
  const int kb0 = kg0 * 4;
  const int kb_n = min(kg_n * 4, p.bpr - kb0);
  const int n_units = rt_n * kg_n;
  const int K = p.bpr * kBlock;

  // shared memory carve-up
  const int x_tile_bytes = kg_n * 4 * kXBlockBytes;
  __half* xs = reinterpret_cast<__half*>(smem);
  float* acc = reinterpret_cast<float*>(smem + NT * x_tile_bytes);
  const int acc_n = p.tr * 16 * NT * 8;
  uint8_t* inv = reinterpret_cast<uint8_t*>(acc + acc_n);
  __shared__ int s_last;

  // First unit's loads go out before the activation tile is staged.
  uint32_t wa[kWords], wb[kWords], TA[4], TB[4];
  auto issue = [&](int u) {
    const int rtl = u / kg_n, kgl = u - rtl * kg_n;
    const int row_a = 16 * (rt0 + rtl) + g, row_b = row_a + 8;
    const int kb = kb0 + 4 * kgl + t;
    const bool vk = kb < p.bpr;
    const bool va = vk && row_a < p.N, vb = vk && row_b < p.N;
    const size_t ba = (size_t)row_a * p.bpr + kb, bb = (size_t)row_b * p.bpr + kb;
    load_block<BITS>(p.packed, ba, va, wa);
    load_block<BITS>(p.packed, bb, vb, wb);
    load_table<BITS>(p.codebook, p.cb_dtype, ba, va, TA);
    load_table<BITS>(p.codebook, p.cb_dtype, bb, vb, TB);
  };
  if (warp < n_units) issue(warp);

  if (tid < kBlock) inv[slot_to_position<BITS>(tid)] = (uint8_t)tid;
  for (int i = tid; i < acc_n; i += kGemvThreads) acc[i] = 0.f;
  __syncthreads();
  {
    // k-blocks past the end of the row (last k-group) are staged as zeros: their weights are
    // zero too, and 0 x garbage must not produce a NaN.
    const int per_row = kg_n * 4 * kBlock;
    for (int e = tid; e < p.M * per_row; e += kGemvThreads) {
      const int m = e / per_row, r = e - m * per_row;
      const int kbl = r >> 7, pos = r & 127;
      float v = 0.f;
      if (kbl < kb_n) v = load_x(p.x, p.x_dtype, (size_t)m * K + (size_t)kb0 * kBlock + r);
      v = fminf(fmaxf(v, -65504.f), 65504.f);
      const int slot = inv[pos];
      const int off = (m >> 3) * (x_tile_bytes / 2) + kbl * (kXBlockBytes / 2) + (slot >> 2) * 32 + (m & 7) * 4 + (slot & 3);
      xs[off] = __float2half_rn(v);
    }
  }
  __syncthreads();

  for (int u = warp; u < n_units; u += kGemvWarps) {
    const int rtl = u / kg_n, kgl = u - rtl * kg_n;
    float c[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f; }
    const uint8_t* xrow = smem + (4 * kgl + t) * kXBlockBytes + g * 8;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t UA[4], UB[4];
      group_selectors<BITS>(wa, q, UA);
      group_selectors<BITS>(wb, q, UB);
#pragma unroll
      for (int uu = 0; uu < 4; ++uu) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int s = 8 * q + 2 * uu + h;
          const uint32_t sa = h ? (UA[uu] >> 16) : UA[uu];
          const uint32_t sb = h ? (UB[uu] >> 16) : UB[uu];
          uint32_t a0, a1, a2, a3;
          lookup4(sa, TA, a0, a2);
          lookup4(sb, TB, a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint2 xb = *reinterpret_cast<const uint2*>(xrow + nt * x_tile_bytes + s * 64);
            mma_16816(c[nt], a0, a1, a2, a3, xb.x, xb.y);
          }
        }
      }
    }
    if (u + kGemvWarps < n_units) issue(u + kGemvWarps);
    float* arow = acc + (rtl * 16 + g) * (NT * 8) + 2 * t;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int n = nt * 8 + 2 * t;
      if (n < p.M) { atomicAdd(arow + nt * 8, c[nt][0]); atomicAdd(arow + 8 * NT * 8 + nt * 8, c[nt][2]); }
      if (n + 1 < p.M) { atomicAdd(arow + nt * 8 + 1, c[nt][1]); atomicAdd(arow + 8 * NT * 8 + nt * 8 + 1, c[nt][3]); }
    }
  }
  __syncthreads();

  const int rows_here = rt_n * 16;
  const int row0 = rt0 * 16;
  if (gridDim.y == 1) {
    for (int e = tid; e < p.M * rows_here; e += kGemvThreads) {
      const int m = e / rows_here, r = e - m * rows_here;
      if (row0 + r < p.N) store_y(p.y, p.y_dtype, (size_t)m * p.N + row0 + r, acc[r * (NT * 8) + m]);
    }
    return;
  }
  // split-K fix-up
  const int tile_elems = p.tr * 16 * p.M;
  float* mine = p.scratch + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * tile_elems;
  for (int e = tid; e < p.M * rows_here; e += kGemvThreads) {
    const int m = e / rows_here, r = e - m * rows_here;
    __stcg(mine + e, acc[r * (NT * 8) + m]);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(p.counters + blockIdx.x, 1);
    s_last = (ticket == (int)gridDim.y - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* base = p.scratch + (size_t)blockIdx.x * gridDim.y * tile_elems;
  for (int e = tid; e < p.M * rows_here; e += kGemvThreads) {
    const int m = e / rows_here, r = e - m * rows_here;
    float v = 0.f;
    for (int part = 0; part < (int)gridDim.y; ++part) v += __ldcg(base + (size_t)part * tile_elems + e);
    if (row0 + r < p.N) store_y(p.y, p.y_dtype, (size_t)m * p.N + row0 + r, v);
  }
  if (tid == 0) p.counters[blockIdx.x] = 0;
}

static size_t plan_smem(int tr, int kg_per_part, int nt) {
  return (size_t)nt * kg_per_part * 4 * kXBlockBytes + (size_t)tr * 16 * nt * 8 * 4 + kBlock + 16;
}

// Picks rows-per-CTA and the k split so that the grid is close to one full wave of CTAs with
// about one unit per warp.  cost = waves * (latency + ceil(units/warps)) + fix-up penalty.
static GemvPlan make_plan(int M, int N, int K, int sms) {
  const int nt = M > 8 ? 2 : 1;
  const int row_tiles = (N + 15) / 16, bpr = K / kBlock, kgroups = (bpr + 3) / 4;
  GemvPlan best{};
  double best_cost = 1e30;
  for (int parts_req = 1; parts_req <= std::min(kgroups, 32); ++parts_req) {
    const int kgp = (kgroups + parts_req - 1) / parts_req;
    const int parts = (kgroups + kgp - 1) / kgp;
    if (parts != parts_req) continue;
    for (int tr = 1; tr <= std::min(row_tiles, 64); ++tr) {
      const size_t smem = plan_smem(tr, kgp, nt);
      if (smem > (size_t)kMaxSmem) break;
      const int gx = (row_tiles + tr - 1) / tr;
      const long ctas = (long)gx * parts;
      const long waves = (ctas + sms - 1) / sms;
      const int rounds = (tr * kgp + kGemvWarps - 1) / kGemvWarps;
      double cost = waves * (1.5 + rounds) + (parts > 1 ? 0.4 + 0.02 * parts : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = GemvPlan{tr, parts, kgp, gx, smem};
      }
    }
  }
  return best;
}

static size_t plan_workspace(const GemvPlan& pl, int M) {
  const size_t counters = ((size_t)pl.grid_x * sizeof(int) + 255) / 256 * 256;
  const size_t scratch = pl.parts > 1 ? (size_t)pl.grid_x * pl.parts * pl.tr * 16 * M * sizeof(float) : 0;
  return counters + scratch;
}

template <int BITS, int NT>
static int launch(const GemvParams& prm, const GemvPlan& pl, cudaStream_t st) {
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<BITS, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return record_cuda_error(e);
    attr_done[dev & 63] = true;
  }
  gemv_kernel<BITS, NT><<<dim3(pl.grid_x, pl.parts), kGemvThreads, pl.smem, st>>>(prm);
  return check_launch();
}

}  // namespace nb

using namespace nb;

static int gemv_check_shape(int M, int N, int K, int bits, int block_size) {
  if (M < 1 || N < 1 || K < 1) return NB_ERR_ARG;
  if (bits != 2 && bits != 3) return NB_ERR_SHAPE;
  if (block_size != kBlock) return NB_ERR_SHAPE;
  if (M > 16 || K % kBlock != 0) return NB_ERR_SHAPE;
  return NB_OK;
}

extern "C" size_t nb_gemv_workspace_bytes(int M, int N, int K, int bits, int block_size) {
  if (gemv_check_shape(M, N, K, bits, block_size) != NB_OK) return 0;
  return plan_workspace(make_plan(M, N, K, sm_count()), M);
}

extern "C" int nb_gemv(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                       int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
                       size_t workspace_bytes, void* stream) {
  if (!x || !packed || !codebook || !y) return NB_ERR_ARG;
  if (x_dtype < NB_F32 || x_dtype > NB_BF16 || y_dtype < NB_F32 || y_dtype > NB_BF16) return NB_ERR_ARG;
  if (cb_dtype != NB_F16 && cb_dtype != NB_F32) return NB_ERR_ARG;
  if (int rc = gemv_check_shape(M, N, K, bits, block_size)) return rc;
  if ((uintptr_t)packed % 16 || (uintptr_t)codebook % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const GemvPlan pl = make_plan(M, N, K, sm_count());
  const size_t need = plan_workspace(pl, M);
  if (pl.parts > 1 && (!workspace || workspace_bytes < need)) return NB_ERR_WORKSPACE;
  if (pl.parts > 1 && (uintptr_t)workspace % 16) return NB_ERR_ALIGN;

  GemvParams prm{};
  prm.x = x; prm.packed = packed; prm.codebook = codebook; prm.y = y;
  const size_t counters = ((size_t)pl.grid_x * sizeof(int) + 255) / 256 * 256;
  prm.counters = reinterpret_cast<int*>(workspace);
  prm.scratch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + counters);
  prm.M = M; prm.N = N; prm.bpr = K / kBlock; prm.row_tiles = (N + 15) / 16; prm.kgroups = (prm.bpr + 3) / 4;
  prm.tr = pl.tr; prm.kg_per_part = pl.kg_per_part;
  prm.x_dtype = x_dtype; prm.y_dtype = y_dtype; prm.cb_dtype = cb_dtype;
  cudaStream_t st = (cudaStream_t)stream;
  if (bits == 3) return M > 8 ? launch<3, 2>(prm, pl, st) : launch<3, 1>(prm, pl, st);
  return M > 8 ? launch<2, 2>(prm, pl, st) : launch<2, 1>(prm, pl, st);
}

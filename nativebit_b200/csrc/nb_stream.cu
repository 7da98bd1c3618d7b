// Persistent multi-matrix decode kernel for NativeBit packed linears on sm_100a.
//
// One launch executes a PROGRAM: a list of operations (packed matvecs with their activation
// prologues, single-query attention, the LM head, the greedy argmax) over one CTA per SM.  The
// reference runs the same sequence as ~400 library launches per token with a host round trip
// (inference/generate_torch.py:150-162 forward, :307-311 token loop; inference/cuda_kernel.py:38-104 the
// matvec); a launch per matvec leaves every kernel on a fixed latency floor of several microseconds,
// several times the 1.4 us its bytes take to stream.  Here:
//
//  * Weight stream.  Packed weights are held in a tile-major "stream layout" (nb_stream_pack, built
//    once at load time): a unit is 16 output rows x one 128-weight codebook block = the 32 lanes' index
//    words followed by the 16 rows' byte-plane lookup tables, 1 KB at 3 bits, and the units of a matrix
//    are consecutive.  Every operation's units are split evenly over CTAs and, inside a CTA, over its
//    16 warps as contiguous runs, so a warp's share of a matrix is one contiguous byte range.  Each warp
//    owns a private ring of shared-memory stages that it fills itself with bulk copies (cp.async.bulk,
//    one lane, completion on an mbarrier): the refill of a stage is issued the moment the warp has
//    consumed it, and the sequence of chunks runs on across operation boundaries, because weights
//    never depend on earlier results.  About 128 KB of weights per SM are in flight or resident at
//    all times, which covers the dependency waits between operations.
//  * Compute.  Lane (g, t) of a warp unpacks 32 weights of row g and 32 of row g+8 of the unit
//    (selector words + byte-permute table lookups, nb_common.cuh) and feeds them, four per row at a
//    time, as the A fragment of an m16n8k16 fp16 tensor-core MMA whose B fragment is the matching four
//    activations; fp32 activations are carried as two fp16 terms.  Partial sums of a warp's run are
//    kept per row tile, stored to a per-warp slot in shared memory and added in warp order.
//  * Dependencies.  After an operation a CTA publishes a sequence number in its flag word; an
//    operation that consumes the previous one's results first waits (bounded) until every CTA's flag has
//    reached that number.  No atomics on values: a row tile that straddles two CTAs is written as two
//    partial "slots" which the consumer adds in a fixed order, so results are bit-identical from run to
//    run.  The residual stream lives in every CTA's shared memory and never travels.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cfloat>
#include <cstdio>
#include <cstring>

#include "nb_common.cuh"
#include "nb_device.cuh"
#include "nb_host.h"

namespace nb {

constexpr int kSW = 16;                                   // warps per CTA
constexpr int kSThreads = kSW * 32;
constexpr int kChunkBytes = 2048;                         // one ring stage
constexpr int kStages = 4;                                // stages per warp
constexpr int kRingBytes = kSW * kStages * kChunkBytes;   // 128 KB
constexpr int kMaxOps = 160;
constexpr int kMaxKBlocks = 56;                           // K <= 7168
constexpr int kXSegBytes = 72;                            // 32 halves of one (k-block, lane t) + skew
constexpr int kXTermBytes = kMaxKBlocks * 4 * kXSegBytes; // 15.75 KB per fp16 term
constexpr int kMaxC = 3072;                               // residual width
constexpr int kRedHalf = 2048;                            // floats: 8 local row tiles x 16 warps x 16 rows
constexpr int kMaxCtas = 256;
constexpr uint32_t kCopySpin = 1u << 22;
constexpr uint32_t kFlagSpinDefault = 1u << 22;

using StreamOp = nb_stream_op;

// What the weight stream needs to know about an operation, computed once per launch.
struct OpInfo {
  int cta_a, cta_b;           // this CTA's unit range
  int bpr;                    // units per row tile (GEMV: k-blocks per row; head: pieces per row)
  uint16_t ubytes;            // bytes of a unit (GEMV) or of a full piece (head)
  uint8_t per_chunk, kind;
  const uint8_t* w;           // first unit
  int row_bytes;              // head: bytes of a table row
  int flags;                  // bit 0: the next operation waits for this one (or it is the last)
};
static_assert(sizeof(OpInfo) == 32, "OpInfo layout");

// shared-memory layout (dynamic)
constexpr int kOffRing = 0;
constexpr int kOffInfo = kOffRing + kRingBytes;
constexpr int kOffX = kOffInfo + kMaxOps * (int)sizeof(OpInfo);
constexpr int kOffH = kOffX + 2 * kXTermBytes;
constexpr int kOffRed = kOffH + kMaxC * 4;
constexpr int kOffDst = kOffRed + 2 * kRedHalf * 4;
constexpr int kOffOp = kOffDst + 256;
constexpr int kStreamSmem = kOffOp + 2 * (int)sizeof(StreamOp);
static_assert(sizeof(StreamOp) == 160, "nb_stream_op layout");
static_assert(kStreamSmem <= 226 * 1024, "shared memory budget");

template <int BITS> struct UnitFmt {
  static constexpr int kW = Fmt<BITS>::kWords / 4;          // words of one lane's 32 indices
  static constexpr int kIdxBytes = kW * 256;                // 32 lanes x 2 rows x kW words
  static constexpr int kTabBytes = BITS == 4 ? 32 : 16;     // one row's lookup table
  static constexpr int kBytes = kIdxBytes + 16 * kTabBytes; // 1024 at 3 bits, 768 at 2, 1536 at 4
};

__host__ __device__ inline int unit_bytes(int bits) { return bits == 3 ? UnitFmt<3>::kBytes : bits == 2 ? UnitFmt<2>::kBytes : UnitFmt<4>::kBytes; }

// ---- work split (32-bit arithmetic: the host refuses programs where units * (CTAs + 1) >= 2^31) ----
// [lo, hi) of part `i` of `parts` equal shares of n items.
__host__ __device__ inline void share(int n, int parts, int i, int& lo, int& hi) {
  lo = (int)((unsigned)n * (unsigned)i / (unsigned)parts);
  hi = (int)((unsigned)n * (unsigned)(i + 1) / (unsigned)parts);
}
// CTA that owns unit u when U units are split over G CTAs by share().
__host__ __device__ inline int cta_of_unit(int u, int U, int G) { return (int)(((unsigned)(u + 1) * (unsigned)G - 1u) / (unsigned)U); }

struct OpGeom {
  int kind, bits, bpr, rt, align, ubytes, per_chunk, units;
  int head_piece_bytes, head_row_bytes;
};

__host__ __device__ inline OpGeom geom_of(const StreamOp& o) {
  OpGeom g{};
  g.kind = o.kind;
  if (o.kind == NB_SOP_GEMV) {
    g.bits = o.i[2];
    g.bpr = o.i[1] / kBlock;
    g.rt = (o.i[0] + 15) / 16;
    g.align = (o.flags & NB_SOPF_ALIGN) ? 1 : 0;
    g.ubytes = unit_bytes(g.bits);
    g.per_chunk = kChunkBytes / g.ubytes;
    g.units = g.rt * g.bpr;
  } else if (o.kind == NB_SOP_HEAD) {
    g.head_row_bytes = o.i[1] * 2;
    g.bpr = (g.head_row_bytes + kChunkBytes - 1) / kChunkBytes;          // pieces per row
    g.head_piece_bytes = ((g.head_row_bytes / g.bpr + 15) / 16) * 16;
    g.ubytes = g.head_piece_bytes;
    g.rt = o.i[0];                                                       // rows
    g.align = 1;
    g.per_chunk = 1;
    g.units = g.rt * g.bpr;
  }
  return g;
}

// Unit range of a CTA in an operation; empty for operations without a weight stream.
__host__ __device__ inline void cta_range(const OpGeom& g, int cta, int G, int& a, int& b) {
  a = b = 0;
  if (g.units == 0) return;
  if (g.align) {
    int r0, r1;
    share(g.rt, G, cta, r0, r1);
    a = r0 * g.bpr; b = r1 * g.bpr;
  } else {
    share(g.units, G, cta, a, b);
  }
}
// A warp's part of its CTA's range: equal shares of the units (of whole rows for the head).
__host__ __device__ inline void warp_part(int kind, int bpr, int cta_a, int cta_b, int warp, int& a, int& b) {
  if (kind == NB_SOP_HEAD) {
    const int rows = (cta_b - cta_a) / bpr;
    a = cta_a + (rows * warp / kSW) * bpr;
    b = cta_a + (rows * (warp + 1) / kSW) * bpr;
  } else {
    const int n = cta_b - cta_a;
    a = cta_a + n * warp / kSW;
    b = cta_a + n * (warp + 1) / kSW;
  }
}

// ---- small device helpers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum of CTA-wide values in a fixed order (warp shuffles, then the warps' results in index order).
__device__ __forceinline__ float block_sum(float v, float* s16, int tid) {
  v = warp_sum_f(v);
  __syncthreads();
  if ((tid & 31) == 0) s16[tid >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kSW; ++i) t += s16[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* s16, int tid) {
  v = warp_max_f(v);
  __syncthreads();
  if ((tid & 31) == 0) s16[tid >> 5] = v;
  __syncthreads();
  float t = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < kSW; ++i) t = fmaxf(t, s16[i]);
  return t;
}

// Four consecutive activations (positions 4*i4 .. 4*i4+3 of the row) -> fp16 hi (+ lo) terms in slot order.
template <int XS>
__device__ __forceinline__ void stage4(uint8_t* x_s, const uint16_t* dst_off, int i4, float u0, float u1, float u2, float u3) {
  const int kb = i4 >> 5;                       // 32 groups of four per k-block
  const uint2 o2 = *reinterpret_cast<const uint2*>(dst_off + ((i4 & 31) << 2));
  uint16_t* blk = reinterpret_cast<uint16_t*>(x_s + kb * 4 * kXSegBytes);
  const uint32_t h01 = f32x2_to_f16x2_sat(u0, u1), h23 = f32x2_to_f16x2_sat(u2, u3);
  blk[o2.x & 0xFFFFu] = (uint16_t)(h01 & 0xFFFFu); blk[o2.x >> 16] = (uint16_t)(h01 >> 16);
  blk[o2.y & 0xFFFFu] = (uint16_t)(h23 & 0xFFFFu); blk[o2.y >> 16] = (uint16_t)(h23 >> 16);
  if (XS == 2) {
    const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
    const float2 r23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
    const uint32_t l01 = f32x2_to_f16x2_sat(fminf(fmaxf(u0, -65504.f), 65504.f) - r01.x, fminf(fmaxf(u1, -65504.f), 65504.f) - r01.y);
    const uint32_t l23 = f32x2_to_f16x2_sat(fminf(fmaxf(u2, -65504.f), 65504.f) - r23.x, fminf(fmaxf(u3, -65504.f), 65504.f) - r23.y);
    uint16_t* lo = blk + kXTermBytes / 2;
    lo[o2.x & 0xFFFFu] = (uint16_t)(l01 & 0xFFFFu); lo[o2.x >> 16] = (uint16_t)(l01 >> 16);
    lo[o2.y & 0xFFFFu] = (uint16_t)(l23 & 0xFFFFu); lo[o2.y >> 16] = (uint16_t)(l23 >> 16);
  }
}

// ---- the per-warp weight stream ------------------------------------------------------------------
// Both cursors walk the same sequence of chunks: for every operation with a weight stream, this
// warp's unit range cut into pieces of at most per_chunk units.  `fetch` runs up to kStages chunks
// ahead of `use`.
struct Cursor {
  int op;          // operation index (n_ops when exhausted)
  int u, u_end;    // next unit and end of the warp's range in that operation
  uint32_t count;  // chunks passed so far: stage = count % kStages, phase = (count / kStages) & 1
};

struct StreamCtx {
  const OpInfo* info;    // in shared memory
  int n_ops, warp, lane;
  uint8_t* ring;         // this warp's kStages stages
  uint64_t* full;        // this warp's kStages barriers
  int* status;
  bool dead;             // a copy wait of this warp ran out: later waits are not repeated
};

__device__ __forceinline__ void cursor_seek(const StreamCtx& c, Cursor& k) {   // skip to the next non-empty range
  while (k.op < c.n_ops && k.u >= k.u_end) {
    ++k.op;
    if (k.op < c.n_ops) {
      const OpInfo& f = c.info[k.op];
      if (f.cta_b > f.cta_a) warp_part(f.kind, f.bpr, f.cta_a, f.cta_b, c.warp, k.u, k.u_end);
    }
  }
}

__device__ __forceinline__ void cursor_init(const StreamCtx& c, Cursor& k) {
  k.op = -1; k.u = 0; k.u_end = 0; k.count = 0;
  cursor_seek(c, k);
}

// Units and bytes of the chunk at the cursor, and its source address.
__device__ __forceinline__ int chunk_at(const StreamCtx& c, const Cursor& k, const uint8_t*& src, uint32_t& bytes) {
  const OpInfo& f = c.info[k.op];
  if (f.kind == NB_SOP_HEAD) {
    const int row = k.u / f.bpr, piece = k.u - row * f.bpr;
    const int off = piece * f.ubytes;
    bytes = (uint32_t)min((int)f.ubytes, f.row_bytes - off);
    src = f.w + (size_t)row * f.row_bytes + off;
    return 1;
  }
  const int n = min((int)f.per_chunk, k.u_end - k.u);
  bytes = (uint32_t)(n * f.ubytes);
  src = f.w + (size_t)k.u * f.ubytes;
  return n;
}

// Request the chunk at the fetch cursor into its stage (if any is left); lane 0 issues the copy.
__device__ __forceinline__ void fetch_next(const StreamCtx& c, Cursor& f) {
  if (f.op >= c.n_ops) return;
  const uint8_t* src;
  uint32_t bytes;
  const int n = chunk_at(c, f, src, bytes);
  const int s = f.count % kStages;
  if (c.lane == 0) {
    mbar_arrive_expect_tx(&c.full[s], bytes);
    bulk_g2s(c.ring + s * kChunkBytes, src, bytes, &c.full[s]);
  }
  f.u += n;
  ++f.count;
  cursor_seek(c, f);
}

// Bounded wait for the chunk at the use cursor; returns its stage.
__device__ __forceinline__ const uint8_t* wait_chunk(StreamCtx& c, const Cursor& k) {
  const int s = k.count % kStages;
  const uint32_t parity = (k.count / kStages) & 1u;
  uint32_t spins = 0;
  while (!c.dead && !mbar_try_wait(&c.full[s], parity)) {
    __nanosleep(32);
    if (++spins > kCopySpin) {
      if (c.status) atomicExch(c.status, (int)NB_ERR_TIMEOUT);
      c.dead = true;
    }
  }
  return c.ring + s * kChunkBytes;
}

// ---- one unit: 16 rows x 128 weights against the staged activations -----------------------------
template <int BITS, int XS>
__device__ __forceinline__ void unit_mma(const uint8_t* ub, const uint8_t* x_s, int kb, int lane, float (&c)[2][4]) {
  using F = UnitFmt<BITS>;
  const int g = lane >> 2, t = lane & 3;
  uint32_t w[2 * F::kW];
#pragma unroll
  for (int j = 0; j < F::kW; ++j) {
    const uint2 v = *reinterpret_cast<const uint2*>(ub + j * 256 + lane * 8);
    w[2 * j] = v.x; w[2 * j + 1] = v.y;
  }
  uint32_t TA[BITS == 4 ? 8 : 4], TB[BITS == 4 ? 8 : 4];
  const uint8_t* tab = ub + F::kIdxBytes;
#pragma unroll
  for (int j = 0; j < F::kTabBytes / 16; ++j) {
    const uint4 a = *reinterpret_cast<const uint4*>(tab + g * F::kTabBytes + 16 * j);
    const uint4 b = *reinterpret_cast<const uint4*>(tab + (g + 8) * F::kTabBytes + 16 * j);
    TA[4 * j] = a.x; TA[4 * j + 1] = a.y; TA[4 * j + 2] = a.z; TA[4 * j + 3] = a.w;
    TB[4 * j] = b.x; TB[4 * j + 1] = b.y; TB[4 * j + 2] = b.z; TB[4 * j + 3] = b.w;
  }
  uint32_t UA[4], UB[4];
  if (BITS == 3) {
    selectors3(w[0], w[1], w[2], UA);
    selectors3(w[3], w[4], w[5], UB);
  } else if (BITS == 2) {
    selectors2(w[0], w[1], UA);
    selectors2(w[2], w[3], UB);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) { UA[j] = w[j]; UB[j] = w[4 + j]; }
  }
  const uint8_t* xseg = x_s + (kb * 4 + t) * kXSegBytes;
#pragma unroll
  for (int uu = 0; uu < 4; ++uu) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int s = 2 * uu + h;
      const uint32_t sa = h ? (UA[uu] >> 16) : UA[uu];
      const uint32_t sb = h ? (UB[uu] >> 16) : UB[uu];
      uint32_t a0, a1, a2, a3;
      lookup4<BITS>(sa, TA, a0, a2);
      lookup4<BITS>(sb, TB, a1, a3);
#pragma unroll
      for (int xs = 0; xs < XS; ++xs) {
        const uint2 xb = *reinterpret_cast<const uint2*>(xseg + xs * kXTermBytes + s * 8);
        mma_16816(c[h], a0, a1, a2, a3, xb.x, xb.y);
      }
    }
  }
}

// This warp's run of units of a packed matvec: streams the chunks, accumulates per row tile, stores
// the partial sums of every row tile it touched into its slot of `red` ([local row tile][warp][16]).
template <int BITS, int XS>
__device__ __forceinline__ void run_units(StreamCtx& c, Cursor& use, Cursor& fetch, int op_index, const uint8_t* x_s, float* red,
                                          int rt_first) {
  using F = UnitFmt<BITS>;
  const int lane = c.lane;
  if (use.op != op_index) return;
  const int bpr = c.info[op_index].bpr, per_chunk = c.info[op_index].per_chunk;
  float acc[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  int rt = use.u / bpr, kb = use.u - rt * bpr;
  while (use.op == op_index) {
    const uint8_t* st = wait_chunk(c, use);
    const int n = min(per_chunk, use.u_end - use.u);
    for (int j = 0; j < n; ++j) {
      unit_mma<BITS, XS>(st + j * F::kBytes, x_s, kb, lane, acc);
      if (++kb == bpr || (j == n - 1 && use.u + n == use.u_end)) {   // row tile (or this warp's part of it) complete
        if ((lane & 3) == 0) {
          float* dst = red + ((rt - rt_first) * kSW + c.warp) * 16;
          dst[lane >> 2] = acc[0][0] + acc[1][0];
          dst[(lane >> 2) + 8] = acc[0][2] + acc[1][2];
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
        if (kb == bpr) { kb = 0; ++rt; }
      }
    }
    use.u += n;
    ++use.count;
    cursor_seek(c, use);
    __syncwarp();               // every lane has consumed the stage before it is overwritten
    fetch_next(c, fetch);
  }
}

// ---- dependency flags ----------------------------------------------------------------------------
// Every CTA's flag must have reached `target` (sequence numbers only grow; compared as signed differences).
__device__ __forceinline__ void wait_flags(const uint32_t* flags, int G, uint32_t target, uint32_t spin_limit, int* status, int tid) {
  for (int i = tid; i < G; i += kSThreads) {
    uint32_t spins = (*reinterpret_cast<volatile int*>(status) == (int)NB_ERR_TIMEOUT) ? spin_limit : 0;  // a wait that ran out is not repeated
    while ((int)(ld_acquire_gpu_u32(flags + i) - target) < 0) {
      __nanosleep(20);
      if (++spins > spin_limit) {
        atomicExch(status, (int)NB_ERR_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
}

#ifdef NB_STREAM_TRACE
__device__ unsigned long long nb_stream_trace_buf[kMaxOps * 8];
#define NB_STRACE(op, i)                                                     \
  do {                                                                       \
    if (blockIdx.x == 0 && threadIdx.x == 0) {                               \
      unsigned long long t_;                                                 \
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                  \
      nb_stream_trace_buf[(op) * 8 + (i)] = t_;                              \
    }                                                                        \
  } while (0)
#else
#define NB_STRACE(op, i) do {} while (0)
#endif

// ---- the kernel -----------------------------------------------------------------------------------
// state: [0 .. kMaxCtas) flags, [kMaxCtas] epoch, [kMaxCtas + 1] status.
template <int BITS>
__global__ void __launch_bounds__(kSThreads, 1) stream_kernel(const StreamOp* __restrict__ ops_g, int n_ops, uint32_t* state, uint32_t spin_limit) {
  extern __shared__ __align__(128) uint8_t smem[];
  OpInfo* info = reinterpret_cast<OpInfo*>(smem + kOffInfo);
  uint8_t* x_s = smem + kOffX;
  float* h_s = reinterpret_cast<float*>(smem + kOffH);
  float* red_base = reinterpret_cast<float*>(smem + kOffRed);
  uint16_t* dst_off = reinterpret_cast<uint16_t*>(smem + kOffDst);
  StreamOp* op_slots = reinterpret_cast<StreamOp*>(smem + kOffOp);
  __shared__ __align__(8) uint64_t bars[kSW * kStages];
  __shared__ float s16[kSW];
  __shared__ float s_scale[2];
  __shared__ float s_best[kSW];
  __shared__ int s_besti[kSW];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  uint32_t* flags = state;
  int* status = reinterpret_cast<int*>(state + kMaxCtas + 1);
  const uint32_t base = state[kMaxCtas];      // sequence numbers of this launch start above the previous launch's

  for (int i = tid; i < n_ops; i += kSThreads) {
    const StreamOp& o = ops_g[i];
    const OpGeom g = geom_of(o);
    OpInfo f;
    cta_range(g, cta, G, f.cta_a, f.cta_b);
    f.bpr = g.bpr > 0 ? g.bpr : 1;
    f.ubytes = (uint16_t)g.ubytes;
    f.per_chunk = (uint8_t)g.per_chunk;
    f.kind = (uint8_t)g.kind;
    f.w = reinterpret_cast<const uint8_t*>(o.p[0]);
    f.row_bytes = g.head_row_bytes;
    f.flags = (i + 1 == n_ops || (ops_g[i + 1].flags & NB_SOPF_WAIT_PREV)) ? 1 : 0;
    info[i] = f;
  }
  for (int i = tid; i < (int)(sizeof(StreamOp) / 4) * min(n_ops, 2); i += kSThreads)
    reinterpret_cast<uint32_t*>(op_slots)[i] = reinterpret_cast<const uint32_t*>(ops_g)[i];
  if (tid < kSW * kStages) mbar_init(&bars[tid], 1);
  if (tid < kBlock) {
    // position inside a 128-weight block -> offset (in halves) of its activation inside the block's four segments
    const int slot = tid, pos = slot_to_position<BITS>(slot);
    dst_off[pos] = (uint16_t)((slot >> 5) * (kXSegBytes / 2) + (slot & 31));
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  StreamCtx ctx{info, n_ops, warp, lane, smem + kOffRing + warp * kStages * kChunkBytes, &bars[warp * kStages], status, false};
  Cursor fetch, use;
  cursor_init(ctx, fetch);
  cursor_init(ctx, use);
  for (int s = 0; s < kStages; ++s) fetch_next(ctx, fetch);

  for (int oi = 0; oi < n_ops; ++oi) {
    const StreamOp& op = op_slots[oi & 1];
    const uint32_t seq = base + (uint32_t)oi + 1u;     // published after this operation
    if (oi > 0 && (op.flags & NB_SOPF_WAIT_PREV)) wait_flags(flags, G, seq - 1u, spin_limit, status, tid);
    NB_STRACE(oi, 0);
    // the descriptor after the next one is fetched into the slot of the operation that just ended
    auto prefetch_op = [&]() {
      if (oi >= 1 && oi + 1 < n_ops && tid < (int)(sizeof(StreamOp) / 4))
        reinterpret_cast<uint32_t*>(&op_slots[(oi + 1) & 1])[tid] = __ldg(reinterpret_cast<const uint32_t*>(ops_g + oi + 1) + tid);
    };

    if (op.kind == NB_SOP_GEMV) {
      const int N = op.i[0], K = op.i[1];
      const int bpr = info[oi].bpr, cta_a = info[oi].cta_a, cta_b = info[oi].cta_b;
      const int rt_first = cta_a / bpr;
      const int n_rt = cta_b > cta_a ? (cta_b - 1) / bpr - rt_first + 1 : 0;
      float* red = red_base + (oi & 1) * kRedHalf;
      for (int i = tid; i < n_rt * kSW * 16; i += kSThreads) red[i] = 0.f;

      // ---- stage the activations
      int xs_terms = 1;
      if (!(op.flags & NB_SOPF_REUSE_X)) {
        if (op.pro == NB_SPRO_VEC) {
          const int dt = op.i[3];
          xs_terms = dt == NB_F32 ? 2 : 1;
          for (int i4 = tid; i4 < K / 4; i4 += kSThreads) {
            float v[4];
            if (dt == NB_F32) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(op.p[1]) + i4);
              v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            } else {
              const uint2 r = __ldcg(reinterpret_cast<const uint2*>(op.p[1]) + i4);
              if (dt == NB_BF16) {
                v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
                v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
              } else {
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
                v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
              }
            }
            if (dt == NB_F32) stage4<2>(x_s, dst_off, i4, v[0], v[1], v[2], v[3]);
            else stage4<1>(x_s, dst_off, i4, v[0], v[1], v[2], v[3]);
          }
          if (tid == 0) s_scale[oi & 1] = 1.f;
        } else if (op.pro == NB_SPRO_EMBED_NORM || op.pro == NB_SPRO_ADD_NORM) {
          // residual: h = table[token] (first layer) or h += sum of the previous projection's partial slots;
          // activation = h * weight, the factor 1/rms (a scalar) is applied to the outputs
          xs_terms = 2;
          const float4* w4 = reinterpret_cast<const float4*>(op.p[3]);
          float ss = 0.f;
          for (int i4 = tid; i4 < K / 4; i4 += kSThreads) {
            float4 h;
            if (op.pro == NB_SPRO_EMBED_NORM) {
              const long long tok = *reinterpret_cast<const long long*>(op.p[2]);
              const uint2 r = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(op.p[1]) + (size_t)tok * K) + i4);
              h = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u), __uint_as_float(r.y << 16),
                              __uint_as_float(r.y & 0xFFFF0000u));
            } else {
              h = reinterpret_cast<const float4*>(h_s)[i4];
              float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int sl = 0; sl < op.i[5]; ++sl) {
                const float4 e = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.p[1]) + (size_t)sl * op.i[7]) + i4);
                d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
              }
              h.x += d.x; h.y += d.y; h.z += d.z; h.w += d.w;
            }
            reinterpret_cast<float4*>(h_s)[i4] = h;
            ss += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
            const float4 w = __ldg(w4 + i4);
            stage4<2>(x_s, dst_off, i4, h.x * w.x, h.y * w.y, h.z * w.z, h.w * w.w);
          }
          const float tot = block_sum(ss, s16, tid);
          if (tid == 0) s_scale[oi & 1] = 1.0f / sqrtf(tot / (float)K + op.f[0]);
        } else if (op.pro == NB_SPRO_ATTN_MERGE) {
          // activations = attention output: per head, the splits' partial softmax numerators and
          // denominators merged; columns outside this rank's heads are zero
          xs_terms = 2;
          const int Hl = op.i[9], S = op.i[10], hd = op.i[11], col0 = op.i[12];
          const float* part = reinterpret_cast<const float*>(op.p[1]);
          for (int i4 = tid; i4 < K / 4; i4 += kSThreads) {
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int col = 4 * i4 + e - col0;
              float r = 0.f;
              if (col >= 0 && col < Hl * hd) {
                const int h = col / hd, d = col - h * hd;
                const float* ph = part + (size_t)h * S * (hd + 2);
                float mx = -FLT_MAX;
                for (int s = 0; s < S; ++s) mx = fmaxf(mx, __ldcg(ph + s * (hd + 2) + hd));
                float num = 0.f, den = 0.f;
                for (int s = 0; s < S; ++s) {
                  const float wgt = __expf(__ldcg(ph + s * (hd + 2) + hd) - mx);
                  num += wgt * __ldcg(ph + s * (hd + 2) + d);
                  den += wgt * __ldcg(ph + s * (hd + 2) + hd + 1);
                }
                r = num / den;
              }
              v[e] = r;
            }
            stage4<2>(x_s, dst_off, i4, v[0], v[1], v[2], v[3]);
          }
          if (tid == 0) s_scale[oi & 1] = 1.f;
        }
      } else {
        xs_terms = op.i[3] == NB_F32 ? 2 : 1;
        if (tid == 0) s_scale[oi & 1] = s_scale[(oi & 1) ^ 1];
      }
      __syncthreads();
      NB_STRACE(oi, 1);
      prefetch_op();

      // ---- this warp's units
      if (xs_terms == 2) run_units<BITS, 2>(ctx, use, fetch, oi, x_s, red, rt_first);
      else run_units<BITS, 1>(ctx, use, fetch, oi, x_s, red, rt_first);
      __syncthreads();
      NB_STRACE(oi, 2);

      // ---- add the warps' partial sums in warp order and write the results
      const float scale = s_scale[oi & 1];
      if (op.epi == NB_SEPI_SWIGLU) {
        // rows 0..7 of a tile are gate channels, rows 8..15 the matching up channels
        float* out = reinterpret_cast<float*>(op.p[4]);
        for (int e = tid; e < n_rt * 8; e += kSThreads) {
          const int tl = e >> 3, r = e & 7;
          float gsum = 0.f, usum = 0.f;
#pragma unroll
          for (int w = 0; w < kSW; ++w) { gsum += red[(tl * kSW + w) * 16 + r]; usum += red[(tl * kSW + w) * 16 + r + 8]; }
          gsum *= scale; usum *= scale;
          const int ch = (rt_first + tl) * 8 + r;
          if (ch < N / 2) out[ch] = gsum / (1.0f + __expf(-gsum)) * usum;
        }
      } else {
        const int units = ((N + 15) >> 4) * bpr;
        for (int e = tid; e < n_rt * 16; e += kSThreads) {
          const int tl = e >> 4, r = e & 15;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kSW; ++w) v += red[(tl * kSW + w) * 16 + r];
          v *= scale;
          const int rt = rt_first + tl, row = rt * 16 + r;
          if (row >= N) continue;
          if (op.epi == NB_SEPI_STORE) {
            store_y(op.p[4], op.i[4], row, v);
          } else {  // NB_SEPI_SLOTS: slot = index of this CTA among the CTAs that share the row tile
            const int first = cta_of_unit(rt * bpr, units, G), last = cta_of_unit((rt + 1) * bpr - 1, units, G);
            float* out = reinterpret_cast<float*>(op.p[4]);
            out[(size_t)(cta - first) * op.i[8] + row] = v;
            if (cta == first) {
              // the first CTA of a row tile clears the slots nobody writes: those past the last CTA, and
              // those of CTAs in between whose share of the units is empty (fewer units than CTAs)
              for (int sl = 1; sl < op.i[6]; ++sl) {
                bool unused = sl > last - first;
                if (!unused) {
                  int lo, hi;
                  share(units, G, first + sl, lo, hi);
                  unused = lo == hi;
                }
                if (unused) out[(size_t)sl * op.i[8] + row] = 0.f;
              }
            }
          }
        }
      }
    } else if (op.kind == NB_SOP_ATTN) {
      // ---- single-query attention of one new token: items (head, split) over the CTAs
      __syncthreads();
      prefetch_op();
      __syncthreads();
      const int Hl = op.i[0], hd = op.i[1], ctx_len = op.i[2], S = op.i[3], in_slots = op.i[5], in_stride = op.i[7];
      const float* qkv = reinterpret_cast<const float*>(op.p[0]);
      const float* cos2 = reinterpret_cast<const float*>(op.p[1]);
      const float* sin2 = reinterpret_cast<const float*>(op.p[2]);
      float* kc = reinterpret_cast<float*>(op.p[4]);
      float* vc = reinterpret_cast<float*>(op.p[5]);
      float* part = reinterpret_cast<float*>(op.p[6]);
      long long pos = *reinterpret_cast<const long long*>(op.p[3]);
      if (pos < 0) pos = 0;
      if (pos >= ctx_len) pos = ctx_len - 1;
      const int n = (int)pos + 1;
      const int per = (((n + S - 1) / S) + 7) & ~7;
      float* raw = reinterpret_cast<float*>(x_s);          // q | k | v of the head, raw then rotated: 6 * 128 floats
      float* sc = raw + 6 * 128;                           // scores of this split's keys
      float* pacc = sc + 2048;                             // [6][hd] partial value sums
      for (int item = cta; item < Hl * S; item += G) {
        const int h = item / S, s = item - h * S;
        const int k0 = s * per, cnt = max(0, min(n, k0 + per) - k0);
        __syncthreads();
        if (tid < 3 * hd) {
          const int which = tid / hd, i = tid - which * hd;
          float v = 0.f;
          for (int sl = 0; sl < in_slots; ++sl) v += __ldcg(qkv + (size_t)sl * in_stride + which * Hl * hd + h * hd + i);
          raw[which * 128 + i] = v;
        }
        __syncthreads();
        if (tid < 2 * hd) {
          const int which = tid / hd, i = tid - which * hd;
          const float cs = __ldg(cos2 + pos * hd + i), sn = __ldg(sin2 + pos * hd + i);
          const float sign = (i & 1) ? 1.f : -1.f;   // rot = (-x2, x1) on interleaved pairs
          const float v = raw[which * 128 + i] * cs + sign * raw[which * 128 + (i ^ 1)] * sn;
          raw[(3 + which) * 128 + i] = which == 0 ? v * rsqrtf((float)hd) : v;
        }
        __syncthreads();
        const float* qs = raw + 3 * 128;
        const float* kn = raw + 4 * 128;
        const float* vn = raw + 2 * 128;
        const size_t head_off = (size_t)h * ctx_len * hd;
        const bool owner = pos >= k0 && pos < k0 + cnt;
        if (owner && tid < hd) {
          kc[head_off + (size_t)pos * hd + tid] = kn[tid];
          vc[head_off + (size_t)pos * hd + tid] = vn[tid];
        }
        // scores: one warp per key, lanes over the head dimension
        const int hd4 = hd >> 2;
        for (int j = warp; j < cnt; j += kSW) {
          const int key = k0 + j;
          float d = 0.f;
          if (lane < hd4) {
            const float4 q4 = reinterpret_cast<const float4*>(qs)[lane];
            const float4 k4 = key == (int)pos ? reinterpret_cast<const float4*>(kn)[lane]
                                              : __ldg(reinterpret_cast<const float4*>(kc + head_off + (size_t)key * hd) + lane);
            d = q4.x * k4.x + q4.y * k4.y + q4.z * k4.z + q4.w * k4.w;
          }
          d = warp_sum_f(d);
          if (lane == 0) sc[j] = d;
        }
        __syncthreads();
        float mx = -FLT_MAX;
        for (int j = tid; j < cnt; j += kSThreads) mx = fmaxf(mx, sc[j]);
        mx = block_max(mx, s16, tid);
        float sum = 0.f;
        for (int j = tid; j < cnt; j += kSThreads) {
          const float p = __expf(sc[j] - mx);
          sc[j] = p;
          sum += p;
        }
        sum = block_sum(sum, s16, tid);   // its barriers also publish the probabilities
        // values: six groups of hd threads, group q takes keys j = q, q + 6, ...
        const int grp = tid / hd, d = tid - grp * hd;
        if (grp < 6) {
          float a = 0.f;
          for (int j = grp; j < cnt; j += 6) {
            const int key = k0 + j;
            const float v = key == (int)pos ? vn[d] : __ldg(vc + head_off + (size_t)key * hd + d);
            a += sc[j] * v;
          }
          pacc[grp * hd + d] = a;
        }
        __syncthreads();
        if (tid < hd) {
          float a = 0.f;
#pragma unroll
          for (int q = 0; q < 6; ++q) a += pacc[q * hd + tid];
          part[(size_t)item * (hd + 2) + tid] = a;
        }
        if (tid == 0) {
          part[(size_t)item * (hd + 2) + hd] = cnt > 0 ? mx : -FLT_MAX;
          part[(size_t)item * (hd + 2) + hd + 1] = sum;
        }
      }
    } else if (op.kind == NB_SOP_HEAD) {
      // ---- final norm + LM head rows of this CTA + soft-cap + the CTA's best candidate
      __syncthreads();
      prefetch_op();
      const OpInfo& f = info[oi];
      const int C = op.i[1];
      float* xh = reinterpret_cast<float*>(x_s);
      const float4* w4 = reinterpret_cast<const float4*>(op.p[3]);
      float ss = 0.f;
      for (int i4 = tid; i4 < C / 4; i4 += kSThreads) {
        float4 h = reinterpret_cast<const float4*>(h_s)[i4];
        float4 dl = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sl = 0; sl < op.i[5]; ++sl) {
          const float4 e = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.p[1]) + (size_t)sl * op.i[7]) + i4);
          dl.x += e.x; dl.y += e.y; dl.z += e.z; dl.w += e.w;
        }
        h.x += dl.x; h.y += dl.y; h.z += dl.z; h.w += dl.w;
        reinterpret_cast<float4*>(h_s)[i4] = h;
        ss += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
        const float4 w = __ldg(w4 + i4);
        reinterpret_cast<float4*>(xh)[i4] = make_float4(h.x * w.x, h.y * w.y, h.z * w.z, h.w * w.w);
      }
      const float tot = block_sum(ss, s16, tid);
      const float inv = 1.0f / sqrtf(tot / (float)C + op.f[0]);
      __syncthreads();
      const float cap = op.f[1];
      float* logits = reinterpret_cast<float*>(op.p[4]);
      float best = -FLT_MAX;
      int besti = 0x7fffffff;
      float acc = 0.f;
      while (use.op == oi) {
        const uint8_t* st = wait_chunk(ctx, use);
        const int row = use.u / f.bpr, piece = use.u - row * f.bpr;
        const int off = piece * f.ubytes;
        const int bytes = min((int)f.ubytes, f.row_bytes - off);
        for (int j = lane; j < bytes / 16; j += 32) {
          const uint4 r = *reinterpret_cast<const uint4*>(st + 16 * j);
          const float* xv = xh + (off >> 1) + 8 * j;
          const float4 x0 = *reinterpret_cast<const float4*>(xv), x1 = *reinterpret_cast<const float4*>(xv + 4);
          acc += __uint_as_float(r.x << 16) * x0.x + __uint_as_float(r.x & 0xFFFF0000u) * x0.y +
                 __uint_as_float(r.y << 16) * x0.z + __uint_as_float(r.y & 0xFFFF0000u) * x0.w +
                 __uint_as_float(r.z << 16) * x1.x + __uint_as_float(r.z & 0xFFFF0000u) * x1.y +
                 __uint_as_float(r.w << 16) * x1.z + __uint_as_float(r.w & 0xFFFF0000u) * x1.w;
        }
        if (piece == f.bpr - 1) {
          const float v = cap * tanhf(warp_sum_f(acc) * inv / cap);
          acc = 0.f;
          if (lane == 0) logits[row] = v;
          const int gi = op.i[8] + row;      // index in the whole vocabulary
          if (v > best || (v == best && gi < besti)) { best = v; besti = gi; }
        }
        use.u += 1;
        ++use.count;
        cursor_seek(ctx, use);
        __syncwarp();
        fetch_next(ctx, fetch);
      }
      if (lane == 0) { s_best[warp] = best; s_besti[warp] = besti; }
      __syncthreads();
      if (tid == 0) {
        float b = -FLT_MAX;
        int bi = 0x7fffffff;
        for (int w = 0; w < kSW; ++w)
          if (s_best[w] > b || (s_best[w] == b && s_besti[w] < bi)) { b = s_best[w]; bi = s_besti[w]; }
        float* cand = reinterpret_cast<float*>(op.p[5]);
        cand[2 * cta] = b;
        reinterpret_cast<int*>(cand)[2 * cta + 1] = bi;
      }
    } else if (op.kind == NB_SOP_REDUCE) {
      // ---- y = sum of a projection's partial slots (in slot order), converted to the output type
      __syncthreads();
      prefetch_op();
      __syncthreads();
      const int N = op.i[0];
      for (int i = cta * kSThreads + tid; i < N; i += G * kSThreads) {
        float v = 0.f;
        for (int sl = 0; sl < op.i[5]; ++sl) v += __ldcg(reinterpret_cast<const float*>(op.p[1]) + (size_t)sl * op.i[7] + i);
        store_y(op.p[4], op.i[4], i, v);
      }
    } else if (op.kind == NB_SOP_ARGMAX) {
      // ---- the best of the CTAs' candidates (lowest index among equals) becomes the next token
      __syncthreads();
      prefetch_op();
      __syncthreads();
      if (cta == 0 && warp == 0) {
        const float* cand = reinterpret_cast<const float*>(op.p[0]);
        float b = -FLT_MAX;
        int bi = 0x7fffffff;
        for (int i = lane; i < op.i[0]; i += 32) {
          const float v = __ldcg(cand + 2 * i);
          const int vi = __ldcg(reinterpret_cast<const int*>(cand) + 2 * i + 1);
          if (v > b || (v == b && vi < bi)) { b = v; bi = vi; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, b, o);
          const int obi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ob > b || (ob == b && obi < bi)) { b = ob; bi = obi; }
        }
        if (lane == 0) {
          *reinterpret_cast<long long*>(op.p[1]) = (long long)bi;
          if (op.p[2]) *reinterpret_cast<long long*>(op.p[2]) += 1;
        }
      }
    }

    // ---- publish (only when somebody will wait for it): this CTA's results up to operation oi are complete
    if (info[oi].flags & 1) {
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        st_release_gpu_u32(flags + cta, seq);
      }
    }
    NB_STRACE(oi, 3);
  }

  // the next launch's sequence numbers start above this one's: written once every CTA is done
  wait_flags(flags, G, base + (uint32_t)n_ops, spin_limit, status, tid);
  if (cta == 0 && tid == 0) state[kMaxCtas] = base + (uint32_t)n_ops + 1u;
}

#ifdef NB_STREAM_TRACE
extern "C" int nb_stream_trace_read(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, nb_stream_trace_buf, sizeof(nb_stream_trace_buf));
}
#endif

// ---- relayout: nativebit/pack.py byte stream -> stream layout ------------------------------------
// One thread per (unit, lane): writes the lane's index words; threads with lane < 16 also write row `lane`'s table.
template <int BITS>
__global__ void __launch_bounds__(256) stream_pack_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ codebook, int cb_dtype,
                                                          int N, int bpr, int row_mode, uint8_t* __restrict__ out, long long units) {
  using F = UnitFmt<BITS>;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long u = gid >> 5;
  if (u >= units) return;
  const int lane = (int)(gid & 31), g = lane >> 2, t = lane & 3;
  const int rt = (int)(u / bpr), kb = (int)(u - (long long)rt * bpr);
  // source row of tile row i: identity, or (row_mode 1) rows 0..7 = gate channels 8rt..8rt+7, rows 8..15 = the
  // matching up channels of a fused [gate | up] matrix of N rows
  auto src_row = [&](int i) -> int {
    if (row_mode == 1) return i < 8 ? rt * 8 + i : N / 2 + rt * 8 + (i - 8);
    return rt * 16 + i;
  };
  constexpr int kBlkBytes = 16 * BITS;
  uint8_t* ub = out + u * F::kBytes;
  uint32_t seq[2 * F::kW];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = src_row(g + 8 * half);
    const bool valid = row < N;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + ((size_t)row * bpr + kb) * kBlkBytes) + F::kW * t;
#pragma unroll
    for (int j = 0; j < F::kW; ++j) seq[half * F::kW + j] = valid ? src[j] : 0u;
  }
#pragma unroll
  for (int j = 0; j < F::kW; ++j) *reinterpret_cast<uint2*>(ub + j * 256 + lane * 8) = make_uint2(seq[2 * j], seq[2 * j + 1]);
  if (lane < 16) {
    const int row = src_row(lane);
    const bool valid = row < N;
    const int cb_blk = (cb_dtype == NB_F16 ? 2 : 4) << BITS;
    uint32_t T[BITS == 4 ? 8 : 4];
    make_table<BITS>(reinterpret_cast<const uint8_t*>(codebook) + ((size_t)(valid ? row : 0) * bpr + kb) * cb_blk, cb_dtype, valid, T);
    uint32_t* dst = reinterpret_cast<uint32_t*>(ub + F::kIdxBytes + lane * F::kTabBytes);
#pragma unroll
    for (int j = 0; j < F::kTabBytes / 4; ++j) dst[j] = T[j];
  }
}

}  // namespace nb

using namespace nb;

extern "C" size_t nb_stream_packed_bytes(int N, int K, int bits) {
  if (N < 1 || K < 1 || K % kBlock != 0 || (bits != 2 && bits != 3 && bits != 4)) return 0;
  return (size_t)((N + 15) / 16) * (K / kBlock) * unit_bytes(bits);
}

extern "C" int nb_stream_pack(const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int N, int K, int row_mode,
                              uint8_t* out, void* stream) {
  if (!packed || !codebook || !out || N < 1 || K < 1) return NB_ERR_ARG;
  if (cb_dtype != NB_F16 && cb_dtype != NB_F32) return NB_ERR_ARG;
  if (K % kBlock != 0 || (bits != 2 && bits != 3 && bits != 4)) return NB_ERR_SHAPE;
  if (row_mode != 0 && row_mode != 1) return NB_ERR_ARG;
  if (row_mode == 1 && (N % 16 != 0)) return NB_ERR_SHAPE;       // gate and up halves in whole groups of 8 channels
  if ((uintptr_t)packed % 4 || (uintptr_t)codebook % 16 || (uintptr_t)out % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const int bpr = K / kBlock;
  const long long units = (long long)((N + 15) / 16) * bpr;
  const long long threads = units * 32;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (bits == 3) stream_pack_kernel<3><<<grid, 256, 0, st>>>(packed, codebook, cb_dtype, N, bpr, row_mode, out, units);
  else if (bits == 2) stream_pack_kernel<2><<<grid, 256, 0, st>>>(packed, codebook, cb_dtype, N, bpr, row_mode, out, units);
  else stream_pack_kernel<4><<<grid, 256, 0, st>>>(packed, codebook, cb_dtype, N, bpr, row_mode, out, units);
  return check_launch();
}

extern "C" size_t nb_stream_state_bytes(void) { return (size_t)(kMaxCtas + 64) * sizeof(uint32_t); }

extern "C" int nb_stream_max_ops(void) { return kMaxOps; }

// Host-side validation of one operation; returns the bits of its weight stream (0 = none) through *bits.
static int check_op(const nb_stream_op& o, int index, int G, int* bits) {
  char msg[200];
  auto fail = [&](const char* why) {
    std::snprintf(msg, sizeof(msg), "nb_stream_run: operation %d: %s", index, why);
    set_last_error(msg);
    return (int)NB_ERR_SHAPE;
  };
  *bits = 0;
  if (o.kind == NB_SOP_GEMV) {
    const int N = o.i[0], K = o.i[1], b = o.i[2];
    if (N < 1 || K < kBlock || K % kBlock != 0 || K / kBlock > kMaxKBlocks) return fail("needs N >= 1 and K a multiple of 128 up to 7168");
    if (b != 2 && b != 3 && b != 4) return fail("bits must be 2, 3 or 4");
    if (!o.p[0] || !o.p[4] || (uintptr_t)o.p[0] % 16) return fail("null or misaligned weight / output pointer");
    if (!(o.flags & NB_SOPF_REUSE_X) && !o.p[1]) return fail("null activation pointer");
    if ((uintptr_t)o.p[1] % 16) return fail("activations must be 16-byte aligned");
    if (o.pro < NB_SPRO_VEC || o.pro > NB_SPRO_ATTN_MERGE) return fail("unknown prologue");
    if ((o.pro == NB_SPRO_EMBED_NORM || o.pro == NB_SPRO_ADD_NORM) && (K > kMaxC || !o.p[3])) return fail("norm prologue needs K <= 3072 and a weight");
    if (o.pro == NB_SPRO_EMBED_NORM && !o.p[2]) return fail("embedding prologue needs a token pointer");
    if (o.epi < NB_SEPI_STORE || o.epi > NB_SEPI_SWIGLU) return fail("unknown epilogue");
    if (o.epi != NB_SEPI_SLOTS && !(o.flags & NB_SOPF_ALIGN)) return fail("only the slot epilogue may split a row tile between CTAs");
    if (o.epi == NB_SEPI_SWIGLU && N % 16 != 0) return fail("SwiGLU epilogue needs N % 16 == 0");
    if ((long long)((N + 15) / 16) * (K / kBlock) * (G + 1) >= (1ll << 31)) return fail("matrix too large for the 32-bit work split");
    const OpGeom g = geom_of(o);
    // local row tiles of a CTA must fit the reduction buffer, and the slots must cover every CTA of a row tile
    int worst_rt = 0, worst_slots = 1;
    for (int c = 0; c < G; ++c) {
      int ca, cb;
      cta_range(g, c, G, ca, cb);
      if (cb > ca) worst_rt = std::max(worst_rt, (cb - 1) / g.bpr - ca / g.bpr + 1);
    }
    if (!g.align)
      for (int rt = 0; rt < g.rt; ++rt)
        worst_slots = std::max(worst_slots, cta_of_unit((rt + 1) * g.bpr - 1, g.units, G) - cta_of_unit(rt * g.bpr, g.units, G) + 1);
    if (worst_rt * kSW * 16 > kRedHalf) return fail("too many row tiles per CTA for the reduction buffer");
    if (o.epi == NB_SEPI_SLOTS && (o.i[6] < worst_slots || o.i[8] < N)) return fail("too few output slots (see nb_stream_slots) or slot stride < N");
    *bits = b;
  } else if (o.kind == NB_SOP_ATTN) {
    const int Hl = o.i[0], hd = o.i[1], ctx = o.i[2], S = o.i[3];
    if (Hl < 1 || hd < 4 || hd > 128 || hd % 4 || 3 * hd > kSThreads || ctx < 1 || S < 1) return fail("attention needs head_dim % 4 == 0, <= 128");
    if ((((ctx + S - 1) / S) + 7) > 2048) return fail("more than 2048 keys per attention split");
    for (int j = 0; j < 7; ++j) if (!o.p[j]) return fail("null pointer");
  } else if (o.kind == NB_SOP_HEAD) {
    if (o.i[0] < 1 || o.i[1] < 8 || o.i[1] % 8 || o.i[1] > kMaxC) return fail("head needs C % 8 == 0, <= 3072");
    if (!o.p[0] || !o.p[3] || !o.p[4] || !o.p[5] || (uintptr_t)o.p[0] % 16) return fail("null or misaligned pointer");
  } else if (o.kind == NB_SOP_REDUCE) {
    if (!o.p[1] || !o.p[4] || o.i[0] < 1 || o.i[5] < 1 || o.i[7] < o.i[0]) return fail("null pointer or bad slot geometry");
  } else if (o.kind == NB_SOP_ARGMAX) {
    if (!o.p[0] || !o.p[1] || o.i[0] < 1) return fail("null pointer");
  } else {
    return fail("unknown kind");
  }
  return NB_OK;
}

extern "C" int nb_stream_slots(int N, int K, int ctas) {
  if (N < 1 || K < kBlock || K % kBlock || ctas < 1) return 0;
  const int bpr = K / kBlock, rt_n = (N + 15) / 16;
  if ((long long)rt_n * bpr * (ctas + 1) >= (1ll << 31)) return 0;
  const int U = rt_n * bpr;
  int worst = 1;
  for (int rt = 0; rt < rt_n; ++rt)
    worst = std::max(worst, cta_of_unit((rt + 1) * bpr - 1, U, ctas) - cta_of_unit(rt * bpr, U, ctas) + 1);
  return worst;
}

extern "C" int nb_stream_ctas(void) {
  return std::min(sm_count(), kMaxCtas);
}

extern "C" int nb_stream_run(const nb_stream_op* ops_host, const nb_stream_op* ops_device, int n_ops, void* state, uint32_t spin_limit,
                             void* stream) {
  if (!ops_host || !ops_device || !state || n_ops < 1) return NB_ERR_ARG;
  if (n_ops > kMaxOps) return NB_ERR_SHAPE;
  if ((uintptr_t)ops_device % 4 || (uintptr_t)state % 4) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const int G = nb_stream_ctas();
  int bits = 0;
  for (int i = 0; i < n_ops; ++i) {
    int b = 0;
    if (int rc = check_op(ops_host[i], i, G, &b)) return rc;
    if (b && bits && b != bits) { set_last_error("nb_stream_run: all packed matrices of a program must use the same bits"); return NB_ERR_SHAPE; }
    if (b) bits = b;
  }
  if (!bits) bits = 3;
  static bool attr_done[64][5] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const void* fn = bits == 3 ? (const void*)stream_kernel<3> : bits == 2 ? (const void*)stream_kernel<2> : (const void*)stream_kernel<4>;
  if (!attr_done[dev & 63][bits]) {
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem)) return record_cuda_error(e);
    attr_done[dev & 63][bits] = true;
  }
  // All CTAs wait on one another's flags: the launch is cooperative, so either all are resident or it fails.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(kSThreads);
  cfg.dynamicSmemBytes = kStreamSmem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const uint32_t spin = spin_limit ? spin_limit : kFlagSpinDefault;
  uint32_t* st = reinterpret_cast<uint32_t*>(state);
  if (bits == 3) return record_cuda_error(cudaLaunchKernelEx(&cfg, stream_kernel<3>, ops_device, n_ops, st, spin));
  if (bits == 2) return record_cuda_error(cudaLaunchKernelEx(&cfg, stream_kernel<2>, ops_device, n_ops, st, spin));
  return record_cuda_error(cudaLaunchKernelEx(&cfg, stream_kernel<4>, ops_device, n_ops, st, spin));
}

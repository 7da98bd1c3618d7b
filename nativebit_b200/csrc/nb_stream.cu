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
//    are consecutive.  Every operation's units are split evenly over the CTAs and, inside a CTA, over
//    its 32 warps as contiguous runs, so a warp's share of a matrix is one contiguous byte range.  Each
//    warp owns a private ring of shared-memory stages (one unit each) that it fills itself with 16-byte
//    asynchronous copies (cp.async, all lanes, one commit group per unit): the refill of a stage is
//    issued the moment the warp has consumed it, and the sequence of units runs on across operation
//    boundaries, because weights never depend on earlier results.  About 96 KB of weights per SM are in
//    flight or resident at all times, which covers the dependency waits between operations.
//  * Compute.  Lane (g, t) of a warp unpacks 32 weights of row g and 32 of row g+8 of the unit
//    (selector words + byte-permute table lookups, nb_common.cuh) and feeds them, four per row at a
//    time, as the A fragment of an m16n8k16 fp16 tensor-core MMA whose B fragment is the matching four
//    activations; fp32 activations are carried as two fp16 terms.  A warp keeps the partial sums of its
//    run per row tile and stores them to a slot in shared memory; warps do not wait for one another at
//    the end of a matrix: the warp that delivers the last units of a row tile adds the tile's slots in k
//    order and writes the results while the others are already unpacking the next matrix.
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
#include <cstdlib>
#include <cstring>
#include <functional>
#include <queue>
#include <utility>
#include <vector>

#include "nb_common.cuh"
#include "nb_device.cuh"
#include "nb_host.h"

namespace nb {

#ifndef NB_STREAM_WARPS
#define NB_STREAM_WARPS 16
#endif
constexpr int kSW = NB_STREAM_WARPS;                      // warps per CTA (one CTA per SM)
constexpr int kSThreads = kSW * 32;
constexpr int kRingBytes = 120 * 1024;                    // kSW warps x stages x one unit
constexpr int kMaxOps = 160;
constexpr int kMaxKBlocks = 56;                           // K <= 7168
constexpr int kXSegBytes = 80;                            // 32 halves of one (k-block, lane t) + skew (16-byte aligned)
constexpr int kXTermBytes = kMaxKBlocks * 4 * kXSegBytes; // 17.5 KB per fp16 term
constexpr int kMaxC = 2560;                               // residual width
constexpr int kRedBufs = 4;                               // operations whose partial sums may be alive at once
constexpr int kRedUnits = 128;                            // units of one operation per CTA
constexpr int kRedSegs = 3;                               // row tiles one warp's run may touch
constexpr int kRedBufFloats = kSW * kRedSegs * 16;
constexpr int kMaxLocalTiles = 8;                         // row tiles of one operation a CTA may touch
constexpr int kMaxCtas = 512;
constexpr uint32_t kCopySpin = 1u << 22;
constexpr uint32_t kFlagSpinDefault = 1u << 22;

using StreamOp = nb_stream_op;

// What the weight stream needs to know about an operation, computed once per launch.
struct OpInfo {
  int cta_a, cta_b;           // this CTA's unit range
  int bpr;                    // units per row tile (GEMV: k-blocks per row; head: pieces per table row)
  uint32_t bpr_magic;         // ceil(2^32 / bpr): u / bpr = umulhi(u, magic) for u < 65536
  const uint8_t* w;           // unit 0
  uint16_t ubytes;            // bytes of a unit (GEMV: 16 rows x one block; head: one piece of a table row)
  uint8_t kind;
  uint8_t flags;              // bit 0: the next operation waits for this one (or it is the last)
  uint8_t slot_first;         // slot epilogue: this CTA's slot in its first row tile when earlier CTAs share that tile
  uint8_t last_span;          // ... and how many later CTAs reach into its last row tile
  uint16_t next_empty;        // bit j: CTA cta+1+j has no units of this operation
};
static_assert(sizeof(OpInfo) == 32, "OpInfo layout");
// u / bpr for u < 65536 (bpr == 1 has no 32-bit magic number)
__device__ __forceinline__ int div_bpr(const OpInfo& f, int u) { return f.bpr == 1 ? u : (int)__umulhi((uint32_t)u, f.bpr_magic); }

// shared-memory layout (dynamic)
constexpr int kOffRing = 0;
constexpr int kOffInfo = kOffRing + kRingBytes;
constexpr int kOffRun = kOffInfo + kMaxOps * (int)sizeof(OpInfo);   // [op][warp] {first unit, units} of every warp's run
constexpr int kOffX = kOffRun + kMaxOps * kSW * 4;
constexpr int kOffH = kOffX + 2 * kXTermBytes;
constexpr int kOffRed = kOffH + kMaxC * 4;
constexpr int kOffDst = kOffRed + kRedBufs * kRedBufFloats * 4;
constexpr int kStreamSmem = kOffDst + 256;
static_assert(sizeof(StreamOp) == 160, "nb_stream_op layout");
static_assert(kStreamSmem <= 224 * 1024, "shared memory budget");

// A unit in the stream layout: the 32 lanes' selector words, then the 16 rows' lookup tables.  Lane
// (g, t) owns weights 32t .. 32t+31 of the block in rows g and g+8: four words per row, word j = the
// indices of positions 32t + 8j .. + 7, one per nibble in position order, ready for the byte-permute
// lookups (the 3- and 2-bit fields are spread to nibbles when the copy is built, so the kernels spend
// no instructions on it, and activations are used in their natural order).
template <int BITS> struct UnitFmt {
  static constexpr int kW = Fmt<BITS>::kWords / 4;          // packed words of one lane's 32 indices in the source layout
  static constexpr int kIdxBytes = 1024;                    // 32 lanes x 2 rows x 4 selector words
  static constexpr int kTabBytes = BITS == 4 ? 32 : 16;     // one row's lookup table
  static constexpr int kBytes = kIdxBytes + 16 * kTabBytes; // 1280 at 2 and 3 bits, 1536 at 4: one ring stage
  static constexpr int kStages = kRingBytes / (kSW * kBytes) < 16 ? kRingBytes / (kSW * kBytes) : 16;   // per warp: 6, 6, 5 with 16 warps
  // units a warp works on per loop iteration (one wait, one round of bookkeeping for all of them)
#ifdef NB_STREAM_BATCH
  static constexpr int kBatch = NB_STREAM_BATCH < kStages ? NB_STREAM_BATCH : kStages - 1;
#else
  static constexpr int kBatch = kStages >= 6 ? 4 : (kStages >= 4 ? 2 : 1);
#endif
};

__host__ __device__ inline int unit_bytes(int bits) { return bits == 3 ? UnitFmt<3>::kBytes : bits == 2 ? UnitFmt<2>::kBytes : UnitFmt<4>::kBytes; }

// ---- work split (32-bit arithmetic; the host refuses matrices of 65536 units or more) ----
// [lo, hi) of part `i` of `parts` equal shares of n items.
__host__ __device__ inline void share(int n, int parts, int i, int& lo, int& hi) {
  lo = (int)((unsigned)n * (unsigned)i / (unsigned)parts);
  hi = (int)((unsigned)n * (unsigned)(i + 1) / (unsigned)parts);
}
// Part that owns item u when U items are split into G parts by share().
__host__ __device__ inline int part_of(int u, int U, int G) { return (int)(((unsigned)(u + 1) * (unsigned)G - 1u) / (unsigned)U); }
__host__ __device__ inline int cta_of_unit(int u, int U, int G) { return part_of(u, U, G); }

struct OpGeom {
  int kind, bits, bpr, rt, align, ubytes, units, row_bytes;
};

// prog_bits: the bits of the program's packed matrices (they set the size of a ring stage).
__host__ __device__ inline OpGeom geom_of(const StreamOp& o, int prog_bits) {
  OpGeom g{};
  g.kind = o.kind;
  if (o.kind == NB_SOP_GEMV) {
    g.bits = o.i[2];
    g.bpr = o.i[1] / kBlock;
    g.rt = (o.i[0] + 15) / 16;
    g.align = (o.flags & NB_SOPF_ALIGN) ? 1 : 0;
    g.ubytes = unit_bytes(g.bits);
    g.units = g.rt * g.bpr;
  } else if (o.kind == NB_SOP_HEAD) {
    const int stage = unit_bytes(prog_bits);
    g.row_bytes = o.i[1] * 2;
    g.bpr = (g.row_bytes + stage - 1) / stage;                   // pieces per table row, each at most one stage
    g.ubytes = ((g.row_bytes / g.bpr + 15) / 16) * 16;           // bytes of a full piece
    g.rt = o.i[0];                                               // rows
    g.align = 1;
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
// A warp's part of its CTA's range [0, n) (local unit indices): equal shares of the units (of whole rows for the head).
__host__ __device__ inline void warp_part(int kind, int bpr, int n, int warp, int& a, int& b) {
  if (kind == NB_SOP_HEAD) {
    const int rows = n / bpr;
    a = (rows * warp / kSW) * bpr;
    b = (rows * (warp + 1) / kSW) * bpr;
  } else {
    a = n * warp / kSW;
    b = n * (warp + 1) / kSW;
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

// Four consecutive activations (positions 4*i4 .. 4*i4+3 of the row) -> fp16 hi (+ lo) terms.  The staged
// row keeps the natural order; every 32 activations (one lane's share of a k-block) start a new segment of
// kXSegBytes, which spreads the four lanes t of a warp over different banks.
template <int XS>
__device__ __forceinline__ void stage4(uint8_t* x_s, int i4, float u0, float u1, float u2, float u3) {
  uint8_t* dst = x_s + (i4 >> 3) * kXSegBytes + (i4 & 7) * 8;      // 8 groups of four per segment
  const uint32_t h01 = f32x2_to_f16x2_sat(u0, u1), h23 = f32x2_to_f16x2_sat(u2, u3);
  *reinterpret_cast<uint2*>(dst) = make_uint2(h01, h23);
  if (XS == 2) {
    const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
    const float2 r23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
    const uint32_t l01 = f32x2_to_f16x2_sat(fminf(fmaxf(u0, -65504.f), 65504.f) - r01.x, fminf(fmaxf(u1, -65504.f), 65504.f) - r01.y);
    const uint32_t l23 = f32x2_to_f16x2_sat(fminf(fmaxf(u2, -65504.f), 65504.f) - r23.x, fminf(fmaxf(u3, -65504.f), 65504.f) - r23.y);
    *reinterpret_cast<uint2*>(dst + kXTermBytes) = make_uint2(l01, l23);
  }
}

// ---- the per-warp weight stream ------------------------------------------------------------------
// Every warp streams its own units: for every operation with a weight stream, its contiguous part of
// the CTA's unit range, one unit (a piece of a table row for the head) per ring stage.  The copies are
// 16-byte asynchronous copies issued by all lanes (cp.async: bulk copies were measured to deliver only
// a few GB/s per SM here), one commit group per unit; `fetch` runs kStages - 1 units ahead of `use`.
struct Cursor {
  int op;          // operation index (n_ops when exhausted)
  int u, u_end;    // next unit and end of the warp's range, relative to the CTA's range of that operation
  int stage;       // ring stage of the next unit
  const uint8_t* src;   // packed matrices: address of the next unit
  int ubytes;           // ... and its size
  int head;             // the operation is the LM head (pieces of table rows)
};

struct StreamCtx {
  const OpInfo* info;    // in shared memory
  const uint32_t* runs;  // in shared memory: [op][warp] first unit | units << 16 of the warp's run
  const StreamOp* ops;   // in global memory
  int n_ops, warp, lane;
  int stages, stage_bytes;
  uint8_t* ring;         // this warp's stages
};

__device__ __forceinline__ void cursor_seek(const StreamCtx& c, Cursor& k) {   // skip to the next non-empty range
  while (k.op < c.n_ops && k.u >= k.u_end) {
    ++k.op;
    if (k.op < c.n_ops) {
      const uint32_t run = c.runs[k.op * kSW + c.warp];
      k.u = (int)(run & 0xFFFFu);
      k.u_end = k.u + (int)(run >> 16);
      if (k.u_end > k.u) {
        const OpInfo& f = c.info[k.op];
        k.ubytes = f.ubytes;
        k.head = f.kind == NB_SOP_HEAD;
        k.src = f.w + (size_t)(f.cta_a + k.u) * f.ubytes;
      }
    }
  }
}
__device__ __forceinline__ void cursor_init(const StreamCtx& c, Cursor& k) {
  k.op = -1; k.u = 0; k.u_end = 0; k.stage = 0; k.src = nullptr; k.ubytes = 0; k.head = 0;
  cursor_seek(c, k);
}
__device__ __forceinline__ void cursor_step(const StreamCtx& c, Cursor& k) {   // one unit further
  ++k.u;
  k.src += k.ubytes;
  if (++k.stage == c.stages) k.stage = 0;
  if (k.u >= k.u_end) cursor_seek(c, k);
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// All lanes: request the unit at the fetch cursor into its stage (if any is left) and close the commit group.
template <int BITS>
__device__ __forceinline__ void fetch_next(const StreamCtx& c, Cursor& f) {
  if (f.op < c.n_ops) {
    const uint8_t* src = f.src;
    uint8_t* dst = c.ring + f.stage * c.stage_bytes;
    if (!f.head) {               // a unit of a packed matrix: fixed size, straight-line copies
      constexpr int kChunks = UnitFmt<BITS>::kBytes / 16;
#pragma unroll
      for (int i = 0; i < (kChunks + 31) / 32; ++i)
        if (i * 32 + 32 <= kChunks || c.lane + i * 32 < kChunks) cp_async16(dst + 16 * (c.lane + i * 32), src + 16 * (c.lane + i * 32));
      cursor_step(c, f);
      cp_async_commit();
      return;
    }
    int bytes = f.ubytes;
    {
      const OpInfo& fi = c.info[f.op];
      const int lu = f.u;                                        // local unit = local row * pieces + piece
      const int row = div_bpr(fi, lu), piece = lu - row * fi.bpr;
      const int row_bytes = c.ops[f.op].i[1] * 2, off = piece * fi.ubytes;
      bytes = min(bytes, row_bytes - off);
      src = fi.w + ((size_t)(fi.cta_a / fi.bpr) + row) * row_bytes + off;
    }
    for (int i = c.lane; i < (bytes >> 4); i += 32) cp_async16(dst + 16 * i, src + 16 * i);
    cursor_step(c, f);
  }
  cp_async_commit();
}

// ---- one unit: 16 rows x 128 weights against the staged activations -----------------------------
// `xseg`: this lane's 32 activations of the unit's k-block (fp16, 64 bytes), the second fp16 term `term_stride`
// bytes further on.
template <int BITS, int XS>
__device__ __forceinline__ void unit_mma_x(const uint8_t* ub, const uint8_t* xseg, int term_stride, int lane, float (&c)[2][4]) {
  using F = UnitFmt<BITS>;
  const int g = lane >> 2;
  const uint4 ua = *reinterpret_cast<const uint4*>(ub + lane * 16);
  const uint4 ub4 = *reinterpret_cast<const uint4*>(ub + 512 + lane * 16);
  const uint32_t UA[4] = {ua.x, ua.y, ua.z, ua.w}, UB[4] = {ub4.x, ub4.y, ub4.z, ub4.w};
  uint32_t TA[BITS == 4 ? 8 : 4], TB[BITS == 4 ? 8 : 4];
  const uint8_t* tab = ub + F::kIdxBytes;
#pragma unroll
  for (int j = 0; j < F::kTabBytes / 16; ++j) {
    const uint4 a = *reinterpret_cast<const uint4*>(tab + g * F::kTabBytes + 16 * j);
    const uint4 b = *reinterpret_cast<const uint4*>(tab + (g + 8) * F::kTabBytes + 16 * j);
    TA[4 * j] = a.x; TA[4 * j + 1] = a.y; TA[4 * j + 2] = a.z; TA[4 * j + 3] = a.w;
    TB[4 * j] = b.x; TB[4 * j + 1] = b.y; TB[4 * j + 2] = b.z; TB[4 * j + 3] = b.w;
  }
#pragma unroll
  for (int uu = 0; uu < 4; ++uu) {
    uint4 xq[XS];    // the activations of steps 2*uu and 2*uu + 1
#pragma unroll
    for (int xs = 0; xs < XS; ++xs) xq[xs] = *reinterpret_cast<const uint4*>(xseg + xs * term_stride + uu * 16);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t sa = h ? (UA[uu] >> 16) : UA[uu];
      const uint32_t sb = h ? (UB[uu] >> 16) : UB[uu];
      uint32_t a0, a1, a2, a3;
      lookup4<BITS>(sa, TA, a0, a2);
      lookup4<BITS>(sb, TB, a1, a3);
#pragma unroll
      for (int xs = 0; xs < XS; ++xs) mma_16816(c[h], a0, a1, a2, a3, h ? xq[xs].z : xq[xs].x, h ? xq[xs].w : xq[xs].y);
    }
  }
}

template <int BITS, int XS>
__device__ __forceinline__ void unit_mma(const uint8_t* ub, const uint8_t* x_s, int kb, int lane, float (&c)[2][4]) {
  unit_mma_x<BITS, XS>(ub, x_s + (kb * 4 + (lane & 3)) * kXSegBytes, kXTermBytes, lane, c);
}

// Two units at once, their steps interleaved: two independent instruction streams per warp hide the
// latencies of the shared-memory loads, the byte permutes and the tensor-core MMAs (a warp's own stream is
// one long dependency chain; four warps per scheduler do not cover it).
template <int BITS, int XS>
__device__ __forceinline__ void unit_mma2(const uint8_t* ub0, const uint8_t* ub1, const uint8_t* x_s, int kb0, int kb1, int lane,
                                          float (&c0)[2][4], float (&c1)[2][4]) {
  using F = UnitFmt<BITS>;
  constexpr int kT = BITS == 4 ? 8 : 4;
  const int g = lane >> 2, t = lane & 3;
  const uint8_t* ubs[2] = {ub0, ub1};
  uint32_t UA[2][4], UB[2][4], TA[2][kT], TB[2][kT];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const uint4 a = *reinterpret_cast<const uint4*>(ubs[u] + lane * 16);
    const uint4 b = *reinterpret_cast<const uint4*>(ubs[u] + 512 + lane * 16);
    UA[u][0] = a.x; UA[u][1] = a.y; UA[u][2] = a.z; UA[u][3] = a.w;
    UB[u][0] = b.x; UB[u][1] = b.y; UB[u][2] = b.z; UB[u][3] = b.w;
    const uint8_t* tab = ubs[u] + F::kIdxBytes;
#pragma unroll
    for (int j = 0; j < F::kTabBytes / 16; ++j) {
      const uint4 ta = *reinterpret_cast<const uint4*>(tab + g * F::kTabBytes + 16 * j);
      const uint4 tb = *reinterpret_cast<const uint4*>(tab + (g + 8) * F::kTabBytes + 16 * j);
      TA[u][4 * j] = ta.x; TA[u][4 * j + 1] = ta.y; TA[u][4 * j + 2] = ta.z; TA[u][4 * j + 3] = ta.w;
      TB[u][4 * j] = tb.x; TB[u][4 * j + 1] = tb.y; TB[u][4 * j + 2] = tb.z; TB[u][4 * j + 3] = tb.w;
    }
  }
  const uint8_t* xseg[2] = {x_s + (kb0 * 4 + t) * kXSegBytes, x_s + (kb1 * 4 + t) * kXSegBytes};
#pragma unroll
  for (int uu = 0; uu < 4; ++uu) {
    uint4 xq[2][XS];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int xs = 0; xs < XS; ++xs) xq[u][xs] = *reinterpret_cast<const uint4*>(xseg[u] + xs * kXTermBytes + uu * 16);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t a0[2], a1[2], a2[2], a3[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t sa = h ? (UA[u][uu] >> 16) : UA[u][uu];
        const uint32_t sb = h ? (UB[u][uu] >> 16) : UB[u][uu];
        lookup4<BITS>(sa, TA[u], a0[u], a2[u]);
        lookup4<BITS>(sb, TB[u], a1[u], a3[u]);
      }
#pragma unroll
      for (int xs = 0; xs < XS; ++xs) {
        mma_16816(c0[h], a0[0], a1[0], a2[0], a3[0], h ? xq[0][xs].z : xq[0][xs].x, h ? xq[0][xs].w : xq[0][xs].y);
        mma_16816(c1[h], a0[1], a1[1], a2[1], a3[1], h ? xq[1][xs].z : xq[1][xs].x, h ? xq[1][xs].w : xq[1][xs].y);
      }
    }
  }
}

// Warp that owns local unit v when a CTA's n units are split by warp_part() (packed matrices).
__device__ __forceinline__ int warp_of_unit(int v, int n) { return part_of(v, n, kSW); }

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
__device__ unsigned long long nb_stream_trace_warp_end[kMaxCtas * kSW];
#define NB_STRACE(op, i)                                                     \
  do {                                                                       \
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {                        \
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
  constexpr int kStages = UnitFmt<BITS>::kStages, kStageBytes = UnitFmt<BITS>::kBytes;
  OpInfo* info = reinterpret_cast<OpInfo*>(smem + kOffInfo);
  uint8_t* x_s = smem + kOffX;
  float* h_s = reinterpret_cast<float*>(smem + kOffH);
  float* red_base = reinterpret_cast<float*>(smem + kOffRed);
  __shared__ float s16[kSW];
  __shared__ float s_scale;
  __shared__ float s_best[kSW];
  __shared__ int s_besti[kSW];
  __shared__ int s_tile_cnt[kRedBufs][kMaxLocalTiles];   // units of a row tile whose partial sums are in, per operation (ring)
  __shared__ int s_tiles_done[kRedBufs];                 // row tiles of an operation that have been written
  __shared__ volatile int s_finished;                    // operations whose results are completely written

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  uint32_t* flags = state;
  int* status = reinterpret_cast<int*>(state + kMaxCtas + 1);
  const uint32_t base = state[kMaxCtas];      // sequence numbers of this launch start above the previous launch's

  for (int i = tid; i < n_ops; i += kSThreads) {
    const StreamOp& o = ops_g[i];
    const OpGeom g = geom_of(o, BITS);
    OpInfo f;
    cta_range(g, cta, G, f.cta_a, f.cta_b);
    f.bpr = g.bpr > 0 ? g.bpr : 1;
    f.bpr_magic = (uint32_t)((0x100000000ull + (unsigned)f.bpr - 1) / (unsigned)f.bpr);
    f.ubytes = (uint16_t)g.ubytes;
    f.kind = (uint8_t)g.kind;
    f.w = reinterpret_cast<const uint8_t*>(o.p[0]);
    f.flags = (i + 1 == n_ops || (ops_g[i + 1].flags & NB_SOPF_WAIT_PREV)) ? 1 : 0;
    f.slot_first = 0; f.last_span = 0; f.next_empty = 0;
    if (g.kind == NB_SOP_GEMV && !g.align && f.cta_b > f.cta_a) {
      const int rt_a = f.cta_a / g.bpr, rt_b = (f.cta_b - 1) / g.bpr;
      f.slot_first = (uint8_t)(cta - cta_of_unit(rt_a * g.bpr, g.units, G));
      f.last_span = (uint8_t)(cta_of_unit((rt_b + 1) * g.bpr - 1, g.units, G) - cta);
      for (int j = 0; j < 16 && cta + 1 + j < G; ++j) {
        int lo, hi;
        share(g.units, G, cta + 1 + j, lo, hi);
        if (lo == hi) f.next_empty |= (uint16_t)(1u << j);
      }
    }
    info[i] = f;
  }
  if (tid < kRedBufs * kMaxLocalTiles) (&s_tile_cnt[0][0])[tid] = 0;
  if (tid < kRedBufs) s_tiles_done[tid] = 0;
  if (tid == 0) s_finished = 0;
  __syncthreads();

  // every warp's run of every operation: equal shares of the CTA's units, handed out in an order that
  // rotates from operation to operation (the same warps would otherwise get the larger shares every time)
  uint32_t* runs = reinterpret_cast<uint32_t*>(smem + kOffRun);
  for (int i = tid; i < n_ops * kSW; i += kSThreads) {
    const int o = i / kSW, w = i - o * kSW;
    const OpInfo& f = info[o];
    int a = 0, b = 0;
    if (f.cta_b > f.cta_a) warp_part(f.kind, f.bpr, f.cta_b - f.cta_a, (w + o) & (kSW - 1), a, b);
    runs[i] = (uint32_t)a | ((uint32_t)(b - a) << 16);
  }
  __syncthreads();
  StreamCtx ctx{info, runs, ops_g, n_ops, warp, lane, kStages, kStageBytes, smem + kOffRing + warp * kStages * kStageBytes};
  Cursor fetch, use;
  cursor_init(ctx, fetch);
  cursor_init(ctx, use);
  for (int s = 0; s < kStages - 1; ++s) fetch_next<BITS>(ctx, fetch);

  // One thread of the CTA, after all of the CTA's writes for operation oi: make them visible and raise the flag.
  auto publish = [&](int oi) {
    if (info[oi].flags & 1) {
      __threadfence();
      st_release_gpu_u32(flags + cta, base + (uint32_t)oi + 1u);
    }
    s_finished = oi + 1;
  };

  for (int oi = 0; oi < n_ops; ++oi) {
    const StreamOp& op = ops_g[oi];
    const OpInfo& fi = info[oi];
    const uint32_t seq = base + (uint32_t)oi + 1u;     // published after this operation
    const bool waits = oi > 0 && (op.flags & NB_SOPF_WAIT_PREV);
    if (warp == 0) NB_STRACE(oi, 4);

    if (op.kind == NB_SOP_GEMV) {
      const int N = op.i[0], K = op.i[1];
      // ---- stage the activations (all warps together), unless the previous matvec's are used again
      if (waits) wait_flags(flags, G, seq - 1u, spin_limit, status, tid);
      const bool stage = !(op.flags & NB_SOPF_REUSE_X);
      const int xs_terms = op.pro == NB_SPRO_VEC ? (op.i[3] == NB_F32 ? 2 : 1) : 2;
      if (stage) {
        if (!waits) __syncthreads();   // every warp is done with the activations of the matvec before
        NB_STRACE(oi, 0);
        if (op.pro == NB_SPRO_VEC) {
          const int dt = op.i[3];
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
            if (dt == NB_F32) stage4<2>(x_s, i4, v[0], v[1], v[2], v[3]);
            else stage4<1>(x_s, i4, v[0], v[1], v[2], v[3]);
          }
          if (tid == 0) s_scale = 1.f;
        } else if (op.pro == NB_SPRO_EMBED_NORM || op.pro == NB_SPRO_ADD_NORM) {
          // residual: h = table[token] (first layer) or h += sum of the previous projection's partial slots;
          // activation = h * weight, the factor 1/rms (a scalar) is applied to the outputs
          const float4* w4 = reinterpret_cast<const float4*>(op.p[3]);
          float ss = 0.f;
          for (int i4 = tid; i4 < K / 4; i4 += kSThreads) {
            float4 h;
            if (op.pro == NB_SPRO_EMBED_NORM) {
              long long tok = *reinterpret_cast<const long long*>(op.p[2]);
              tok = tok < 0 ? 0 : (tok >= op.i[13] ? op.i[13] - 1 : tok);   // never read outside the table
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
            stage4<2>(x_s, i4, h.x * w.x, h.y * w.y, h.z * w.z, h.w * w.w);
          }
          const float tot = block_sum(ss, s16, tid);
          if (tid == 0) s_scale = 1.0f / sqrtf(tot / (float)K + op.f[0]);
        } else if (op.pro == NB_SPRO_ATTN_MERGE) {
          // activations = attention output: per head, the splits' partial softmax numerators and
          // denominators merged; columns outside this rank's heads are zero
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
            stage4<2>(x_s, i4, v[0], v[1], v[2], v[3]);
          }
          if (tid == 0) s_scale = 1.f;
        }
        __syncthreads();
        NB_STRACE(oi, 1);
      }

      // ---- this warp's units.  Warps run ahead of one another by at most kRedBufs - 1 operations (the
      // partial sums live in a ring of kRedBufs buffers).
      if (lane == 0) {
        uint32_t spins = 0;
        while (s_finished < oi - (kRedBufs - 1)) {
          __nanosleep(64);
          if (++spins > kCopySpin) { atomicExch(status, (int)NB_ERR_TIMEOUT); break; }
        }
      }
      __syncwarp();
      const int buf = oi & (kRedBufs - 1);
      float* red = red_base + buf * kRedBufFloats;
      const int bpr = fi.bpr, cta_a = fi.cta_a, cta_b = fi.cta_b, n_units = cta_b - cta_a;
      const int rt_first = n_units > 0 ? div_bpr(fi, cta_a) : 0;
      const int n_rt = n_units > 0 ? div_bpr(fi, cta_b - 1) - rt_first + 1 : 0;
      // This CTA's part of the matrix is complete: results are published in order (the matrix before this
      // one may still be in another warp's hands).
      auto op_complete = [&]() {
        uint32_t spins = 0;
        while (s_finished < oi) {
          __nanosleep(64);
          if (++spins > kCopySpin) { atomicExch(status, (int)NB_ERR_TIMEOUT); break; }
        }
        publish(oi);
      };
      if (n_units == 0 && tid == 0) op_complete();
      if (use.op == oi) {
        constexpr int kBatch = UnitFmt<BITS>::kBatch;
        const int sh = (warp + oi) & (kSW - 1);          // this warp's share of the units in this operation
        float* red_w = red + sh * (kRedSegs * 16);
        int rt = div_bpr(fi, cta_a + use.u), kb = cta_a + use.u - rt * bpr;
        int left = use.u_end - use.u;                    // units left in the run
        int v0 = use.u;                                  // first unit of the segment (inside the CTA's range)
        // the run, row tile by row tile
        for (int seg = 0; left > 0; ++seg) {
          const int seg_len = min(left, bpr - kb);
          float acc[2][2][4];   // [unit parity][step parity]: four independent MMA chains
#pragma unroll
          for (int q = 0; q < 16; ++q) (&acc[0][0][0])[q] = 0.f;
          for (int done = 0; done < seg_len;) {
            // up to kBatch consecutive units per iteration: one wait, one round of bookkeeping
            const int nb = min(kBatch, seg_len - done);
            cp_async_wait<kStages - 1 - kBatch>();       // this lane's copies of the oldest kBatch units have landed ...
            __syncwarp();                                // ... and so have the other lanes'
            auto stage_of = [&](int b2) {
              int sidx = use.stage + b2;
              if (sidx >= kStages) sidx -= kStages;
              return ctx.ring + sidx * kStageBytes;
            };
            // units in pairs (interleaved), then a single one if the count is odd
#pragma unroll
            for (int b2 = 0; b2 + 1 < kBatch; b2 += 2) {
              if (b2 + 1 < nb) {
                if (xs_terms == 2) unit_mma2<BITS, 2>(stage_of(b2), stage_of(b2 + 1), x_s, kb + b2, kb + b2 + 1, lane, acc[0], acc[1]);
                else unit_mma2<BITS, 1>(stage_of(b2), stage_of(b2 + 1), x_s, kb + b2, kb + b2 + 1, lane, acc[0], acc[1]);
              }
            }
            if (nb & 1) {
              if (xs_terms == 2) unit_mma<BITS, 2>(stage_of(nb - 1), x_s, kb + nb - 1, lane, acc[0]);
              else unit_mma<BITS, 1>(stage_of(nb - 1), x_s, kb + nb - 1, lane, acc[0]);
            }
            use.u += nb;
            use.stage += nb;
            if (use.stage >= kStages) use.stage -= kStages;
            __syncwarp();                                // every lane has consumed the stages before they are overwritten
#pragma unroll
            for (int b2 = 0; b2 < kBatch; ++b2)
              if (b2 < nb) fetch_next<BITS>(ctx, fetch);
            kb += nb;
            done += nb;
          }
          // ---- the segment's partial sums go to this share's slot; the warp that delivers the last units of
          // a row tile adds the tile's partial sums in k order and writes the results, while the others carry on
          if ((lane & 3) == 0) {
            red_w[seg * 16 + (lane >> 2)] = (acc[0][0][0] + acc[0][1][0]) + (acc[1][0][0] + acc[1][1][0]);
            red_w[seg * 16 + (lane >> 2) + 8] = (acc[0][0][2] + acc[0][1][2]) + (acc[1][0][2] + acc[1][1][2]);
          }
          const int tl = rt - rt_first;
          const int v_lo = max(rt * bpr, cta_a) - cta_a, v_hi = min((rt + 1) * bpr, cta_b) - cta_a;
          __syncwarp();
          int ticket = 0;
          if (lane == 0) {
            __threadfence_block();
            ticket = atomicAdd(&s_tile_cnt[buf][tl], seg_len);
          }
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket + seg_len == v_hi - v_lo) {
            __threadfence_block();
            const float scale = s_scale;
            const int r = lane & 15, half = lane >> 4;
            // segments of this tile: one per share from sh_lo to sh_hi; lanes 0-15 add the first half of them, lanes 16-31 the rest
            const int sh_lo = part_of(v_lo, n_units, kSW), sh_hi = part_of(v_hi - 1, n_units, kSW);
            const int sh_mid = sh_lo + ((sh_hi - sh_lo + 2) >> 1);
            float y = 0.f;
            for (int w = half ? sh_mid : sh_lo; w < (half ? sh_hi + 1 : sh_mid); ++w) {
              const int a_w = n_units * w / kSW, b_w = n_units * (w + 1) / kSW;
              if (b_w > a_w) {
                const int first = div_bpr(fi, cta_a + a_w);   // first row tile of that share's run
                y += red[(w * kRedSegs + (rt - first)) * 16 + r];
              }
            }
            y += __shfl_down_sync(0xffffffffu, y, 16);      // row r: first half + second half
            y *= scale;
            if (op.epi == NB_SEPI_SWIGLU) {
              // rows 0..7 of a tile are gate channels, rows 8..15 the matching up channels
              const float up = __shfl_down_sync(0xffffffffu, y, 8);
              const int ch = rt * 8 + r;
              if (lane < 8 && ch < N / 2) reinterpret_cast<float*>(op.p[4])[ch] = y / (1.0f + __expf(-y)) * up;
            } else {
              const int row = rt * 16 + r;
              if (!half && row < N) {
                if (op.epi == NB_SEPI_STORE) {
                  store_y(op.p[4], op.i[4], row, y);
                } else {  // NB_SEPI_SLOTS: slot = index of this CTA among the CTAs that share the row tile
                  // only a CTA's first and last row tile can be shared (with earlier / later CTAs)
                  const bool shared_before = tl == 0 && rt * bpr < cta_a;
                  const int span_after = (tl == n_rt - 1 && (rt + 1) * bpr > cta_b) ? fi.last_span : 0;
                  float* out = reinterpret_cast<float*>(op.p[4]);
                  out[(size_t)(shared_before ? fi.slot_first : 0) * op.i[8] + row] = y;
                  if (!shared_before) {
                    // the first CTA of a row tile clears the slots nobody writes: those past the last CTA, and
                    // those of CTAs in between whose share of the units is empty (fewer units than CTAs)
                    for (int sl = 1; sl < op.i[6]; ++sl)
                      if (sl > span_after || ((fi.next_empty >> (sl - 1)) & 1)) out[(size_t)sl * op.i[8] + row] = 0.f;
                  }
                }
              }
            }
            __syncwarp();
            if (lane == 0) {
              s_tile_cnt[buf][tl] = 0;
              if (fi.flags & 1) __threadfence();          // someone will wait for this operation: the tile's stores are out
              if (atomicAdd(&s_tiles_done[buf], 1) == n_rt - 1) {
                s_tiles_done[buf] = 0;
                op_complete();
              }
            }
          }
          left -= seg_len;
          v0 += seg_len;
          kb = 0;
          ++rt;
        }
        (void)v0;
        cursor_seek(ctx, use);
      }
      if (warp == 0) NB_STRACE(oi, 6);
      continue;
    }

    // ---- the other kinds run with all warps in step
    if (waits) wait_flags(flags, G, seq - 1u, spin_limit, status, tid);
    else __syncthreads();
    if (op.kind == NB_SOP_ATTN) {
      // ---- single-query attention of one new token: items (head, split) over the CTAs
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
      float* pacc = sc + 2048;                             // [groups][hd] partial value sums
      const int n_grp = min(kSThreads / hd, 12);
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
        // values: groups of hd threads, group q takes keys j = q, q + n_grp, ...
        const int grp = tid / hd, d = tid - grp * hd;
        if (grp < n_grp) {
          float a = 0.f;
          for (int j = grp; j < cnt; j += n_grp) {
            const int key = k0 + j;
            const float v = key == (int)pos ? vn[d] : __ldg(vc + head_off + (size_t)key * hd + d);
            a += sc[j] * v;
          }
          pacc[grp * 128 + d] = a;
        }
        __syncthreads();
        if (tid < hd) {
          float a = 0.f;
          for (int q = 0; q < n_grp; ++q) a += pacc[q * 128 + tid];
          part[(size_t)item * (hd + 2) + tid] = a;
        }
        if (tid == 0) {
          part[(size_t)item * (hd + 2) + hd] = cnt > 0 ? mx : -FLT_MAX;
          part[(size_t)item * (hd + 2) + hd + 1] = sum;
        }
      }
    } else if (op.kind == NB_SOP_HEAD) {
      // ---- final norm + LM head rows of this CTA + soft-cap + the CTA's best candidate
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
      const int row_bytes = C * 2, pieces = fi.bpr, row0 = fi.cta_a / fi.bpr;
      float acc = 0.f;
      int row = use.op == oi ? div_bpr(fi, use.u) : 0, piece = use.op == oi ? use.u - row * pieces : 0;
      while (use.op == oi) {
        cp_async_wait<kStages - 2>();
        __syncwarp();
        const uint8_t* st = ctx.ring + use.stage * kStageBytes;
        const int off = piece * fi.ubytes;
        const int bytes = min((int)fi.ubytes, row_bytes - off);
        for (int j = lane; j < bytes / 16; j += 32) {
          const uint4 r = *reinterpret_cast<const uint4*>(st + 16 * j);
          const float* xv = xh + (off >> 1) + 8 * j;
          const float4 x0 = *reinterpret_cast<const float4*>(xv), x1 = *reinterpret_cast<const float4*>(xv + 4);
          acc += __uint_as_float(r.x << 16) * x0.x + __uint_as_float(r.x & 0xFFFF0000u) * x0.y +
                 __uint_as_float(r.y << 16) * x0.z + __uint_as_float(r.y & 0xFFFF0000u) * x0.w +
                 __uint_as_float(r.z << 16) * x1.x + __uint_as_float(r.z & 0xFFFF0000u) * x1.y +
                 __uint_as_float(r.w << 16) * x1.z + __uint_as_float(r.w & 0xFFFF0000u) * x1.w;
        }
        if (piece == pieces - 1) {
          const float v = cap * tanhf(warp_sum_f(acc) * inv / cap);
          acc = 0.f;
          if (lane == 0) logits[row0 + row] = v;
          const int gi = op.i[8] + row0 + row;      // index in the whole vocabulary
          if (v > best || (v == best && gi < besti)) { best = v; besti = gi; }
        }
        if (++piece == pieces) { piece = 0; ++row; }
        cursor_step(ctx, use);
        __syncwarp();
        fetch_next<BITS>(ctx, fetch);
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
      const int N = op.i[0];
      for (int i = cta * kSThreads + tid; i < N; i += G * kSThreads) {
        float v = 0.f;
        for (int sl = 0; sl < op.i[5]; ++sl) v += __ldcg(reinterpret_cast<const float*>(op.p[1]) + (size_t)sl * op.i[7] + i);
        store_y(op.p[4], op.i[4], i, v);
      }
    } else if (op.kind == NB_SOP_ARGMAX) {
      // ---- the best of the CTAs' candidates (lowest index among equals) becomes the next token
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
          *reinterpret_cast<long long*>(op.p[1]) = (long long)(bi == 0x7fffffff ? 0 : bi);
          if (op.p[2]) *reinterpret_cast<long long*>(op.p[2]) += 1;
        }
      }
    }
    // ---- this CTA's results up to operation oi are complete
    __syncthreads();
    if (tid == 0) publish(oi);
    if (warp == 0) NB_STRACE(oi, 5);
  }

  cp_async_wait<0>();
#ifdef NB_STREAM_TRACE
  if ((threadIdx.x & 31) == 0) {   // per warp of every CTA: when it ran out of work
    unsigned long long t_;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));
    nb_stream_trace_warp_end[blockIdx.x * kSW + (threadIdx.x >> 5)] = t_;
  }
#endif
  // the next launch's sequence numbers start above this one's: written once every CTA is done
  wait_flags(flags, G, base + (uint32_t)n_ops, spin_limit, status, tid);
  if (cta == 0 && tid == 0) state[kMaxCtas] = base + (uint32_t)n_ops + 1u;
}

#ifdef NB_STREAM_TRACE
extern "C" int nb_stream_trace_read(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, nb_stream_trace_buf, sizeof(nb_stream_trace_buf));
}
extern "C" int nb_stream_trace_read_ends(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, nb_stream_trace_warp_end, sizeof(nb_stream_trace_warp_end));
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
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = src_row(g + 8 * half);
    const bool valid = row < N;
    // the lane's 32 indices (group t of the block) as packed words, spread to four selector words
    const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + ((size_t)row * bpr + kb) * kBlkBytes) + F::kW * t;
    uint32_t w[F::kW], U[4], P[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < F::kW; ++j) w[j] = valid ? src[j] : 0u;
    group_selectors<BITS>(w, 0, U);
    // nibble k of selector word u holds the index at position slot_position(0, u, k) of the group: put it in position order
#pragma unroll
    for (int uu = 0; uu < 4; ++uu)
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int pos = slot_position<BITS>(0, uu, k);
        P[pos >> 3] |= ((U[uu] >> (4 * k)) & 0xFu) << (4 * (pos & 7));
      }
    *reinterpret_cast<uint4*>(ub + half * 512 + lane * 16) = make_uint4(P[0], P[1], P[2], P[3]);
  }
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


// ====================================================================================================
// Independent matvecs: one warp per row tile
// ====================================================================================================
// A group of packed matvecs none of which reads another's result (the gate, up and down matrices of many
// layers against given activations; the reference runs each as its own launch,
// inference/triton_kernel.py:240-256).  Without dependencies no operation boundary is needed at all: the
// row tiles (16 rows x K) of ALL matrices are dealt out to the CTAs on the host (equal shares of the weight
// bytes, every CTA a mix of all tile lengths), and a CTA's 24 warps take its tiles one at a time, the longest
// first, so that the last warps to finish are at most one short tile apart.  A warp
// streams the units of its tile through its own ring of asynchronous copies and keeps the tile's 16 sums in
// its accumulator registers from the first unit to the last: no partial sums in shared memory, no tickets,
// no flags, no barrier after the activations are staged, and no wait that could fail to end.  Every output
// is the sum of its units in index order whichever warp computes it: bit-identical from run to run.
constexpr int kGroupMaxItems = 256;
constexpr int kGroupMaxX = 6;
constexpr int kGW = 24;                                   // warps per CTA: measured 0.174 ms per 691 MB step against 0.187 with 16 warps
                                                          // working on two units at a time; 20, 28 and 32 warps within 2 % of 24
constexpr int kGroupRing = 160 * 1024;                    // the warps' copy rings (5 stages of one unit per warp at 2 and 3 bits)
constexpr int kGroupRingSmall = 120 * 1024;               // ... 4 stages, when the staged activations need the room (2 and 3 bits)
constexpr int kGroupXBytes = 64 * 1024;                   // shared memory for the staged activations beside the large ring
constexpr int kGroupFifo = 8;                             // row tiles a warp may have taken ahead of its arithmetic
constexpr int kGroupSmem = kGroupRing + kGroupXBytes;

struct GroupItem {            // 48 bytes
  const uint8_t* w;           // stream-layout weights
  void* y;                    // outputs
  int n, bpr;                 // rows, k-blocks per row
  int tile0;                  // index of the matrix' first row tile in the sequence of all row tiles
  int x_off;                  // byte offset of its staged activations in shared memory
  int xs;                     // fp16 terms per activation (2: fp32 activations)
  int y_dtype;
  int m;                      // activation rows (1..8): column g of the MMA carries row g
  int x_row;                  // bytes between the staged rows
};
struct GroupX {               // 32 bytes: one distinct activation matrix (m rows of k values)
  const void* ptr;
  int k, dtype, off, xs, m, row;
};
struct GroupPlan {
  int n_items, n_x, total_tiles, ctas, bits, ring_bytes, pad[2];
  GroupX xv[kGroupMaxX];
  int cta_lo[kMaxCtas + 1];   // CTA c owns entries [cta_lo[c], cta_lo[c + 1]) of the tile list
  GroupItem items[kGroupMaxItems];
  int tile_list[1];           // total_tiles row-tile indices: every CTA's tiles, the longest first (the plan is allocated with the list's real length)
};

template <int BITS, int GW, bool PAIR, int RING>
__global__ void __launch_bounds__(GW * 32, 1) group_kernel(const GroupPlan* __restrict__ plan) {
  using F = UnitFmt<BITS>;
  constexpr int D = RING / (GW * F::kBytes) < 8 ? RING / (GW * F::kBytes) : 8;   // ring stages per warp
  constexpr int kThreads = GW * 32;
  static_assert(D >= 4, "the per-warp ring needs at least four stages");
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_next;
  __shared__ int s_tile0[kGroupMaxItems + 1];
  __shared__ int s_fifo[GW][kGroupFifo];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem + warp * (D * F::kBytes);
  uint8_t* x_all = smem + RING;
  const int n_items = plan->n_items;
  const int t_lo = plan->cta_lo[blockIdx.x], t_hi = plan->cta_lo[blockIdx.x + 1];

  // ---- the activation vectors, staged once for the whole launch (fp16 terms in k order, one segment per
  // lane share of a k-block)
  for (int v = 0; v < plan->n_x; ++v) {
    const GroupX xv = plan->xv[v];
    const int k4 = xv.k / 4;
    for (int e = tid; e < xv.m * k4; e += kThreads) {
      const int r = e / k4, i4 = e - r * k4;
      uint8_t* x_s = x_all + xv.off + r * xv.row;
      float u[4];
      if (xv.dtype == NB_F32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(xv.ptr) + e);
        u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w;
        stage4<2>(x_s, i4, u[0], u[1], u[2], u[3]);
      } else {
        const uint2 q = __ldg(reinterpret_cast<const uint2*>(xv.ptr) + e);
        if (xv.dtype == NB_BF16) {
          u[0] = __uint_as_float(q.x << 16); u[1] = __uint_as_float(q.x & 0xFFFF0000u);
          u[2] = __uint_as_float(q.y << 16); u[3] = __uint_as_float(q.y & 0xFFFF0000u);
        } else {
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
          u[0] = f0.x; u[1] = f0.y; u[2] = f1.x; u[3] = f1.y;
        }
        stage4<1>(x_s, i4, u[0], u[1], u[2], u[3]);
      }
    }
  }
  // 128 zero bytes: the activations of the MMA columns that carry no activation row (with one row, seven of the
  // eight; all columns would otherwise carry the same vector, and zeros cost the tensor cores less power)
  uint8_t* x_zero = smem + kGroupSmem - 128;
  if (tid < 32) reinterpret_cast<uint32_t*>(x_zero)[tid] = 0u;
  for (int i = tid; i <= n_items; i += kThreads) s_tile0[i] = i < n_items ? plan->items[i].tile0 : plan->total_tiles;
  if (tid == 0) s_next = t_lo;
  __syncthreads();

  // matrix that holds row tile t: the last item whose first tile is <= t
  auto item_of = [&](int t) {
    int lo = 0, hi = n_items - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_tile0[mid] <= t) lo = mid; else hi = mid - 1;
    }
    return lo;
  };
  // the warp takes the CTA's next row tile (or learns that none is left); all lanes get the same answer
  auto take = [&]() {
    int t = -1;
    if (lane == 0) {
      const int p = atomicAdd(&s_next, 1);
      if (p < t_hi) t = __ldg(plan->tile_list + p);
    }
    return __shfl_sync(0xffffffffu, t, 0);
  };

  // ---- the copy side: requests run D - 2 units ahead of the arithmetic
  int fifo_w = 0, fifo_r = 0;                              // tiles taken / tiles started (uniform in the warp)
  const uint8_t* f_src = nullptr;                          // next unit to request
  int f_left = 0;                                          // units of the current copy-side tile still to request
  bool f_done = false;
  int rq_stage = 0, use_stage = 0;                         // ring stage of the next request / of the next unit to use
  auto request_one = [&]() {
    if (f_left == 0 && !f_done) {
      const int t = take();
      if (t < 0) {
        f_done = true;
      } else {
        if (lane == 0) s_fifo[warp][fifo_w & (kGroupFifo - 1)] = t;
        ++fifo_w;
        const GroupItem& it = plan->items[item_of(t)];
        f_left = it.bpr;
        f_src = it.w + (size_t)(t - it.tile0) * it.bpr * F::kBytes;
      }
    }
    if (f_left > 0) {
      uint8_t* dst = ring + rq_stage * F::kBytes;
      constexpr int kChunks = F::kBytes / 16;
#pragma unroll
      for (int i = 0; i < (kChunks + 31) / 32; ++i)
        if (i * 32 + 32 <= kChunks || lane + i * 32 < kChunks) cp_async16(dst + 16 * (lane + i * 32), f_src + 16 * (lane + i * 32));
      f_src += F::kBytes;
      --f_left;
    }
    if (++rq_stage == D) rq_stage = 0;                     // a group is closed (and a stage passed over) even when nothing was left to request
    cp_async_commit();
  };
#pragma unroll 1
  for (int i = 0; i < D - 2; ++i) request_one();

  // ---- the arithmetic side
#pragma unroll 1
  while (true) {
    // The copy side is D - 2 >= 2 requests ahead, and the first request after a tile's last unit takes the next
    // tile: when no taken tile is waiting here, the CTA's stretch is exhausted.
    if (fifo_r == fifo_w) break;
    __syncwarp();
    const int t = s_fifo[warp][fifo_r & (kGroupFifo - 1)];
    ++fifo_r;
    const GroupItem it = plan->items[item_of(t)];
    const int rt = t - it.tile0;
    const uint8_t* x_s = x_all + it.x_off;
    float c0[2][4], c1[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) { c0[h][e] = 0.f; c1[h][e] = 0.f; }
#pragma unroll 1
    for (int j = 0; j < it.bpr;) {
      const int nb = (PAIR && it.bpr - j >= 2) ? 2 : 1;
      request_one();
      if (nb == 2) request_one();
      cp_async_wait<D - 2>();                              // all but the newest D - 2 requests have landed: units `consumed` (+1)
      __syncwarp();
      const uint8_t* u0 = ring + use_stage * F::kBytes;
      const uint8_t* u1 = ring + (use_stage + 1 == D ? 0 : use_stage + 1) * F::kBytes;
      if (PAIR && nb == 2) {
        if (it.xs == 2) unit_mma2<BITS, 2>(u0, u1, x_s, j, j + 1, lane, c0, c1);
        else unit_mma2<BITS, 1>(u0, u1, x_s, j, j + 1, lane, c0, c1);
      } else {
        // column g of the MMA carries activation row g (the lanes of group g supply it), columns without a row zeros
        const bool have = (lane >> 2) < it.m;
        const uint8_t* xseg = have ? x_s + (lane >> 2) * it.x_row + (j * 4 + (lane & 3)) * kXSegBytes : x_zero;
        if (it.xs == 2) unit_mma_x<BITS, 2>(u0, xseg, have ? kXTermBytes : 0, lane, c0);
        else unit_mma_x<BITS, 1>(u0, xseg, 0, lane, c0);
      }
      use_stage += nb;
      if (use_stage >= D) use_stage -= D;
      j += nb;
      __syncwarp();                                        // every lane is done with these stages before they are requested again
    }
    // lane (g, t) holds rows g and g + 8 of columns 2t and 2t + 1 = activation rows 2t, 2t + 1
    {
      const int g = lane >> 2, b0 = 2 * (lane & 3);
      const int ra = rt * 16 + g, rb = ra + 8;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (b0 + e < it.m) {
          const float ya = (c0[0][e] + c0[1][e]) + (c1[0][e] + c1[1][e]);
          const float yb = (c0[0][2 + e] + c0[1][2 + e]) + (c1[0][2 + e] + c1[1][2 + e]);
          if (ra < it.n) store_y(it.y, it.y_dtype, (size_t)(b0 + e) * it.n + ra, ya);
          if (rb < it.n) store_y(it.y, it.y_dtype, (size_t)(b0 + e) * it.n + rb, yb);
        }
      }
    }
  }
  cp_async_wait<0>();
}


// ====================================================================================================
// One matrix, one activation row, inside a chain of dependent launches (the decode step)
// ====================================================================================================
// y (N) = W x for ONE packed matrix in the stream layout, with the element-wise step in front of the packed
// linear computed while x is staged (inference/generate_torch.py:109-117): residual add + RMSNorm, or SwiGLU.
// The reference launches its fused matvec once per linear (inference/triton_kernel.py:240-256); so does this,
// but built like the group kernel above: one CTA per SM, 24 warps, every warp streams its own units through its
// own ring of asynchronous copies.  A matrix has far fewer 16-row tiles than the GPU has warps, so the k range of a
// tile is shared by a team of warps of ONE CTA (24, 12, 6 or 3 warps, as many as the row has k-blocks), whose
// partial sums meet in shared memory: no workspace, no tickets, nothing shared between CTAs.  The weights do not
// depend on the launch before: every warp requests its first units, then executes griddepcontrol.wait, then x is
// staged, so the dependent part of the launch is staging + a few units per warp + one block-wide sum per round.
constexpr int kTileRing = 160 * 1024;
constexpr int kTileSmem = kTileRing + 2 * kXTermBytes + 2 * kGW * 16 * 4 + 64;

struct TileGemvParams {
  const uint8_t* w;          // stream-layout weights
  const void* x;             // activations: K values (prologue 0, 1) or 2K values [gate | up] (prologue 2)
  const float* delta;        // prologue 1: added to x before the norm (may be null)
  const float* weight;       // prologue 1: RMSNorm weight
  float* x_out;              // prologue 1: receives x + delta (may be null; must not alias x)
  float* y;                  // N outputs, fp32
  int N, bpr, x_dtype, prologue;
  float eps;
  int wpt;                   // warps per team (24, 12, 6 or 3): chosen on the host
  int wpt_rcp, tpr, rounds;  // 65536 / wpt + 1; 24 / wpt; rounds of the launch
  int swiglu;                // epilogue: rows 0..7 of a tile are gate channels, rows 8..15 the matching up channels
                             // (nb_stream_pack row_mode 1); y receives N / 2 values silu(gate) * up
  int accumulate;            // y += W act(x): the residual update of a block in the matvec that produces it
};

template <int BITS, int XS>
__global__ void __launch_bounds__(kGW * 32, 1) tile_gemv_kernel(const TileGemvParams p) {
  using F = UnitFmt<BITS>;
  constexpr int D = kTileRing / (kGW * F::kBytes) < 8 ? kTileRing / (kGW * F::kBytes) : 8;
  constexpr int kThreads = kGW * 32;
  static_assert(D >= 4, "the per-warp ring needs at least four stages");
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s16[32];
  __shared__ float s_scale;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem + warp * (D * F::kBytes);
  uint8_t* x_s = smem + kTileRing;
  float* s_part = reinterpret_cast<float*>(smem + kTileRing + 2 * kXTermBytes);      // [2][kGW][16]
  const int bpr = p.bpr, K = bpr * kBlock;
  // the warps of a CTA form teams of wpt warps; a team shares the k-blocks of one row tile.  Tiles go round the CTAs
  // first and the teams second, so that a last, partly filled round still has work on every SM.
  // (quotients by the team size as multiply + shift with the host's reciprocal: exact for the few thousand at most
  // that occur here, and a kernel this short feels five integer divisions at its start)
  const int wpt = p.wpt, rcp = p.wpt_rcp;
  const int tpr = p.tpr;                                  // row tiles per CTA per round
  const int team = (warp * rcp) >> 16, wi = warp - team * wpt;
  const int u_lo = (bpr * wi * rcp) >> 16, u_hi = (bpr * (wi + 1) * rcp) >> 16;   // this warp's units of its team's tile
  const int n_tiles = (p.N + 15) >> 4;
  const int per_round = (int)gridDim.x * tpr;
  const int rounds = p.rounds;
  auto tile_at = [&](int r, int tm) { return r * per_round + tm * (int)gridDim.x + (int)blockIdx.x; };
  auto tile_of = [&](int r) { return tile_at(r, team); };

  // ---- copies: requests run D - 2 units ahead of the arithmetic; the first ones go out before the launch this one
  // depends on has finished
  int rq_round = 0, rq_u = u_lo, rq_stage = 0, use_stage = 0;
  auto request_one = [&]() {
    while (rq_round < rounds && (rq_u >= u_hi || tile_of(rq_round) >= n_tiles)) { ++rq_round; rq_u = u_lo; }
    if (rq_round < rounds) {
      const uint8_t* src = p.w + ((size_t)tile_of(rq_round) * bpr + rq_u) * F::kBytes;
      uint8_t* dst = ring + rq_stage * F::kBytes;
      constexpr int kChunks = F::kBytes / 16;
#pragma unroll
      for (int i = 0; i < (kChunks + 31) / 32; ++i)
        if (i * 32 + 32 <= kChunks || lane + i * 32 < kChunks) cp_async16(dst + 16 * (lane + i * 32), src + 16 * (lane + i * 32));
      ++rq_u;
    }
    if (++rq_stage == D) rq_stage = 0;
    cp_async_commit();
  };
#pragma unroll 1
  for (int i = 0; i < D - 2; ++i) request_one();
  // the RMSNorm weight does not depend on the launch before either: a third of the bytes this CTA stages
  constexpr int kIt = (kMaxKBlocks * kBlock / 4 + kThreads - 1) / kThreads;      // K <= 7168: at most three float4 per thread
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 vw[kIt];
#pragma unroll
  for (int j = 0; j < kIt; ++j) {
    const int i4 = tid + j * kThreads;
    vw[j] = (p.prologue == 1 && i4 < K / 4) ? __ldg(reinterpret_cast<const float4*>(p.weight) + i4) : zero4;
  }
  // (the dependents are released only after this kernel's own dependency is met: a launch behind this one may then
  // read, before ITS wait, anything written two or more launches back — the attention kernel does, see nb_decode.cu)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");

  // ---- the activations (and the element-wise step in front of this linear)
  if (p.prologue == 1) {
    const float4* xr = reinterpret_cast<const float4*>(p.x);
    const float4* dr = reinterpret_cast<const float4*>(p.delta);
    const bool writer = blockIdx.x == 0 && p.x_out != nullptr;
    float ss = 0.f;
    // all loads are issued before the first use (one memory round trip)
    float4 vx[kIt], vd[kIt];
#pragma unroll
    for (int j = 0; j < kIt; ++j) {
      const int i4 = tid + j * kThreads;
      const bool in = i4 < K / 4;
      vx[j] = in ? __ldcg(xr + i4) : zero4;
      vd[j] = (in && dr) ? __ldcg(dr + i4) : zero4;
    }
#pragma unroll
    for (int j = 0; j < kIt; ++j) {
      const int i4 = tid + j * kThreads;
      if (i4 < K / 4) {
        float4 v = vx[j];
        v.x += vd[j].x; v.y += vd[j].y; v.z += vd[j].z; v.w += vd[j].w;
        if (writer) reinterpret_cast<float4*>(p.x_out)[i4] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        stage4<XS>(x_s, i4, v.x * vw[j].x, v.y * vw[j].y, v.z * vw[j].z, v.w * vw[j].w);
      }
    }
    ss = warp_sum_f(ss);                                   // the warps' sums, then in warp order: the same bits in every CTA
    if (lane == 0) s16[warp] = ss;
    __syncthreads();
    if (tid == 0) {
      float tot = 0.f;
      for (int i = 0; i < kGW; ++i) tot += s16[i];
      s_scale = 1.0f / sqrtf(tot / (float)K + p.eps);
    }
  } else if (p.prologue == 2) {
    const float4* g4 = reinterpret_cast<const float4*>(p.x);
    const float4* u4 = g4 + K / 4;
    float4 vg[kIt], vu[kIt];
#pragma unroll
    for (int j = 0; j < kIt; ++j) {      // all loads first: one memory round trip
      const int i4 = tid + j * kThreads;
      vg[j] = i4 < K / 4 ? __ldcg(g4 + i4) : zero4;
      vu[j] = i4 < K / 4 ? __ldcg(u4 + i4) : zero4;
    }
#pragma unroll
    for (int j = 0; j < kIt; ++j) {
      const int i4 = tid + j * kThreads;
      const float4 g = vg[j], u = vu[j];
      if (i4 < K / 4)
        stage4<XS>(x_s, i4, g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y, g.z / (1.f + __expf(-g.z)) * u.z,
                  g.w / (1.f + __expf(-g.w)) * u.w);
    }
    if (tid == 0) s_scale = 1.f;
  } else {
#pragma unroll 3
    for (int i4 = tid; i4 < K / 4; i4 += kThreads) {
      float v[4];
      if (p.x_dtype == NB_F32) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.x) + i4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      } else {
        const uint2 q = __ldcg(reinterpret_cast<const uint2*>(p.x) + i4);
        if (p.x_dtype == NB_BF16) {
          v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xFFFF0000u);
          v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xFFFF0000u);
        } else {
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
          v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
        }
      }
      stage4<XS>(x_s, i4, v[0], v[1], v[2], v[3]);
    }
    if (tid == 0) s_scale = 1.f;
  }
  // zeros for the MMA columns that carry no activation row (seven of the eight)
  uint8_t* x_zero = reinterpret_cast<uint8_t*>(s_part + 2 * kGW * 16);
  if (tid < 16) reinterpret_cast<uint32_t*>(x_zero)[tid] = 0u;
  __syncthreads();
  const float scale = s_scale;

  // ---- rounds: every team one row tile; a warp adds its units, the team's sums meet in shared memory
  const bool col0 = lane < 4;
#pragma unroll 1
  for (int r = 0; r < rounds; ++r) {
    const int tile = tile_of(r);
    // accumulate flag: the output's old value (the residual stream) is requested now and added behind the round's barrier
    float res = 0.f;
    if (p.accumulate && tid < tpr * 16) {
      const int n_res = tile_at(r, tid >> 4) * 16 + (tid & 15);
      if (n_res < p.N) res = __ldcg(p.y + n_res);
    }
    float c[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[h][e] = 0.f;
    if (tile < n_tiles) {
#pragma unroll 1
      for (int u = u_lo; u < u_hi; ++u) {
        request_one();
        cp_async_wait<D - 2>();
        __syncwarp();
        const uint8_t* xseg = col0 ? x_s + (u * 4 + (lane & 3)) * kXSegBytes : x_zero;
        unit_mma_x<BITS, XS>(ring + use_stage * F::kBytes, xseg, col0 ? kXTermBytes : 0, lane, c);
        if (++use_stage == D) use_stage = 0;
        __syncwarp();
      }
    }
    float* part = s_part + (r & 1) * (kGW * 16);
    if ((lane & 3) == 0) {
      part[warp * 16 + (lane >> 2)] = c[0][0] + c[1][0];
      part[warp * 16 + 8 + (lane >> 2)] = c[0][2] + c[1][2];
    }
    __syncthreads();                                       // one barrier per round: the buffers alternate
    if (p.swiglu) {
      if (tid < tpr * 8) {
        const int tm = tid >> 3, ch = tid & 7;
        const int t_out = tile_at(r, tm);
        float gate = 0.f, up = 0.f;
        for (int j = 0; j < wpt; ++j) {                                          // the team's warps in k order
          gate += part[(tm * wpt + j) * 16 + ch];
          up += part[(tm * wpt + j) * 16 + 8 + ch];
        }
        gate *= scale; up *= scale;
        const int c_out = t_out * 8 + ch;
        if (t_out < n_tiles && c_out < (p.N >> 1)) p.y[c_out] = gate / (1.f + __expf(-gate)) * up;
      }
    } else if (tid < tpr * 16) {
      const int tm = tid >> 4, row = tid & 15;
      const int t_out = tile_at(r, tm);
      float acc = 0.f;
      for (int j = 0; j < wpt; ++j) acc += part[(tm * wpt + j) * 16 + row];     // the team's warps in k order
      const int n = t_out * 16 + row;
      if (t_out < n_tiles && n < p.N) p.y[n] = acc * scale + res;
    }
  }
  cp_async_wait<0>();
}


// ====================================================================================================
// The same chained matvec for up to eight activation rows (a decode step of 2 .. 8 sequences)
// ====================================================================================================
// Y (m, N) = act(X) W^T with m <= 8 fp32 activation rows against ONE pass over the weights: activation row g rides in
// column g of the m16n8k16 MMAs (the lanes of group g supply it), so eight rows cost the arithmetic of one — the
// columns that tile_gemv_kernel feeds zeros.  Everything else is that kernel: teams of warps per row tile, per-warp
// copy rings, one barrier per round, first weight requests before griddepcontrol.wait.  The staged rows take the
// shared memory that the ring gives up (three stages per warp instead of five): a row is its two fp16 terms back to
// back plus 16 bytes, so the eight lane groups read different banks.  For staging, the warps are dealt to the rows
// (24 / m warps per row, each a contiguous part of it); the squares of a row are added per warp and then in warp
// order, so every CTA scales a row by the same bits.
constexpr int kRowsD = 3;
constexpr int kRowsPartFloats = 2 * kGW * 8 * 16;           // [2][kGW][8 columns][16 rows]

struct TileRowsParams {
  const uint8_t* w;          // stream-layout weights
  const float* x;            // (m, K) activations, or (m, 2K) rows [gate | up] with the SwiGLU prologue
  const float* delta;        // prologue 1: (m, K) added to x before the norm (may be null)
  const float* weight;       // prologue 1: RMSNorm weight (K)
  float* x_out;              // prologue 1: receives x + delta (may be null; must not alias x)
  float* y;                  // (m, N) outputs, fp32
  int N, bpr, prologue, m;
  float eps;
  int wpt;                   // warps per team
  int wpt_rcp, tpr, rounds;  // 65536 / wpt + 1; 24 / wpt; rounds of the launch
  int row_bytes, term_bytes; // a staged row, one fp16 term of it
  int swiglu;                // epilogue: rows 0..7 of a tile are gate channels, rows 8..15 the matching up channels
                             // (nb_stream_pack row_mode 1); y is (m, N / 2) = silu(gate) * up
};

__device__ __forceinline__ void stage4_row(uint8_t* row_s, int term_bytes, int i4, float u0, float u1, float u2, float u3) {
  uint8_t* dst = row_s + (i4 >> 3) * kXSegBytes + (i4 & 7) * 8;
  const uint32_t h01 = f32x2_to_f16x2_sat(u0, u1), h23 = f32x2_to_f16x2_sat(u2, u3);
  *reinterpret_cast<uint2*>(dst) = make_uint2(h01, h23);
  const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
  const float2 r23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
  const uint32_t l01 = f32x2_to_f16x2_sat(fminf(fmaxf(u0, -65504.f), 65504.f) - r01.x, fminf(fmaxf(u1, -65504.f), 65504.f) - r01.y);
  const uint32_t l23 = f32x2_to_f16x2_sat(fminf(fmaxf(u2, -65504.f), 65504.f) - r23.x, fminf(fmaxf(u3, -65504.f), 65504.f) - r23.y);
  *reinterpret_cast<uint2*>(dst + term_bytes) = make_uint2(l01, l23);
}

template <int BITS>
__global__ void __launch_bounds__(kGW * 32, 1) tile_gemv_rows_kernel(const TileRowsParams p) {
  using F = UnitFmt<BITS>;
  constexpr int D = kRowsD;
  constexpr int kThreads = kGW * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_ss[kGW];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m = p.m;
  uint8_t* ring = smem + warp * (D * F::kBytes);
  uint8_t* x_s = smem + kGW * D * F::kBytes;
  float* s_part = reinterpret_cast<float*>(x_s + m * p.row_bytes);
  uint8_t* x_zero = reinterpret_cast<uint8_t*>(s_part + kRowsPartFloats);
  const int bpr = p.bpr, K = bpr * kBlock;
  const int wpt = p.wpt, rcp = p.wpt_rcp;                 // quotients by the team size: multiply + shift, as above
  const int tpr = p.tpr;
  const int team = (warp * rcp) >> 16, wi = warp - team * wpt;
  const int u_lo = (bpr * wi * rcp) >> 16, u_hi = (bpr * (wi + 1) * rcp) >> 16;
  const int n_tiles = (p.N + 15) >> 4;
  const int per_round = (int)gridDim.x * tpr;
  const int rounds = p.rounds;
  auto tile_at = [&](int r, int tm) { return r * per_round + tm * (int)gridDim.x + (int)blockIdx.x; };
  auto tile_of = [&](int r) { return tile_at(r, team); };

  int rq_round = 0, rq_u = u_lo, rq_stage = 0, use_stage = 0;
  auto request_one = [&]() {
    while (rq_round < rounds && (rq_u >= u_hi || tile_of(rq_round) >= n_tiles)) { ++rq_round; rq_u = u_lo; }
    if (rq_round < rounds) {
      const uint8_t* src = p.w + ((size_t)tile_of(rq_round) * bpr + rq_u) * F::kBytes;
      uint8_t* dst = ring + rq_stage * F::kBytes;
      constexpr int kChunks = F::kBytes / 16;
#pragma unroll
      for (int i = 0; i < (kChunks + 31) / 32; ++i)
        if (i * 32 + 32 <= kChunks || lane + i * 32 < kChunks) cp_async16(dst + 16 * (lane + i * 32), src + 16 * (lane + i * 32));
      ++rq_u;
    }
    if (++rq_stage == D) rq_stage = 0;
    cp_async_commit();
  };
#pragma unroll 1
  for (int i = 0; i < D - 2; ++i) request_one();
  // (the dependents are released only after this kernel's own dependency is met: a launch behind this one may then
  // read, before ITS wait, anything written two or more launches back — the attention kernel does, see nb_decode.cu)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");

  // ---- the activation rows (and the element-wise step in front of this linear)
  {
    const int wpr = kGW / m;                                // warps per row; 24 % m warps stay idle here
    const int r = warp / wpr, q = warp - r * wpr;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float ss = 0.f;
    if (r < m) {
      const int n4 = K >> 2;
      const int lo = n4 * q / wpr, hi = n4 * (q + 1) / wpr;
      uint8_t* row_s = x_s + r * p.row_bytes;
      if (p.prologue == 1) {
        const float4* xr = reinterpret_cast<const float4*>(p.x) + (size_t)r * n4;
        const float4* dr = p.delta ? reinterpret_cast<const float4*>(p.delta) + (size_t)r * n4 : nullptr;
        const float4* w4 = reinterpret_cast<const float4*>(p.weight);
        float4* xo = (blockIdx.x == 0 && p.x_out) ? reinterpret_cast<float4*>(p.x_out) + (size_t)r * n4 : nullptr;
#pragma unroll 1
        for (int i0 = lo + lane; i0 < hi; i0 += 128) {
          float4 vx[4], vd[4], vw[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {                     // all loads first: one memory round trip per four
            const int i4 = i0 + 32 * j;
            const bool in = i4 < hi;
            vx[j] = in ? __ldcg(xr + i4) : zero4;
            vd[j] = (in && dr) ? __ldcg(dr + i4) : zero4;
            vw[j] = in ? __ldg(w4 + i4) : zero4;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i4 = i0 + 32 * j;
            if (i4 < hi) {
              float4 v = vx[j];
              v.x += vd[j].x; v.y += vd[j].y; v.z += vd[j].z; v.w += vd[j].w;
              if (xo) xo[i4] = v;
              ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
              stage4_row(row_s, p.term_bytes, i4, v.x * vw[j].x, v.y * vw[j].y, v.z * vw[j].z, v.w * vw[j].w);
            }
          }
        }
      } else if (p.prologue == 2) {
        const float4* g4 = reinterpret_cast<const float4*>(p.x) + (size_t)r * 2 * n4;
        const float4* u4 = g4 + n4;
#pragma unroll 1
        for (int i0 = lo + lane; i0 < hi; i0 += 128) {
          float4 vg[4], vu[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i4 = i0 + 32 * j;
            vg[j] = i4 < hi ? __ldcg(g4 + i4) : zero4;
            vu[j] = i4 < hi ? __ldcg(u4 + i4) : zero4;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i4 = i0 + 32 * j;
            const float4 g = vg[j], u = vu[j];
            if (i4 < hi)
              stage4_row(row_s, p.term_bytes, i4, g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y,
                         g.z / (1.f + __expf(-g.z)) * u.z, g.w / (1.f + __expf(-g.w)) * u.w);
          }
        }
      } else {
        const float4* xr = reinterpret_cast<const float4*>(p.x) + (size_t)r * n4;
#pragma unroll 1
        for (int i0 = lo + lane; i0 < hi; i0 += 128) {
          float4 vx[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) vx[j] = i0 + 32 * j < hi ? __ldcg(xr + i0 + 32 * j) : zero4;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (i0 + 32 * j < hi) stage4_row(row_s, p.term_bytes, i0 + 32 * j, vx[j].x, vx[j].y, vx[j].z, vx[j].w);
        }
      }
    }
    ss = warp_sum_f(ss);
    if (lane == 0) s_ss[warp] = ss;
    if (tid < 16) reinterpret_cast<uint32_t*>(x_zero)[tid] = 0u;      // for the MMA columns that carry no row
    __syncthreads();
  }

  // ---- rounds: every team one row tile; a warp adds its units for all rows, the team's sums meet in shared memory
  const int g = lane >> 2, t = lane & 3;
  const bool have = g < m;
  const uint8_t* xrow = x_s + g * p.row_bytes;
  const int term = have ? p.term_bytes : 0;
#pragma unroll 1
  for (int r = 0; r < rounds; ++r) {
    const int tile = tile_of(r);
    float c[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[h][e] = 0.f;
    if (tile < n_tiles) {
#pragma unroll 1
      for (int u = u_lo; u < u_hi; ++u) {
        request_one();
        cp_async_wait<D - 2>();
        __syncwarp();
        const uint8_t* xseg = have ? xrow + (u * 4 + t) * kXSegBytes : x_zero;
        unit_mma_x<BITS, 2>(ring + use_stage * F::kBytes, xseg, term, lane, c);
        if (++use_stage == D) use_stage = 0;
        __syncwarp();
      }
    }
    // lane (g, t) holds weight rows g and g + 8 of columns 2t and 2t + 1 = activation rows 2t, 2t + 1
    float* part = s_part + (r & 1) * (kGW * 128) + warp * 128;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      part[(2 * t + e) * 16 + g] = c[0][e] + c[1][e];
      part[(2 * t + e) * 16 + g + 8] = c[0][2 + e] + c[1][2 + e];
    }
    __syncthreads();                                       // one barrier per round: the buffers alternate
    const float* pr = s_part + (r & 1) * (kGW * 128);
    const int wpr = kGW / m;
    if (p.swiglu) {
      for (int idx = tid; idx < tpr * 8 * m; idx += kThreads) {
        const int tm = idx / (8 * m), rem = idx - tm * 8 * m;
        const int col = rem >> 3, ch = rem & 7;
        const int t_out = tile_at(r, tm);
        float gate = 0.f, up = 0.f;
        for (int j = 0; j < wpt; ++j) {                                          // the team's warps in k order
          gate += pr[(tm * wpt + j) * 128 + col * 16 + ch];
          up += pr[(tm * wpt + j) * 128 + col * 16 + 8 + ch];
        }
        float scale = 1.f;
        if (p.prologue == 1) {
          float tot = 0.f;
          for (int q = 0; q < wpr; ++q) tot += s_ss[col * wpr + q];
          scale = 1.0f / sqrtf(tot / (float)K + p.eps);
        }
        gate *= scale; up *= scale;
        const int c_out = t_out * 8 + ch;
        if (t_out < n_tiles && c_out < (p.N >> 1)) p.y[(size_t)col * (p.N >> 1) + c_out] = gate / (1.f + __expf(-gate)) * up;
      }
      continue;
    }
    for (int idx = tid; idx < tpr * 16 * m; idx += kThreads) {
      const int tm = idx / (16 * m), rem = idx - tm * 16 * m;
      const int col = rem >> 4, row = rem & 15;
      const int t_out = tile_at(r, tm);
      float acc = 0.f;
      for (int j = 0; j < wpt; ++j) acc += pr[(tm * wpt + j) * 128 + col * 16 + row];      // the team's warps in k order
      float scale = 1.f;
      if (p.prologue == 1) {
        float tot = 0.f;
        for (int q = 0; q < wpr; ++q) tot += s_ss[col * wpr + q];
        scale = 1.0f / sqrtf(tot / (float)K + p.eps);
      }
      const int n = t_out * 16 + row;
      if (t_out < n_tiles && n < p.N) p.y[(size_t)col * p.N + n] = acc * scale;
    }
  }
  cp_async_wait<0>();
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
    if ((o.pro == NB_SPRO_EMBED_NORM || o.pro == NB_SPRO_ADD_NORM) && (K > kMaxC || !o.p[3])) return fail("norm prologue needs K <= 2560 and a weight");
    if (o.pro == NB_SPRO_EMBED_NORM && (!o.p[2] || o.i[13] < 1)) return fail("embedding prologue needs a token pointer and the table's row count");
    if (o.epi < NB_SEPI_STORE || o.epi > NB_SEPI_SWIGLU) return fail("unknown epilogue");
    if (o.epi != NB_SEPI_SLOTS && !(o.flags & NB_SOPF_ALIGN)) return fail("only the slot epilogue may split a row tile between CTAs");
    if (o.epi == NB_SEPI_SWIGLU && N % 16 != 0) return fail("SwiGLU epilogue needs N % 16 == 0");
    if ((long long)((N + 15) / 16) * (K / kBlock) >= 65536) return fail("matrix too large for one launch (more than 65535 units)");
    const OpGeom g = geom_of(o, b);
    // a CTA's units of one operation must fit the partial-sum buffer, and the slots must cover every CTA of a row tile
    int worst_slots = 1;
    for (int c = 0; c < G; ++c) {
      int ca, cb;
      cta_range(g, c, G, ca, cb);
      if (cb - ca > kRedUnits) return fail("too many units per CTA for the partial-sum buffer (N * K too large for one launch)");
      if (cb > ca && (cb - 1) / g.bpr - ca / g.bpr + 1 > kMaxLocalTiles) return fail("too many row tiles per CTA");
      if ((cb - ca + kSW - 1) / kSW > (kRedSegs - 1) * g.bpr && (cb - ca + kSW - 1) / kSW > 1)
        return fail("a warp's run of units would touch too many row tiles (K too small for this N)");
    }
    if (!g.align)
      for (int rt = 0; rt < g.rt; ++rt)
        worst_slots = std::max(worst_slots, cta_of_unit((rt + 1) * g.bpr - 1, g.units, G) - cta_of_unit(rt * g.bpr, g.units, G) + 1);
    if (o.epi == NB_SEPI_SLOTS && (o.i[6] < worst_slots || o.i[6] > 16 || o.i[8] < N)) return fail("output slots: need nb_stream_slots(N, K, CTAs) <= slots <= 16 and slot stride >= N");
    *bits = b;
  } else if (o.kind == NB_SOP_ATTN) {
    const int Hl = o.i[0], hd = o.i[1], ctx = o.i[2], S = o.i[3];
    if (Hl < 1 || hd < 4 || hd > 128 || hd % 4 || 3 * hd > kSThreads || ctx < 1 || S < 1) return fail("attention needs head_dim % 4 == 0, <= 128");
    if ((((ctx + S - 1) / S) + 7) > 2048) return fail("more than 2048 keys per attention split");
    for (int j = 0; j < 7; ++j) if (!o.p[j]) return fail("null pointer");
  } else if (o.kind == NB_SOP_HEAD) {
    if (o.i[0] < 1 || o.i[1] < 8 || o.i[1] % 8 || o.i[1] > kMaxC) return fail("head needs C % 8 == 0, <= 2560");
    if (o.i[1] * 2 > 65535) return fail("head row too long");
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

// ---- independent matvecs: plan on the host, run from device memory ----------------------------------
extern "C" size_t nb_group_plan_bytes(const nb_group_item* items, int n_items) {
  if (!items || n_items < 1) return 0;
  long long tiles = 0;
  for (int i = 0; i < n_items; ++i) tiles += items[i].n > 0 ? (items[i].n + 15) / 16 : 0;
  return sizeof(GroupPlan) + (size_t)tiles * sizeof(int);
}

extern "C" int nb_group_max_items(void) { return kGroupMaxItems; }

extern "C" int nb_group_build(const nb_group_item* items, int n_items, int bits, void* plan_out, size_t plan_bytes) {
  auto fail = [&](int index, const char* why) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "nb_group_build: matvec %d: %s", index, why);
    set_last_error(msg);
    return (int)NB_ERR_SHAPE;
  };
  if (!items || !plan_out || n_items < 1) return NB_ERR_ARG;
  if (n_items > kGroupMaxItems) return fail(n_items, "too many matvecs for one launch");
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_SHAPE;
  if (plan_bytes < nb_group_plan_bytes(items, n_items)) return NB_ERR_WORKSPACE;
  GroupPlan* pl = reinterpret_cast<GroupPlan*>(plan_out);
  std::memset(pl, 0, sizeof(GroupPlan));
  const int G = nb_stream_ctas();
  pl->n_items = n_items; pl->bits = bits; pl->ctas = G;
  long long tiles = 0, units = 0;
  int x_bytes = 0;
  for (int i = 0; i < n_items; ++i) {
    const nb_group_item& in = items[i];
    if (!in.w || !in.x || !in.y) return fail(i, "null pointer");
    if ((uintptr_t)in.w % 16 || (uintptr_t)in.x % 16) return fail(i, "weights and activations must be 16-byte aligned");
    if (in.n < 1 || in.k < kBlock || in.k % kBlock || in.k / kBlock > kMaxKBlocks) return fail(i, "needs N >= 1 and K a multiple of 128 up to 7168");
    if (in.x_dtype != NB_F32 && in.x_dtype != NB_F16 && in.x_dtype != NB_BF16) return fail(i, "unknown activation type");
    if (in.y_dtype != NB_F32 && in.y_dtype != NB_F16 && in.y_dtype != NB_BF16) return fail(i, "unknown output type");
    const int m = in.m < 1 ? 1 : in.m;
    if (m > 8) return fail(i, "at most 8 activation rows per matvec");
    if (m > 1 && in.x_dtype == NB_F32) return fail(i, "several activation rows need 16-bit activations");
    int v = 0;
    for (; v < pl->n_x; ++v)
      if (pl->xv[v].ptr == in.x && pl->xv[v].k == in.k && pl->xv[v].dtype == in.x_dtype && pl->xv[v].m == m) break;
    if (v == pl->n_x) {
      if (v == kGroupMaxX) return fail(i, "too many distinct activation vectors for one launch");
      const int xs = in.x_dtype == NB_F32 ? 2 : 1;
      // a vector's terms are kXTermBytes apart (the lookup code's fixed stride); the last term is cut to its length.
      // Rows are one 16-byte chunk more than a row's segments apart: an odd number of chunks, so that the eight
      // lane groups of a warp (one row each) read from different banks.
      const int row = (in.k / kBlock) * 4 * kXSegBytes + 16;
      const int need = m > 1 ? m * row : (xs - 1) * kXTermBytes + (in.k / kBlock) * 4 * kXSegBytes;
      if (x_bytes + need > kGroupSmem - kGroupRingSmall - 128) return fail(i, "the activations of the group do not fit in shared memory");
      pl->xv[v].ptr = in.x; pl->xv[v].k = in.k; pl->xv[v].dtype = in.x_dtype; pl->xv[v].off = x_bytes; pl->xv[v].xs = xs;
      pl->xv[v].m = m; pl->xv[v].row = row;
      x_bytes += (need + 127) / 128 * 128;
      pl->n_x = v + 1;
    }
    GroupItem& it = pl->items[i];
    it.w = reinterpret_cast<const uint8_t*>(in.w); it.y = in.y; it.n = in.n; it.bpr = in.k / kBlock;
    it.tile0 = (int)tiles; it.x_off = pl->xv[v].off; it.xs = pl->xv[v].xs; it.y_dtype = in.y_dtype;
    it.m = m; it.x_row = pl->xv[v].row;
    tiles += (in.n + 15) / 16;
    units += (long long)((in.n + 15) / 16) * it.bpr;
    if (tiles > (1ll << 30)) return fail(i, "too many row tiles");
  }
  pl->total_tiles = (int)tiles;
  // the large ring when the activations leave room for it; 4-bit units are longer and always need it
  pl->ring_bytes = x_bytes <= kGroupXBytes - 128 ? kGroupRing : kGroupRingSmall;
  if (bits == 4 && pl->ring_bytes != kGroupRing) return fail(n_items - 1, "the activations of a 4-bit group must fit 64 KB of shared memory");
  // Deal the row tiles out: longest tiles first, to the CTA that holds the fewest units so far (ties: lowest
  // CTA).  Every CTA's list is then in descending tile length, its share within one short tile of the mean.
  {
    std::vector<int> order(n_items);
    for (int i = 0; i < n_items; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return pl->items[a].bpr > pl->items[b].bpr; });
    std::vector<long long> load(G, 0);
    std::vector<std::vector<int>> lists(G);
    // a min-heap of (units, CTA): all tiles of one matrix have the same length, so they go round the CTAs in turn
    std::priority_queue<std::pair<long long, int>, std::vector<std::pair<long long, int>>, std::greater<>> heap;
    for (int c = 0; c < G; ++c) heap.push({0, c});
    for (int oi = 0; oi < n_items; ++oi) {
      const GroupItem& it = pl->items[order[oi]];
      const int rt = (it.n + 15) / 16;
      for (int t = 0; t < rt; ++t) {
        auto top = heap.top();
        heap.pop();
        lists[top.second].push_back(it.tile0 + t);
        heap.push({top.first + it.bpr, top.second});
      }
    }
    int pos = 0;
    for (int c = 0; c < G; ++c) {
      pl->cta_lo[c] = pos;
      for (int t : lists[c]) pl->tile_list[pos++] = t;
    }
    for (int c = G; c <= kMaxCtas; ++c) pl->cta_lo[c] = pos;
  }
  return NB_OK;
}

extern "C" int nb_group_run(const void* plan_device, const void* plan_host, void* stream) {
  if (!plan_device || !plan_host) return NB_ERR_ARG;
  if ((uintptr_t)plan_device % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const GroupPlan* pl = reinterpret_cast<const GroupPlan*>(plan_host);
  const int bits = pl->bits, G = pl->ctas;
  if ((bits != 2 && bits != 3 && bits != 4) || G < 1 || G > kMaxCtas || pl->n_items < 1 || pl->n_items > kGroupMaxItems) return NB_ERR_ARG;
  if (G != nb_stream_ctas()) { set_last_error("nb_group_run: the plan was built for another device"); return NB_ERR_ARG; }
  int dev = 0;
  cudaGetDevice(&dev);
  const GroupPlan* pd = reinterpret_cast<const GroupPlan*>(plan_device);
  cudaStream_t st = (cudaStream_t)stream;
  const bool big = pl->ring_bytes == kGroupRing;
  if (!big && pl->ring_bytes != kGroupRingSmall) return NB_ERR_ARG;
  const void* fn = bits == 3 ? (big ? (const void*)group_kernel<3, kGW, false, kGroupRing> : (const void*)group_kernel<3, kGW, false, kGroupRingSmall>)
                 : bits == 2 ? (big ? (const void*)group_kernel<2, kGW, false, kGroupRing> : (const void*)group_kernel<2, kGW, false, kGroupRingSmall>)
                             : (const void*)group_kernel<4, kGW, false, kGroupRing>;
  if (bits == 4 && !big) return NB_ERR_ARG;
  const int slot = bits * 2 + (big ? 1 : 0);
  static bool attr_done[64][10] = {};
  if (!attr_done[dev & 63][slot]) {
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kGroupSmem)) return record_cuda_error(e);
    attr_done[dev & 63][slot] = true;
  }
  if (bits == 3 && big) group_kernel<3, kGW, false, kGroupRing><<<G, kGW * 32, kGroupSmem, st>>>(pd);
  else if (bits == 3) group_kernel<3, kGW, false, kGroupRingSmall><<<G, kGW * 32, kGroupSmem, st>>>(pd);
  else if (bits == 2 && big) group_kernel<2, kGW, false, kGroupRing><<<G, kGW * 32, kGroupSmem, st>>>(pd);
  else if (bits == 2) group_kernel<2, kGW, false, kGroupRingSmall><<<G, kGW * 32, kGroupSmem, st>>>(pd);
  else group_kernel<4, kGW, false, kGroupRing><<<G, kGW * 32, kGroupSmem, st>>>(pd);
  return check_launch();
}

// ---- one matrix in a chain of dependent launches --------------------------------------------------
extern "C" int nb_gemv_stream(int prologue, const void* x, int x_dtype, const float* delta, const float* norm_weight, float eps,
                              float* x_out, const uint8_t* w_stream, int bits, int N, int K, float* y, int swiglu, void* stream) {
  if (!x || !w_stream || !y || N < 1) return NB_ERR_ARG;
  if (prologue < 0 || prologue > 2) return NB_ERR_ARG;
  if (swiglu < 0 || swiglu > 7 || ((swiglu & 1) && (swiglu & 4))) return NB_ERR_ARG;
  if ((swiglu & 1) && N % 16 != 0) return NB_ERR_SHAPE;
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_SHAPE;
  if (K < kBlock || K % kBlock != 0 || K / kBlock > kMaxKBlocks) return NB_ERR_SHAPE;
  if (prologue == 1 && !norm_weight) return NB_ERR_ARG;
  if (prologue != 0 && x_dtype != NB_F32) return NB_ERR_ARG;
  if (x_dtype != NB_F32 && x_dtype != NB_F16 && x_dtype != NB_BF16) return NB_ERR_ARG;
  if ((uintptr_t)w_stream % 16 || (uintptr_t)x % 16 || (uintptr_t)delta % 16 || (uintptr_t)norm_weight % 16 || (uintptr_t)x_out % 16)
    return NB_ERR_ALIGN;
  if (x_out && x_out == x) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  TileGemvParams p{};
  p.w = w_stream; p.x = x; p.delta = delta; p.weight = norm_weight; p.x_out = x_out; p.y = y;
  p.N = N; p.bpr = K / kBlock; p.x_dtype = x_dtype; p.prologue = prologue; p.eps = eps; p.swiglu = (swiglu & 1) ? 1 : 0;
  p.accumulate = (swiglu & 4) ? 1 : 0;
  {  // team size: rounds x (units per warp + the round's barrier and sum, about two thirds of a unit)
    const int G = nb_stream_ctas(), n_tiles = (N + 15) / 16;
    double best = 1e30;
    for (int wpt : {24, 12, 6, 3}) {
      const int per_round = G * (kGW / wpt);
      const int rounds = (n_tiles + per_round - 1) / per_round;
      const double cost = rounds * ((p.bpr + wpt - 1) / wpt + 0.67);
      if (cost < best) { best = cost; p.wpt = wpt; p.rounds = rounds; }
    }
    p.tpr = kGW / p.wpt;
    p.wpt_rcp = 65536 / p.wpt + 1;
  }
  const int xs = (x_dtype == NB_F32 && !(swiglu & 2)) ? 2 : 1;      // flag 2: fp32 activations rounded to ONE fp16 term
  const void* fn = nullptr;
  if (bits == 3) fn = xs == 2 ? (const void*)tile_gemv_kernel<3, 2> : (const void*)tile_gemv_kernel<3, 1>;
  else if (bits == 2) fn = xs == 2 ? (const void*)tile_gemv_kernel<2, 2> : (const void*)tile_gemv_kernel<2, 1>;
  else fn = xs == 2 ? (const void*)tile_gemv_kernel<4, 2> : (const void*)tile_gemv_kernel<4, 1>;
  static bool attr_done[64][12] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int slot = bits * 2 + xs - 1;
  if (!attr_done[dev & 63][slot]) {
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileSmem)) return record_cuda_error(e);
    attr_done[dev & 63][slot] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nb_stream_ctas());
  cfg.blockDim = dim3(kGW * 32);
  cfg.dynamicSmemBytes = kTileSmem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void* args[] = {&p};
  return record_cuda_error(cudaLaunchKernelExC(&cfg, fn, args));
}

// shared memory of tile_gemv_rows_kernel for m rows of K activations (0: bad arguments)
static size_t rows_smem_bytes(int bits, int K, int m) {
  if ((bits != 2 && bits != 3 && bits != 4) || K < kBlock || K % kBlock != 0 || K / kBlock > kMaxKBlocks || m < 1 || m > 8) return 0;
  const size_t unit = bits == 4 ? UnitFmt<4>::kBytes : UnitFmt<3>::kBytes;
  const size_t term = (size_t)(K / kBlock) * 4 * kXSegBytes;
  return (size_t)kGW * kRowsD * unit + (size_t)m * (2 * term + 16) + (size_t)kRowsPartFloats * 4 + 64;
}
constexpr size_t kRowsSmemLimit = 227 * 1024 - 256;         // per CTA, less the kernel's static shared memory

extern "C" int nb_gemv_stream_max_rows(int bits, int K) {
  int best = 0;
  for (int m = 1; m <= 8; ++m) {
    const size_t need = rows_smem_bytes(bits, K, m);
    if (need != 0 && need <= kRowsSmemLimit) best = m;
  }
  return best;
}

extern "C" int nb_gemv_stream_rows(int prologue, const float* x, int M, const float* delta, const float* norm_weight, float eps,
                                   float* x_out, const uint8_t* w_stream, int bits, int N, int K, float* y, int swiglu, void* stream) {
  if (!x || !w_stream || !y || N < 1 || M < 1) return NB_ERR_ARG;
  if (prologue < 0 || prologue > 2 || swiglu < 0 || swiglu > 1) return NB_ERR_ARG;
  if (swiglu && N % 16 != 0) return NB_ERR_SHAPE;
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_SHAPE;
  if (K < kBlock || K % kBlock != 0 || K / kBlock > kMaxKBlocks) return NB_ERR_SHAPE;
  if (M > nb_gemv_stream_max_rows(bits, K)) return NB_ERR_SHAPE;
  if (prologue == 1 && !norm_weight) return NB_ERR_ARG;
  if ((uintptr_t)w_stream % 16 || (uintptr_t)x % 16 || (uintptr_t)delta % 16 || (uintptr_t)norm_weight % 16 || (uintptr_t)x_out % 16)
    return NB_ERR_ALIGN;
  if (x_out && x_out == x) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  TileRowsParams p{};
  p.w = w_stream; p.x = x; p.delta = delta; p.weight = norm_weight; p.x_out = x_out; p.y = y;
  p.N = N; p.bpr = K / kBlock; p.prologue = prologue; p.m = M; p.eps = eps; p.swiglu = swiglu;
  p.term_bytes = p.bpr * 4 * kXSegBytes;
  p.row_bytes = 2 * p.term_bytes + 16;
  {
    const int G = nb_stream_ctas(), n_tiles = (N + 15) / 16;
    double best = 1e30;
    for (int wpt : {24, 12, 6, 3}) {
      const int per_round = G * (kGW / wpt);
      const int rounds = (n_tiles + per_round - 1) / per_round;
      const double cost = rounds * ((p.bpr + wpt - 1) / wpt + 0.67);
      if (cost < best) { best = cost; p.wpt = wpt; p.rounds = rounds; }
    }
    p.tpr = kGW / p.wpt;
    p.wpt_rcp = 65536 / p.wpt + 1;
  }
  const void* fn = bits == 3 ? (const void*)tile_gemv_rows_kernel<3> : bits == 2 ? (const void*)tile_gemv_rows_kernel<2>
                                                                                 : (const void*)tile_gemv_rows_kernel<4>;
  const size_t smem = rows_smem_bytes(bits, K, M);
  static size_t attr_bytes[64][5] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_bytes[dev & 63][bits] < smem) {
    if (cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRowsSmemLimit)) return record_cuda_error(e);
    attr_bytes[dev & 63][bits] = kRowsSmemLimit;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nb_stream_ctas());
  cfg.blockDim = dim3(kGW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void* args[] = {&p};
  return record_cuda_error(cudaLaunchKernelExC(&cfg, fn, args));
}

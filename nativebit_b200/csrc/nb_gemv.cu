// Fused decode GEMV / skinny GEMM for NativeBit packed linears on sm_100a (M = 1..16 rows).
//
// Data movement.  A CTA owns `tr` row tiles (16 output rows each) x one contiguous range of
// k-blocks.  In its first cycles every thread issues 16-byte asynchronous copies (cp.async,
// L2 -> shared, no register or L1 staging) for the CTA's index rows and codebook rows,
// consecutive threads on consecutive chunks of a row, and posts one deferred arrival per row
// tile on that tile's mbarrier: every byte the CTA will read from HBM is requested before
// anything else happens, and a warp can start on a row tile as soon as that tile has landed.
// When the CTA covers whole rows (no k split) the 16 rows of a tile are one contiguous span and
// are fetched instead by two bulk copies (cp.async.bulk, the 1-D form of TMA) issued by one
// lane, which blocks no warp; one bulk copy per 960-byte row was measured at about 30 ns of
// issue time per copy, which is why the split-k case uses the 16-byte copies.  The kernel is
// launched with programmatic stream serialization: after requesting its weights it lets the
// next launch of the stream begin (which requests its own weights) and only then waits for
// the previous kernel, whose output may be this kernel's x.
//
// Compute.  A "unit" is 16 rows x 4 k-blocks: lane (g, t) (g = lane/4, t = lane%4) owns the
// 128-weight block of row g and of row g+8 at k-block 4*kgroup+t.  It reads its two 48-byte
// index blocks and 16-byte codebooks from shared memory (conflict free: row stride is 64 mod
// 128 bytes), turns the packed 3-bit fields into nibble selectors with a few mask operations
// (nb_common.cuh) and gathers four fp16 weights per pair of byte-permutes from a low-byte and a
// high-byte plane of the codebook held in registers.  Four weights of row g and four of row
// g+8 form the A fragment of one m16n8k16 tensor-core MMA whose B fragment is the matching
// four activations of up to 8 batch rows: fp16 x fp16 products are exact, accumulation is
// fp32, and the multiply-accumulate costs one instruction per 256 weights, leaving the issue
// slots to the unpack.  Weights are consumed in "slot" order rather than position order, so
// the activation tile is staged into shared memory once per CTA in that order, as fp16.
//
// Reduction.  Every unit stores its 16 x 8 partial tile into its own shared-memory slot and the
// slots of a row tile are added in k order.  When the k range is split over several CTAs
// (grid.y > 1) each CTA writes its partial tile to scratch and takes a ticket; the CTA that takes
// the last ticket adds the partials in fixed order, writes y and resets the counter.  No sum
// depends on which warp or CTA finished first: results are bit-identical from run to run, and the
// scratch needs no clearing between launches.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>
#include <cstdio>
#include <mutex>

#include "nb_common.cuh"
#include "nb_device.cuh"
#include "nb_host.h"

// Optional phase tracing for tuning builds (-DNB_TRACE): block 0..63 thread 0 stores %globaltimer.
#ifdef NB_TRACE
__device__ unsigned long long nb_trace_buf[64 * 8];
#define NB_TRACE_MARK(i)                                                                  \
  do {                                                                                    \
    if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x < 64) {                         \
      unsigned long long t_;                                                              \
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                               \
      nb_trace_buf[blockIdx.x * 8 + (i)] = t_;                                            \
    }                                                                                     \
  } while (0)
extern "C" int nb_trace_read(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, nb_trace_buf, sizeof(nb_trace_buf));
}
#else
#define NB_TRACE_MARK(i) do {} while (0)
#endif

namespace nb {

constexpr int kMaxWarps = 16;
constexpr int kMaxTr = 16;                      // row tiles per CTA (one mbarrier each)
// Bytes of one k-block of an activation tile of XR rows (32 steps x XR rows x 4 fp16), plus a skew
// that spreads the four k-blocks read by lanes t = 0..3 over different banks.
__host__ __device__ constexpr int x_block_bytes(int xr) { return 32 * xr * 8 + (xr == 8 ? 32 : 8); }
constexpr int kMaxSmem = 110 * 1024;            // two CTAs (of consecutive launches) fit one SM
constexpr int kCounterInts = 4096;              // workspace head: ticket counters + status word
constexpr uint32_t kSpinLimit = 1u << 21;       // bounded wait on the copy barriers (about 0.1 s with the back-off)

struct GemvPlan {
  int tr;           // row tiles (of 16 rows) per CTA
  int parts;        // k partitions = grid.y
  int kg_per_part;  // k-groups (of 4 blocks) per partition
  int grid_x;
  int warps;
  size_t smem;
  int w_stride, c_stride;
};

// Kernel parameter block.  Kept small on purpose: together with GemvExtra it stays within 128
// bytes (measured on B200: a launch whose parameters exceed 128 bytes costs 0.4 to 0.8 us more
// inside a dependent chain).  The kernel expands it into a GemvView with one plain field per value.
struct GemvParams {
  const void* x;
  const uint8_t* packed;
  const void* codebook;
  void* y;
  int* counters;            // workspace head: ticket counters, status word at int kCounterInts - 1, then the partial tiles (may be null)
  int N;
  int w_stride, c_stride;   // shared-memory row strides (bytes) of the index and codebook tiles
  uint16_t bpr, kg_per_part;
  uint8_t M, tr;
  uint8_t dtypes;           // x_dtype | y_dtype << 2 | cb_dtype << 4
  uint8_t flags;            // x_vec | cb_bulk << 1 | tile_bulk << 2
};
static_assert(sizeof(GemvParams) <= 64, "keep the GEMV parameter block small");

struct GemvView {
  const void* x;
  const uint8_t* packed;
  const void* codebook;
  void* y;
  float* scratch;
  int* counters;
  int* status;      // set to NB_ERR_TIMEOUT if a bounded wait runs out (may be null)
  int M, N, bpr, row_tiles, kgroups;
  int tr, kg_per_part;
  int x_dtype, y_dtype, cb_dtype;
  int x_vec;        // x is 16-byte aligned: staged with 16-byte loads
  int w_stride, c_stride;
  int cb_bulk;      // codebook rows are whole 16-byte chunks (else they are fetched with 8-byte loads)
  int tile_bulk;    // the CTA covers whole rows: a row tile is one contiguous span, fetched by bulk copies
  __device__ __forceinline__ explicit GemvView(const GemvParams& q)
      : x(q.x), packed(q.packed), codebook(q.codebook), y(q.y),
        scratch(q.counters ? reinterpret_cast<float*>(q.counters + kCounterInts) : nullptr), counters(q.counters),
        status(q.counters ? q.counters + (kCounterInts - 1) : nullptr), M(q.M), N(q.N), bpr(q.bpr), row_tiles((q.N + 15) >> 4),
        kgroups((q.bpr + 3) >> 2), tr(q.tr), kg_per_part(q.kg_per_part), x_dtype(q.dtypes & 3), y_dtype((q.dtypes >> 2) & 3),
        cb_dtype((q.dtypes >> 4) & 3), x_vec(q.flags & 1), w_stride(q.w_stride), c_stride(q.c_stride), cb_bulk((q.flags >> 1) & 1),
        tile_bulk((q.flags >> 2) & 1) {}
};

// Arguments of the activation prologues and of the tensor-parallel exchange.  Kernels without
// either take an empty struct instead, which keeps their parameter block small.
struct GemvExtra {
  const float* pro_delta;   // PRO 1: added to x before the norm (may be null)
  const float* pro_weight;  // PRO 1: RMSNorm weight (K)
  float* pro_x_out;         // PRO 1: receives x + delta (M, K) (may be null; must not alias x)
  float pro_eps;
  uint32_t xchg_spin;       // bound of the wait for the peers' vectors
  uint8_t* xchg_self;       // tensor-parallel exchange (see nb_gemv_tp): this rank's exchange buffer
  int xchg_world, xchg_rank, xchg_max_count;
  int gather;               // PRO 1: delta = sum over the ranks of the vectors pushed last
};
static_assert(sizeof(GemvParams) + sizeof(GemvExtra) <= 128, "keep the GEMV parameter block within 128 bytes");
struct GemvNoExtra {
  static constexpr const float* pro_delta = nullptr;
  static constexpr const float* pro_weight = nullptr;
  static constexpr float* pro_x_out = nullptr;
  static constexpr float pro_eps = 0.f;
  static constexpr uint8_t* xchg_self = nullptr;
  static constexpr int xchg_world = 0, xchg_rank = 0, xchg_max_count = 0, gather = 0;
  static constexpr uint32_t xchg_spin = 0;
};
template <bool kUsed> struct ExtraSel { using type = GemvExtra; };
template <> struct ExtraSel<false> { using type = GemvNoExtra; };

// Exchange buffer of one rank (the same layout on every rank):
//   slots  [2 sets][world][max_count] fp32   slot r of a set is written by rank r (all of its CTAs)
//   flags  [2 sets][world] uint32            written by rank r after its slot is complete: sequence number
//   seq    uint32, ticket int                private to the owner: vectors pushed so far; CTA ticket counter
//   table  [8] uint64                        every rank's buffer as mapped into the owner's process (nb_exchange_init)
// Pushes alternate between the two sets.  A rank can be at most one push ahead of the slowest rank
// (between two of its pushes it consumes a sum, which needs every rank's flag), so a set is never
// overwritten while a peer still reads it.  The counters live in device memory: a captured CUDA
// graph stays replayable.  The peer pointers live there too, not in the kernel parameters.
__host__ __device__ inline size_t xchg_slots_bytes(int world, int max_count) { return (size_t)2 * world * max_count * sizeof(float); }
__host__ __device__ inline uint32_t* xchg_flags(const uint8_t* buf, int world, int max_count) {
  return reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(buf) + xchg_slots_bytes(world, max_count));
}
__host__ __device__ inline uint32_t* xchg_seq(const uint8_t* buf, int world, int max_count) {
  return xchg_flags(buf, world, max_count) + 2 * world;
}
__host__ __device__ inline unsigned long long* xchg_table(const uint8_t* buf, int world, int max_count) {
  return reinterpret_cast<unsigned long long*>(xchg_flags(buf, world, max_count) + 2 * world + 2);  // 2*world + 2 words: 8-byte aligned
}
__host__ __device__ inline size_t xchg_bytes(int world, int max_count) {
  return xchg_slots_bytes(world, max_count) + (size_t)(2 * world + 2) * sizeof(uint32_t) + 8 * sizeof(unsigned long long);
}

// XR = activation rows held per tile: 8, or 1 for a single activation vector (all eight B
// columns then read the same row, so the tile is 8x smaller and column 0 carries the result).
// XS = fp16 terms per activation: 1, or 2 for fp32 activations, which are carried as hi + lo fp16
// parts (x = fp16(x) + fp16(x - fp16(x)), about 22 significant bits) and contracted by two MMAs
// into the same accumulator, so that fp32 inputs are not rounded to 11 bits.
//
// PRO = activation prologue, computed while the activations are staged (fp32 activations only):
//   0  none: the activation is x[m, k].
//   1  residual add + RMSNorm: v = x[m, :] + delta[m, :]; activation = v[k] / sqrt(mean(v^2) + eps) * weight[k].
//      Every CTA reads the whole rows once to form the mean (a fixed assignment of row segments to
//      warps and a fixed summation order: all CTAs get the same bits), CTA (0, 0) writes v to x_out.
//   2  SwiGLU: x is (M, 2K) = [gate | up]; activation = silu(gate[m, k]) * up[m, k].
// PUSH = 1: the result goes to the ranks' exchange buffers instead of y (see nb_gemv_tp).
template <int BITS, int NT, int XR, int XS, int PRO, int PUSH>
__global__ void __launch_bounds__(kMaxWarps * 32, 2) gemv_kernel(const GemvParams pp, const typename ExtraSel<(PRO != 0 || PUSH != 0)>::type ex) {
  const GemvView p(pp);
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kWords = Fmt<BITS>::kWords;
  constexpr int kBlkBytes = 16 * BITS;
  constexpr int kXBlockBytes = x_block_bytes(XR);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n_warps = blockDim.x >> 5, n_threads = blockDim.x;

  const int rt0 = blockIdx.x * p.tr;
  const int rt_n = min(p.tr, p.row_tiles - rt0);
  const int kg0 = blockIdx.y * p.kg_per_part;
  const int kg_n = min(p.kg_per_part, p.kgroups - kg0);
  const int kb0 = kg0 * 4;
  const int kb_n = min(kg_n * 4, p.bpr - kb0);
  const int n_units = rt_n * kg_n;
  const int K = p.bpr * kBlock;
  const int cb_blk = (p.cb_dtype == NB_F16 ? 2 : 4) << BITS;  // codebook bytes per block

  // shared memory: index rows | codebook rows | activation tile(s) | fp32 accumulator | per-unit tiles | slot offsets
  const int x_tile_bytes = p.kg_per_part * 4 * kXBlockBytes;
  uint8_t* w_s = smem;
  uint8_t* c_s = w_s + p.tr * 16 * p.w_stride;
  uint8_t* x_s = c_s + p.tr * 16 * p.c_stride;
  float* acc = reinterpret_cast<float*>(x_s + NT * XS * x_tile_bytes);
  const int acc_n = p.tr * 16 * NT * 8;
  constexpr int kUnitCols = XR == 1 ? 1 : NT * 8;                 // a single activation row only has column 0
  constexpr int kUnitTile = 16 * kUnitCols;
  float* unit_acc = acc + acc_n;                                  // one 16 x kUnitCols tile per unit
  uint16_t* dst_off = reinterpret_cast<uint16_t*>(unit_acc + (((size_t)p.tr * p.kg_per_part * kUnitTile + 3) & ~(size_t)3));  // position -> offset (halves) inside a k-block tile
  __shared__ __align__(8) uint64_t bars[kMaxTr];
  __shared__ int s_last;
  __shared__ float s_red[PRO == 1 ? 8 * kMaxWarps : 1];  // PRO 1: partial sums of squares [row][segment]
  __shared__ float s_scale[PRO == 1 ? 8 : 1];            // PRO 1: 1/rms of each activation row
  __shared__ unsigned long long s_peer[PUSH ? 8 : 1];    // PUSH: every rank's exchange buffer
  __shared__ uint32_t s_push_seq;                        // PUSH: sequence number of this push

  NB_TRACE_MARK(0);
  if (tid < rt_n) mbar_init(&bars[tid], p.tile_bulk ? 1 : n_threads);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  // ---- request every byte of weights and codebooks this CTA needs (constant data: no need to
  // wait for earlier kernels) with 16-byte asynchronous copies, consecutive threads on
  // consecutive chunks of a row; each thread then posts one deferred arrival per row tile
  // that fires when its copies of that tile have landed.
  if (p.tile_bulk) {
    // Whole rows: the 16 rows of a tile are contiguous in global memory, so lane 0 of warp j
    // fetches tile j (j + n_warps, ...) with one bulk copy for indices and one for codebooks.
    if (lane == 0) {
      for (int rtl = warp; rtl < rt_n; rtl += n_warps) {
        const size_t row = (size_t)(rt0 + rtl) * 16;
        const uint32_t rows = (uint32_t)min((size_t)16, (size_t)p.N - row);
        const uint32_t wb = rows * (uint32_t)p.w_stride, cbb = rows * (uint32_t)p.c_stride;
        mbar_arrive_expect_tx(&bars[rtl], wb + cbb);
        bulk_g2s(w_s + rtl * 16 * p.w_stride, p.packed + row * p.bpr * kBlkBytes, wb, &bars[rtl]);
        bulk_g2s(c_s + rtl * 16 * p.c_stride, reinterpret_cast<const uint8_t*>(p.codebook) + row * p.bpr * cb_blk, cbb, &bars[rtl]);
      }
    }
  } else {
    const int wch = kb_n * kBlkBytes / 16;                    // 16-byte chunks per index row
    const int cch = p.cb_bulk ? kb_n * cb_blk / 16 : 0;       // ... per codebook row
    const uint8_t* cbase = reinterpret_cast<const uint8_t*>(p.codebook);
    for (int rtl = 0; rtl < rt_n; ++rtl) {
      for (int lr = warp; lr < 16; lr += n_warps) {           // one warp per row
        const int r = rtl * 16 + lr;
        const size_t row = (size_t)rt0 * 16 + r;
        if (row < (size_t)p.N) {
          const size_t blk0 = row * p.bpr + kb0;
          const uint8_t* wsrc = p.packed + blk0 * kBlkBytes;
          uint8_t* wdst = w_s + r * p.w_stride;
          for (int j = lane; j < wch; j += 32) cp_async16(wdst + 16 * j, wsrc + 16 * j);
          const uint8_t* csrc = cbase + blk0 * cb_blk;
          uint8_t* cdst = c_s + r * p.c_stride;
          for (int j = lane; j < cch; j += 32) cp_async16(cdst + 16 * j, csrc + 16 * j);
        }
      }
      cp_async_arrive(&bars[rtl]);
    }
  }
  if (!p.cb_bulk && !p.tile_bulk) {
    // codebook rows that are not 16-byte granular (2-bit fp16 with an odd block count): 8-byte loads
    const int gpr = kb_n * cb_blk / 8;  // granules per row
    for (int i = tid; i < rt_n * 16 * gpr; i += n_threads) {
      const int r = i / gpr, j = i - r * gpr;
      const size_t row = (size_t)rt0 * 16 + r;
      if (row < (size_t)p.N)
        *reinterpret_cast<uint2*>(c_s + r * p.c_stride + 8 * j) =
            __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.codebook) + (row * p.bpr + kb0) * cb_blk) + j);
    }
  }
  NB_TRACE_MARK(1);

  if (tid < kBlock) {
    const int slot = tid, pos = slot_to_position<BITS>(slot);
    dst_off[pos] = (uint16_t)((slot >> 2) * (XR * 4) + (slot & 3));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // dependents are released only now: a launch behind this one may read, before its own wait, what was written two
  // or more launches back (the attention kernel prefetches cached keys and values that way)
  asm volatile("griddepcontrol.launch_dependents;");
  NB_TRACE_MARK(2);
  if (PUSH) {
    // peer pointers and the sequence number of this push: requested now, used after the units, so
    // their latency is hidden (the barrier after the activation staging publishes them)
    if (tid < ex.xchg_world) s_peer[tid] = __ldg(xchg_table(ex.xchg_self, ex.xchg_world, ex.xchg_max_count) + tid);
    if (tid == 32) s_push_seq = __ldcg(xchg_seq(ex.xchg_self, ex.xchg_world, ex.xchg_max_count)) + 1;
  }
  __syncthreads();

  // ---- stage x as fp16 in slot order: x_s[tile m/XR][k-block][step][row m%XR][4].  A thread owns
  // 8-position chunks: it decodes the eight destination offsets once, then for four activation
  // rows at a time loads 8 values each (all loads first), converts pairs with one saturating
  // f32->f16x2 conversion and scatters them; rows differ only by a constant offset.
  if (PRO == 1) {
    // One pass over the whole rows: v = x + delta (delta either a local vector or the sum over the
    // ranks' pushed vectors), sum of squares, and v * weight staged (as fp16 hi + lo) where the
    // column lies in this CTA's k range; the factor 1/rms is a scalar per row and is applied to the
    // output.  A row is cut into segments, one per warp of the row's group, and the segment sums are
    // added in a fixed order: every CTA (and every rank) computes the same bits.
    const float* slots = nullptr;  // [world][max_count] vectors pushed by the ranks, if gathering
    if (ex.gather) {
      const uint8_t* self = ex.xchg_self;
      const uint32_t seq = __ldcg(xchg_seq(self, ex.xchg_world, ex.xchg_max_count));  // vectors pushed so far = the one to collect
      const int set = seq & 1;
      if (tid < ex.xchg_world) {
        const uint32_t* flag = xchg_flags(self, ex.xchg_world, ex.xchg_max_count) + set * ex.xchg_world + tid;
        // a wait that already ran out once is not repeated by later launches: the step finishes quickly
        // and the host finds the status word
        uint32_t spins = (p.status && *reinterpret_cast<volatile int*>(p.status) == (int)NB_ERR_TIMEOUT) ? ex.xchg_spin : 0;
        while (ld_acquire_sys_u32(flag) != seq) {
          __nanosleep(100);
          if (++spins > ex.xchg_spin) {
            if (p.status) atomicExch(p.status, (int)NB_ERR_TIMEOUT);
            break;
          }
        }
      }
      __syncthreads();
      slots = reinterpret_cast<const float*>(self) + (size_t)set * ex.xchg_world * ex.xchg_max_count;
    }
    int mp = 1;
    while (mp < p.M) mp <<= 1;
    const int wpr = max(1, n_warps / mp);           // warps per row
    const int rows_per_round = n_warps / wpr;
    const int seg = warp % wpr;
    const bool writer = blockIdx.x == 0 && blockIdx.y == 0 && ex.pro_x_out != nullptr;
    for (int m = warp / wpr; m < p.M; m += rows_per_round) {
      const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (size_t)m * K);
      const float4* dr = ex.pro_delta ? reinterpret_cast<const float4*>(ex.pro_delta + (size_t)m * K) : nullptr;
      __half* xrow = reinterpret_cast<__half*>(x_s) + (m / XR) * XS * (x_tile_bytes / 2) + (m % XR) * 4;
      float ss = 0.f;
      const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
      auto load_v = [&](int i) {  // x + delta at float4 index i of row m
        float4 v = xr[i];
        if (slots) {
          float4 d = zero4;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (q < ex.xchg_world) {
              const float4 e = __ldcv(reinterpret_cast<const float4*>(slots + (size_t)q * ex.xchg_max_count + (size_t)m * K) + i);
              d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
            }
          }
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        } else if (dr) {
          const float4 d = dr[i];
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        return v;
      };
      auto in_range = [&](int i) { const int kbl = (i >> 5) - kb0; return kbl >= 0 && kbl < kb_n; };  // 32 float4 per k-block
      auto consume = [&](int i, const float4& v, const float4& w4) {
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (writer) reinterpret_cast<float4*>(ex.pro_x_out + (size_t)m * K)[i] = v;
        if (in_range(i)) {
          const int kbl = (i >> 5) - kb0;
          const float u0 = v.x * w4.x, u1 = v.y * w4.y, u2 = v.z * w4.z, u3 = v.w * w4.w;
          const uint2 o2 = *reinterpret_cast<const uint2*>(dst_off + ((i & 31) << 2));
          uint16_t* blk = reinterpret_cast<uint16_t*>(xrow + kbl * (kXBlockBytes / 2));
          const uint32_t h01 = f32x2_to_f16x2_sat(u0, u1), h23 = f32x2_to_f16x2_sat(u2, u3);
          blk[o2.x & 0xFFFFu] = (uint16_t)(h01 & 0xFFFFu); blk[o2.x >> 16] = (uint16_t)(h01 >> 16);
          blk[o2.y & 0xFFFFu] = (uint16_t)(h23 & 0xFFFFu); blk[o2.y >> 16] = (uint16_t)(h23 >> 16);
          if (XS == 2) {
            const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
            const float2 r23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
            const uint32_t l01 = f32x2_to_f16x2_sat(fminf(fmaxf(u0, -65504.f), 65504.f) - r01.x, fminf(fmaxf(u1, -65504.f), 65504.f) - r01.y);
            const uint32_t l23 = f32x2_to_f16x2_sat(fminf(fmaxf(u2, -65504.f), 65504.f) - r23.x, fminf(fmaxf(u3, -65504.f), 65504.f) - r23.y);
            uint16_t* lo = blk + x_tile_bytes / 2;
            lo[o2.x & 0xFFFFu] = (uint16_t)(l01 & 0xFFFFu); lo[o2.x >> 16] = (uint16_t)(l01 >> 16);
            lo[o2.y & 0xFFFFu] = (uint16_t)(l23 & 0xFFFFu); lo[o2.y >> 16] = (uint16_t)(l23 >> 16);
          }
        }
      };
      // two segments per iteration, all loads first: a row costs one memory round trip per two steps
      const int stride = wpr * 32;
      for (int i0 = seg * 32 + lane; i0 < K / 4; i0 += 2 * stride) {
        const int i1 = i0 + stride;
        const bool has1 = i1 < K / 4;
        const float4 v0 = load_v(i0);
        const float4 v1 = has1 ? load_v(i1) : zero4;
        const float4 w0 = in_range(i0) ? reinterpret_cast<const float4*>(ex.pro_weight)[i0] : zero4;
        const float4 w1 = (has1 && in_range(i1)) ? reinterpret_cast<const float4*>(ex.pro_weight)[i1] : zero4;
        consume(i0, v0, w0);
        if (has1) consume(i1, v1, w1);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_red[m * kMaxWarps + seg] = ss;
    }
    // k-blocks past the end of the row are staged as zeros (their weights are zero; 0 x garbage must not be NaN)
    const int tail = kg_n * 4 - kb_n;
    for (int i = tid; i < tail * kBlock * p.M; i += n_threads) {
      const int m = i / (tail * kBlock), j = i - m * (tail * kBlock);
      const int kbl = kb_n + (j >> 7), pos = j & 127;
      uint16_t* blk = reinterpret_cast<uint16_t*>(reinterpret_cast<__half*>(x_s) + (m / XR) * XS * (x_tile_bytes / 2) + (m % XR) * 4 +
                                                  kbl * (kXBlockBytes / 2));
      blk[dst_off[pos]] = 0;
      if (XS == 2) blk[x_tile_bytes / 2 + dst_off[pos]] = 0;
    }
    __syncthreads();
    if (tid < p.M) {
      float tot = 0.f;
      for (int j = 0; j < wpr; ++j) tot += s_red[tid * kMaxWarps + j];
      s_scale[tid] = 1.0f / sqrtf(tot / (float)K + ex.pro_eps);
    }
  } else if (PRO == 2) {
    // SwiGLU: a thread owns 8-position chunks and handles two of them at a time (all loads first), one
    // activation row after the other
    const int chunks = kg_n * 4 * 16;
    for (int c0 = tid; c0 < chunks; c0 += 2 * n_threads) {
#pragma unroll 1
      for (int m = 0; m < p.M; ++m) {
        float4 gv[2][2], uv[2][2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int c = c0 + b * n_threads;
          gv[b][0] = gv[b][1] = uv[b][0] = uv[b][1] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < chunks && (c >> 4) < kb_n) {  // k-blocks past the end of the row are staged as zeros
            const float* gr = reinterpret_cast<const float*>(p.x) + (size_t)m * 2 * K + (size_t)kb0 * kBlock + (size_t)c * 8;
            gv[b][0] = *reinterpret_cast<const float4*>(gr); gv[b][1] = *reinterpret_cast<const float4*>(gr + 4);
            uv[b][0] = *reinterpret_cast<const float4*>(gr + K); uv[b][1] = *reinterpret_cast<const float4*>(gr + K + 4);
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int c = c0 + b * n_threads;
          if (c < chunks) {
            const float gg[8] = {gv[b][0].x, gv[b][0].y, gv[b][0].z, gv[b][0].w, gv[b][1].x, gv[b][1].y, gv[b][1].z, gv[b][1].w};
            const float uu[8] = {uv[b][0].x, uv[b][0].y, uv[b][0].z, uv[b][0].w, uv[b][1].x, uv[b][1].y, uv[b][1].z, uv[b][1].w};
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = gg[j] / (1.0f + __expf(-gg[j])) * uu[j];
            const uint4 o4 = *reinterpret_cast<const uint4*>(dst_off + ((c & 15) << 3));
            const uint32_t o[4] = {o4.x, o4.y, o4.z, o4.w};
            uint16_t* blk = reinterpret_cast<uint16_t*>(reinterpret_cast<__half*>(x_s) + (c >> 4) * (kXBlockBytes / 2) +
                                                        (m / XR) * XS * (x_tile_bytes / 2) + (m % XR) * 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t hi = f32x2_to_f16x2_sat(v[2 * j], v[2 * j + 1]);
              const uint32_t oa = o[j] & 0xFFFFu, ob = o[j] >> 16;
              blk[oa] = (uint16_t)(hi & 0xFFFFu);
              blk[ob] = (uint16_t)(hi >> 16);
              if (XS == 2) {
                const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                const uint32_t lo = f32x2_to_f16x2_sat(fminf(fmaxf(v[2 * j], -65504.f), 65504.f) - rr.x,
                                                       fminf(fmaxf(v[2 * j + 1], -65504.f), 65504.f) - rr.y);
                blk[(x_tile_bytes / 2) + oa] = (uint16_t)(lo & 0xFFFFu);
                blk[(x_tile_bytes / 2) + ob] = (uint16_t)(lo >> 16);
              }
            }
          }
        }
      }
    }
  } else {
    // A thread handles four (chunk, row) items at a time: the raw loads of all four first (nothing
    // consumes them yet), then the conversions, so that the items' memory round trips overlap instead
    // of following one another.  Several rows: the items are four rows of one 8-position chunk.  A
    // single row (XR == 1): they are four chunks, which stages a long row in one round trip.
    const int chunks = kg_n * 4 * 16;  // 8-position chunks per activation row
    const int c_step = XR == 1 ? 4 * n_threads : n_threads;
    const int m_rounds = XR == 1 ? 1 : (p.M + 3) / 4;
    for (int c0 = tid; c0 < chunks; c0 += c_step) {
      // several rows: the four items share the chunk, whose destination offsets are read once
      const uint4 o4_chunk = XR == 1 ? make_uint4(0u, 0u, 0u, 0u) : *reinterpret_cast<const uint4*>(dst_off + ((c0 & 15) << 3));
      for (int r = 0; r < m_rounds; ++r) {
        uint4 raw[4][2];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int c = XR == 1 ? c0 + b * n_threads : c0;
          const int m = XR == 1 ? 0 : 4 * r + b;
          raw[b][0] = raw[b][1] = make_uint4(0u, 0u, 0u, 0u);
          // k-blocks past the end of the row are staged as zeros: their weights are zero, and
          // 0 x garbage must not be NaN
          if (c < chunks && (c >> 4) < kb_n && m < p.M) {
            const size_t at = (size_t)m * K + (size_t)kb0 * kBlock + (size_t)c * 8;
            if (p.x_vec) {
              if (p.x_dtype == NB_F32) {
                raw[b][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.x) + at);
                raw[b][1] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.x) + at + 4);
              } else {
                raw[b][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.x) + at);
              }
            } else {
              float t[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) t[j] = load_x(p.x, NB_F32 == p.x_dtype ? NB_F32 : p.x_dtype, at + j);
              if (p.x_dtype == NB_F32) {
                raw[b][0] = make_uint4(__float_as_uint(t[0]), __float_as_uint(t[1]), __float_as_uint(t[2]), __float_as_uint(t[3]));
                raw[b][1] = make_uint4(__float_as_uint(t[4]), __float_as_uint(t[5]), __float_as_uint(t[6]), __float_as_uint(t[7]));
              } else if (p.x_dtype == NB_BF16) {
                raw[b][0] = make_uint4((__float_as_uint(t[0]) >> 16) | (__float_as_uint(t[1]) & 0xFFFF0000u),
                                       (__float_as_uint(t[2]) >> 16) | (__float_as_uint(t[3]) & 0xFFFF0000u),
                                       (__float_as_uint(t[4]) >> 16) | (__float_as_uint(t[5]) & 0xFFFF0000u),
                                       (__float_as_uint(t[6]) >> 16) | (__float_as_uint(t[7]) & 0xFFFF0000u));
              } else {
                raw[b][0] = make_uint4(pack_half2(t[0], t[1]), pack_half2(t[2], t[3]), pack_half2(t[4], t[5]), pack_half2(t[6], t[7]));
              }
            }
          }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int c = XR == 1 ? c0 + b * n_threads : c0;
          const int m = XR == 1 ? 0 : 4 * r + b;
          if (c < chunks && m < p.M) {
            float v[8];
            if (p.x_dtype == NB_F32) {
              const uint32_t u[8] = {raw[b][0].x, raw[b][0].y, raw[b][0].z, raw[b][0].w, raw[b][1].x, raw[b][1].y, raw[b][1].z, raw[b][1].w};
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(u[j]);
            } else {
              const uint32_t u[4] = {raw[b][0].x, raw[b][0].y, raw[b][0].z, raw[b][0].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (p.x_dtype == NB_BF16) {
                  v[2 * j] = __uint_as_float(u[j] << 16);
                  v[2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
                } else {
                  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[j]));
                  v[2 * j] = f.x; v[2 * j + 1] = f.y;
                }
              }
            }
            const uint4 o4 = XR == 1 ? *reinterpret_cast<const uint4*>(dst_off + ((c & 15) << 3)) : o4_chunk;
            const uint32_t o[4] = {o4.x, o4.y, o4.z, o4.w};
            uint16_t* blk = reinterpret_cast<uint16_t*>(reinterpret_cast<__half*>(x_s) + (c >> 4) * (kXBlockBytes / 2) +
                                                        (m / XR) * XS * (x_tile_bytes / 2) + (m % XR) * 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t hi = f32x2_to_f16x2_sat(v[2 * j], v[2 * j + 1]);
              const uint32_t oa = o[j] & 0xFFFFu, ob = o[j] >> 16;
              blk[oa] = (uint16_t)(hi & 0xFFFFu);
              blk[ob] = (uint16_t)(hi >> 16);
              if (XS == 2) {  // low-order parts of the (clamped) values
                const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                const uint32_t lo = f32x2_to_f16x2_sat(fminf(fmaxf(v[2 * j], -65504.f), 65504.f) - rr.x,
                                                       fminf(fmaxf(v[2 * j + 1], -65504.f), 65504.f) - rr.y);
                blk[(x_tile_bytes / 2) + oa] = (uint16_t)(lo & 0xFFFFu);
                blk[(x_tile_bytes / 2) + ob] = (uint16_t)(lo >> 16);
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  NB_TRACE_MARK(3);

  // ---- units
#pragma unroll 1
  for (int u = warp; u < n_units; u += n_warps) {
    const int rtl = u / kg_n, kgl = u - rtl * kg_n;
    {  // bounded wait for this row tile's copies
      uint32_t spins = 0;
      while (!mbar_try_wait(&bars[rtl], 0)) {
        __nanosleep(40);  // back off: a spinning warp would take issue slots from the warps that unpack
        if (++spins > kSpinLimit) {
          if (p.status) atomicExch(p.status, (int)NB_ERR_TIMEOUT);
          break;
        }
      }
    }
    if (u == 0) NB_TRACE_MARK(4);
    const int kbl = 4 * kgl + t;                 // this lane's k-block inside the CTA's range
    const bool vk = kbl < kb_n;
    const int ra = rtl * 16 + g, rb = ra + 8;
    // 2 and 3 bits: the block's words are read up front; 4 bits: a group's four words are its selector
    // words, read from shared memory group by group (16 + 16 words would not fit the register budget)
    uint32_t wa[BITS == 4 ? 1 : kWords], wb[BITS == 4 ? 1 : kWords], TA[BITS == 4 ? 8 : 4], TB[BITS == 4 ? 8 : 4];
    const uint8_t* blk_a = w_s + ra * p.w_stride + (vk ? kbl : 0) * kBlkBytes;
    const uint8_t* blk_b = w_s + rb * p.w_stride + (vk ? kbl : 0) * kBlkBytes;
    if (BITS != 4) {
      read_block<BITS>(blk_a, reinterpret_cast<uint32_t (&)[kWords]>(wa));
      read_block<BITS>(blk_b, reinterpret_cast<uint32_t (&)[kWords]>(wb));
    }
    make_table<BITS>(c_s + ra * p.c_stride + (vk ? kbl : 0) * cb_blk, p.cb_dtype, vk, TA);
    make_table<BITS>(c_s + rb * p.c_stride + (vk ? kbl : 0) * cb_blk, p.cb_dtype, vk, TB);

    float c[2][NT][4];  // two accumulator sets: even and odd steps
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { c[j][nt][0] = c[j][nt][1] = c[j][nt][2] = c[j][nt][3] = 0.f; }
    const uint8_t* xrow = x_s + kbl * kXBlockBytes + (g % XR) * 8;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t UA[4], UB[4];
      if (BITS == 4) {
        const uint4 va = *reinterpret_cast<const uint4*>(blk_a + 16 * q), vb = *reinterpret_cast<const uint4*>(blk_b + 16 * q);
        UA[0] = va.x; UA[1] = va.y; UA[2] = va.z; UA[3] = va.w;
        UB[0] = vb.x; UB[1] = vb.y; UB[2] = vb.z; UB[3] = vb.w;
      } else {
        group_selectors<BITS>(wa, q, UA);
        group_selectors<BITS>(wb, q, UB);
      }
#pragma unroll
      for (int uu = 0; uu < 4; ++uu) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int s = 8 * q + 2 * uu + h;
          const uint32_t sa = h ? (UA[uu] >> 16) : UA[uu];
          const uint32_t sb = h ? (UB[uu] >> 16) : UB[uu];
          uint32_t a0, a1, a2, a3;
          lookup4<BITS>(sa, TA, a0, a2);
          lookup4<BITS>(sb, TB, a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int xs = 0; xs < XS; ++xs) {
              const uint2 xb = *reinterpret_cast<const uint2*>(xrow + (nt * XS + xs) * x_tile_bytes + s * (XR * 8));
              mma_16816(c[h][nt], a0, a1, a2, a3, xb.x, xb.y);
            }
          }
        }
      }
    }
    // the unit's partial tile goes to its own slot (plain stores, no atomics): the sums over a row
    // tile's units below have a fixed order, so results do not depend on which warp finished first
    float* ut = unit_acc + (size_t)u * kUnitTile;
    if (XR == 1) {
      if (t == 0) {
        ut[g] = c[0][0][0] + c[1][0][0];
        ut[g + 8] = c[0][0][2] + c[1][0][2];
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        *reinterpret_cast<float2*>(ut + g * kUnitCols + nt * 8 + 2 * t) = make_float2(c[0][nt][0] + c[1][nt][0], c[0][nt][1] + c[1][nt][1]);
        *reinterpret_cast<float2*>(ut + (g + 8) * kUnitCols + nt * 8 + 2 * t) = make_float2(c[0][nt][2] + c[1][nt][2], c[0][nt][3] + c[1][nt][3]);
      }
    }
  }
  __syncthreads();
  NB_TRACE_MARK(5);
  // sum over the k-groups of row r (local), column m, in k order
  auto row_sum = [&](int r, int m) {
    const float* src = unit_acc + (size_t)(r >> 4) * kg_n * kUnitTile + (r & 15) * kUnitCols + (XR == 1 ? 0 : m);
    float v = 0.f;
    for (int kg = 0; kg < kg_n; kg += 8) {  // eight loads in flight, then the adds in order
      float part[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) part[j] = (kg + j < kg_n) ? src[(size_t)(kg + j) * kUnitTile] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v += part[j];
    }
    return v;
  };

  const int rows_here = rt_n * 16;
  const int row0 = rt0 * 16;
  // Output: y, or (push) slot `rank` of the next set of every rank's exchange buffer.
  uint32_t push_seq = 0;
  size_t push_off = 0;
  void* const out_y = p.y;
  const int out_n = p.N, out_dtype = p.y_dtype;  // the lambdas below must not refer to the view struct itself
  auto emit = [&](int m, int row, float v) {
    if (PRO == 1) v *= s_scale[m];
    if (PUSH) {
      const size_t off = push_off + (size_t)m * out_n + row;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < ex.xchg_world) reinterpret_cast<float*>(s_peer[PUSH ? q : 0])[off] = v;
    } else {
      store_y(out_y, out_dtype, (size_t)m * out_n + row, v);
    }
  };
  // After a CTA has written its rows: the last writer of the grid (one per row group) raises this
  // rank's flag on every rank.  Each writer CTA fences its stores at device scope (one thread, after a
  // CTA barrier) before it takes its ticket; the last one fences at system scope before the flags.
  auto finish_push = [&]() {
    __syncthreads();          // the CTA's stores happen before thread 0's fence, which is cumulative
    if (tid == 0) {
      __threadfence();        // device scope: orders this CTA's stores before its ticket
      uint8_t* self = ex.xchg_self;
      int* ticket = reinterpret_cast<int*>(xchg_seq(self, ex.xchg_world, ex.xchg_max_count) + 1);
      if (atomicAdd(ticket, 1) == (int)gridDim.x - 1) {
        // the one system-scope fence of the launch: every writer's stores are ordered before its ticket,
        // all tickets before this point, this point before the flags (a system fence in each of some
        // hundred CTAs was measured to cost about 6 us per launch)
        __threadfence_system();
        const int set = push_seq & 1;
        for (int q = 0; q < ex.xchg_world; ++q)
          st_release_sys_u32(xchg_flags(reinterpret_cast<const uint8_t*>(s_peer[PUSH ? q : 0]), ex.xchg_world, ex.xchg_max_count) +
                                 set * ex.xchg_world + ex.xchg_rank, push_seq);
        *xchg_seq(self, ex.xchg_world, ex.xchg_max_count) = push_seq;
        *ticket = 0;
      }
    }
  };
  if (gridDim.y == 1) {
    if (PUSH) {
      push_seq = s_push_seq;
      push_off = ((size_t)(push_seq & 1) * ex.xchg_world + ex.xchg_rank) * ex.xchg_max_count;
    }
    for (int e = tid; e < p.M * rows_here; e += n_threads) {
      const int m = e / rows_here, r = e - m * rows_here;
      if (row0 + r < p.N) emit(m, row0 + r, row_sum(r, m));
    }
    if (PUSH) finish_push();
    NB_TRACE_MARK(6);
    return;
  }
  // ---- split-K fix-up: this CTA's partial tile (rows x NT*8 columns) goes to scratch; the CTA that
  // takes the last ticket of its row group adds all partial tiles in fixed order and writes y.
  {
    float* mine = p.scratch + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * acc_n;
    for (int i = tid; i < acc_n; i += n_threads) {
      const int r = i / (NT * 8), m = i - r * (NT * 8);
      __stcg(mine + i, (r < rows_here && m < p.M) ? row_sum(r, m) : 0.f);
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
    const float4* base = reinterpret_cast<const float4*>(p.scratch + (size_t)blockIdx.x * gridDim.y * acc_n);
    const int parts = gridDim.y, stride4 = acc_n / 4;
    for (int i = tid; i < acc_n / 4; i += n_threads) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int part0 = 0; part0 < parts; part0 += 8) {
        float4 t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          t[j] = (part0 + j < parts) ? __ldcg(base + (size_t)(part0 + j) * stride4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
      }
      reinterpret_cast<float4*>(acc)[i] = v;
    }
    if (tid == 0) p.counters[blockIdx.x] = 0;
    __syncthreads();
  }
  if (PUSH) {
    push_seq = s_push_seq;
    push_off = ((size_t)(push_seq & 1) * ex.xchg_world + ex.xchg_rank) * ex.xchg_max_count;
  }
  for (int e = tid; e < p.M * rows_here; e += n_threads) {
    const int m = e / rows_here, r = e - m * rows_here;
    if (row0 + r < p.N) emit(m, row0 + r, acc[r * (NT * 8) + m]);
  }
  if (PUSH) finish_push();
  NB_TRACE_MARK(6);
}

// Shared-memory row stride: at least `bytes`, 16-byte aligned, and equal to 64 mod 128 so that
// the 16-byte reads of rows g and g+1 land in different banks.
static int skew_stride(int bytes) {
  int s = (bytes + 15) / 16 * 16;
  while (s % 128 != 64) s += 16;
  return s;
}

// Picks rows-per-CTA and the k split so that the grid is close to one full wave of CTAs with
// about one unit per warp.  cost = waves * (latency + ceil(units/warps)) + fix-up penalty.
static GemvPlan make_plan(int M, int N, int K, int bits, int cb_dtype, int x_terms, int sms) {
  const int nt = M > 8 ? 2 : 1;
  const int row_tiles = (N + 15) / 16, bpr = K / kBlock, kgroups = (bpr + 3) / 4;
  const int blk_bytes = 16 * bits, cb_blk = (cb_dtype == NB_F16 ? 2 : 4) << bits;
  GemvPlan best{};
  double best_cost = 1e30;
  for (int parts_req = 1; parts_req <= std::min(kgroups, 32); ++parts_req) {
    const int kgp = (kgroups + parts_req - 1) / parts_req;
    const int parts = (kgroups + kgp - 1) / kgp;
    if (parts != parts_req) continue;
    const int kb_cnt = std::min(kgp * 4, bpr);
    // whole rows (one partition, 16-byte granular codebook rows): natural strides, bulk copies
    const bool whole = parts == 1 && (bpr * cb_blk) % 16 == 0;
    const int ws = whole ? kb_cnt * blk_bytes : skew_stride(kb_cnt * blk_bytes);
    const int cs = whole ? kb_cnt * cb_blk : skew_stride(kb_cnt * cb_blk);
    for (int tr = 1; tr <= std::min(row_tiles, kMaxTr); ++tr) {
      const size_t smem = (size_t)tr * 16 * (ws + cs) + (size_t)nt * x_terms * kgp * 4 * x_block_bytes(M == 1 ? 1 : 8) +
                          (size_t)tr * 16 * nt * 8 * 4 + (size_t)tr * kgp * 16 * (M == 1 ? 1 : nt * 8) * 4 + 2 * kBlock + 144;
      if (smem > (size_t)kMaxSmem) break;
      const int gx = (row_tiles + tr - 1) / tr;
      if (parts > 1 && gx >= kCounterInts - 1) continue;  // one ticket counter per row group
      const long ctas = (long)gx * parts;
      const int upc = tr * kgp;                            // units per CTA
      const int warps = std::min(kMaxWarps, std::max(4, upc));
      // CTAs of one launch that fit an SM together (64 registers per thread, 220 KB shared memory)
      const int resident = std::max(1, std::min(std::min(65536 / (warps * 32 * 64), (int)(220 * 1024 / smem)), 2048 / (warps * 32)));
      const long waves = (ctas + (long)sms * resident - 1) / ((long)sms * resident);
      const int rounds = (upc + warps - 1) / warps;
      // Measured on B200: about ten units per CTA with several CTAs per SM beats one large CTA per SM
      // (phases of co-resident CTAs overlap), hence the mild pull towards upc = 10.
      double cost = waves * (1.5 + rounds) + 0.05 * std::abs(upc - 10) + (parts > 1 ? 0.4 + 0.02 * parts : 0.0) +
                    (ctas < sms ? 3.0 * (double)(sms - ctas) / sms : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = GemvPlan{tr, parts, kgp, gx, warps, smem, ws, cs};
      }
    }
  }
  return best;
}

// The search above costs a few microseconds; launches repeat a handful of shapes, so the last
// plans are kept in a small table.
static GemvPlan cached_plan(int M, int N, int K, int bits, int cb_dtype, int x_terms, int sms) {
  struct Entry { int key[7]; GemvPlan plan; bool used; };
  static Entry table[32];
  static std::mutex mu;
  const int key[7] = {M, N, K, bits, cb_dtype, x_terms, sms};
  const unsigned h = ((unsigned)M * 2654435761u ^ (unsigned)N * 40503u ^ (unsigned)K * 9973u ^ (unsigned)(bits * 8 + cb_dtype * 2 + x_terms)) % 32u;
  {
    std::lock_guard<std::mutex> lock(mu);
    Entry& e = table[h];
    if (e.used && std::equal(key, key + 7, e.key)) return e.plan;
  }
  const GemvPlan pl = make_plan(M, N, K, bits, cb_dtype, x_terms, sms);
  std::lock_guard<std::mutex> lock(mu);
  Entry& e = table[h];
  std::copy(key, key + 7, e.key);
  e.plan = pl;
  e.used = true;
  return pl;
}

// workspace layout: a fixed 16 KB head of ticket counters (int 0..4094) and the status word (int
// 4095), then the fp32 partial tiles.  The head is at the same place for every shape, so a
// workspace shared by launches of different shapes never has partial sums where a later launch
// expects zeroed counters.
static size_t counter_bytes(const GemvPlan&) { return (size_t)kCounterInts * sizeof(int); }

static size_t plan_workspace(const GemvPlan& pl, int M) {
  const size_t scratch = pl.parts > 1 ? (size_t)pl.grid_x * pl.parts * pl.tr * 16 * (M > 8 ? 16 : 8) * sizeof(float) : 0;
  return counter_bytes(pl) + scratch;
}

// `pdl`: launch with programmatic stream serialization (the grid may start, and request its weights,
// while the previous kernel of the stream still runs).  Without it the launch is fully stream
// ordered and the griddepcontrol instructions in the kernel do nothing.
static thread_local bool g_launch_pdl = true;

template <int BITS, int NT, int XR, int XS, int PRO = 0, int PUSH = 0>
static int launch(const GemvParams& prm, const GemvExtra& extra, const GemvPlan& pl, cudaStream_t st) {
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<BITS, NT, XR, XS, PRO, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return record_cuda_error(e);
    attr_done[dev & 63] = true;
  }
  // Programmatic dependent launch: this grid may start (and request its weights) while the
  // previous kernel of the stream is still running; it waits for that kernel before it reads x.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid_x, pl.parts);
  cfg.blockDim = dim3(pl.warps * 32);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_launch_pdl ? 1 : 0;
  if constexpr (PRO != 0 || PUSH != 0) {
    return record_cuda_error(cudaLaunchKernelEx(&cfg, gemv_kernel<BITS, NT, XR, XS, PRO, PUSH>, prm, extra));
  } else {
    return record_cuda_error(cudaLaunchKernelEx(&cfg, gemv_kernel<BITS, NT, XR, XS, PRO, PUSH>, prm, GemvNoExtra{}));
  }
}

}  // namespace nb

using namespace nb;

static int gemv_check_shape(int M, int N, int K, int bits, int block_size) {
  if (M < 1 || N < 1 || K < 1) return NB_ERR_ARG;
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_SHAPE;
  if (block_size != kBlock) return NB_ERR_SHAPE;
  if (M > 16 || K % kBlock != 0) return NB_ERR_SHAPE;
  return NB_OK;
}

extern "C" size_t nb_gemv_workspace_bytes(int M, int N, int K, int bits, int block_size) {
  if (gemv_check_shape(M, N, K, bits, block_size) != NB_OK) return 0;
  // the plan depends on the codebook and activation types: report the largest need
  size_t need = 0;
  for (int cb = NB_F32; cb <= NB_F16; ++cb)
    for (int xt = 1; xt <= 2; ++xt) need = std::max(need, plan_workspace(make_plan(M, N, K, bits, cb, xt, sm_count()), M));
  return need;
}

extern "C" int nb_gemv_plan(int M, int N, int K, int bits, int block_size, int cb_dtype, int* out6) {
  if (!out6) return NB_ERR_ARG;
  if (int rc = gemv_check_shape(M, N, K, bits, block_size)) return rc;
  const GemvPlan pl = make_plan(M, N, K, bits, cb_dtype, 1, sm_count());
  out6[0] = pl.grid_x; out6[1] = pl.parts; out6[2] = pl.warps * 32; out6[3] = (int)pl.smem; out6[4] = pl.tr; out6[5] = pl.kg_per_part;
  return NB_OK;
}

namespace nb {
struct Prologue {
  int kind = 0;                  // 0 none, 1 residual add + RMSNorm, 2 SwiGLU
  const float* delta = nullptr;
  const float* weight = nullptr;
  float* x_out = nullptr;
  float eps = 0.f;
  // tensor-parallel exchange
  void* exchange = nullptr;
  int world = 0, rank = 0, max_count = 0, gather = 0, push = 0;
  uint32_t spin_limit = 0;
};
constexpr uint32_t kXchgSpinLimit = 1u << 23;  // several seconds: a probe is an L2 round trip plus the 100 ns back-off

// Sum over the ranks of the vectors pushed last -> out (count floats); grid of a few CTAs, each waits itself.
__global__ void __launch_bounds__(256) exchange_gather_kernel(float* __restrict__ out, int count, const uint8_t* self, int world,
                                                              int max_count, uint32_t spin_limit, int* status) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const int tid = threadIdx.x;
  const uint32_t seq = __ldcg(xchg_seq(self, world, max_count));
  const int set = seq & 1;
  if (tid < world) {
    const uint32_t* flag = xchg_flags(self, world, max_count) + set * world + tid;
    uint32_t spins = (status && *reinterpret_cast<volatile int*>(status) == (int)NB_ERR_TIMEOUT) ? spin_limit : 0;
    while (ld_acquire_sys_u32(flag) != seq) {
      __nanosleep(100);
      if (++spins > spin_limit) {
        if (status) atomicExch(status, (int)NB_ERR_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  const float* slots = reinterpret_cast<const float*>(self) + (size_t)set * world * max_count;
  for (int i = blockIdx.x * blockDim.x + tid; i < count / 4; i += gridDim.x * blockDim.x) {
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < world; ++q) {
      const float4 e = __ldcv(reinterpret_cast<const float4*>(slots + (size_t)q * max_count) + i);
      d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
    }
    reinterpret_cast<float4*>(out)[i] = d;
  }
}
}  // namespace nb

static int gemv_impl(const Prologue& pro, const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook,
                     int cb_dtype, int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
                     size_t workspace_bytes, void* stream) {
  if (!x || !packed || !codebook) return NB_ERR_ARG;
  if (x_dtype < NB_F32 || x_dtype > NB_BF16 || y_dtype < NB_F32 || y_dtype > NB_BF16) return NB_ERR_ARG;
  if (cb_dtype != NB_F16 && cb_dtype != NB_F32) return NB_ERR_ARG;
  if (int rc = gemv_check_shape(M, N, K, bits, block_size)) return rc;
  if ((uintptr_t)packed % 16 || (uintptr_t)codebook % 16) return NB_ERR_ALIGN;
  if (pro.kind != 0) {
    if (pro.kind != 1 && pro.kind != 2) return NB_ERR_ARG;
    if (x_dtype != NB_F32) return NB_ERR_ARG;
    if (M > 8) return NB_ERR_SHAPE;
    if (pro.kind == 1 && (!pro.weight || pro.x_out == x)) return NB_ERR_ARG;
    if ((uintptr_t)x % 16 || (uintptr_t)pro.delta % 16 || (uintptr_t)pro.weight % 16 || (uintptr_t)pro.x_out % 16) return NB_ERR_ALIGN;
  }
  if (pro.gather || pro.push) {
    if (!pro.exchange || pro.world < 1 || pro.world > 8 || pro.rank < 0 || pro.rank >= pro.world) return NB_ERR_ARG;
    if (pro.max_count < 4 || (pro.max_count & 3)) return NB_ERR_ARG;
    if (pro.push && pro.kind == 1) return NB_ERR_ARG;  // a row-sharded projection follows attention or SwiGLU, never a norm
    if (pro.gather && (pro.kind != 1 || (size_t)M * K > (size_t)pro.max_count)) return NB_ERR_SHAPE;
    if (pro.push && (size_t)M * N > (size_t)pro.max_count) return NB_ERR_SHAPE;
    if ((uintptr_t)pro.exchange % 16) return NB_ERR_ALIGN;
  }
  if (!pro.push && !y) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  const int x_terms = x_dtype == NB_F32 ? 2 : 1;
  const GemvPlan pl = cached_plan(M, N, K, bits, cb_dtype, x_terms, sm_count());
  if (pl.grid_x == 0) return NB_ERR_SHAPE;
  const size_t need = plan_workspace(pl, M);
  const bool have_ws = workspace && workspace_bytes >= need;
  if (pl.parts > 1 && !have_ws) return NB_ERR_WORKSPACE;
  if (have_ws && (uintptr_t)workspace % 16) return NB_ERR_ALIGN;

  GemvParams prm{};
  prm.x = x; prm.packed = packed; prm.codebook = codebook; prm.y = y;
  if (have_ws) prm.counters = reinterpret_cast<int*>(workspace);
  if (K / kBlock > 65535 || pl.kg_per_part > 65535) return NB_ERR_SHAPE;
  prm.M = (uint8_t)M; prm.N = N; prm.bpr = (uint16_t)(K / kBlock);
  prm.tr = (uint8_t)pl.tr; prm.kg_per_part = (uint16_t)pl.kg_per_part;
  prm.dtypes = (uint8_t)(x_dtype | (y_dtype << 2) | (cb_dtype << 4));
  prm.w_stride = pl.w_stride; prm.c_stride = pl.c_stride;
  const int cb_bulk = (((K / kBlock) * ((cb_dtype == NB_F16 ? 2 : 4) << bits)) % 16 == 0) ? 1 : 0;
  const int tile_bulk = (pl.parts == 1 && cb_bulk) ? 1 : 0;
  prm.flags = (uint8_t)((((uintptr_t)x % 16 == 0) ? 1 : 0) | (cb_bulk << 1) | (tile_bulk << 2));
  cudaStream_t st = (cudaStream_t)stream;
  GemvExtra extra{};
  extra.pro_delta = pro.delta; extra.pro_weight = pro.weight; extra.pro_x_out = pro.x_out; extra.pro_eps = pro.eps;
  if (pro.gather || pro.push) {
    extra.xchg_self = reinterpret_cast<uint8_t*>(pro.exchange);
    extra.xchg_world = pro.world; extra.xchg_rank = pro.rank; extra.xchg_max_count = pro.max_count;
    extra.gather = pro.gather;
    extra.xchg_spin = pro.spin_limit ? pro.spin_limit : kXchgSpinLimit;
    if (!prm.counters) return NB_ERR_WORKSPACE;  // the bounded wait reports through the workspace's status word
  }
  if (pro.kind != 0 || pro.push) {  // fp32 activations, M <= 8
    if (M > 8 || x_dtype != NB_F32) return NB_ERR_SHAPE;
#define NB_GEMV_PRO(B, P, E) (M > 1 ? launch<B, 1, 8, 2, P, E>(prm, extra, pl, st) : launch<B, 1, 1, 2, P, E>(prm, extra, pl, st))
#define NB_GEMV_PRO_B(P, E) (bits == 3 ? NB_GEMV_PRO(3, P, E) : bits == 2 ? NB_GEMV_PRO(2, P, E) : NB_GEMV_PRO(4, P, E))
    if (pro.push) return pro.kind == 2 ? NB_GEMV_PRO_B(2, 1) : pro.kind == 0 ? NB_GEMV_PRO_B(0, 1) : NB_ERR_ARG;
    return pro.kind == 1 ? NB_GEMV_PRO_B(1, 0) : NB_GEMV_PRO_B(2, 0);
#undef NB_GEMV_PRO_B
#undef NB_GEMV_PRO
  }
#define NB_GEMV_DISPATCH(B, XSV)                                                               \
  (M > 8 ? launch<B, 2, 8, XSV>(prm, extra, pl, st) : M > 1 ? launch<B, 1, 8, XSV>(prm, extra, pl, st) : launch<B, 1, 1, XSV>(prm, extra, pl, st))
  if (bits == 3) return x_terms == 2 ? NB_GEMV_DISPATCH(3, 2) : NB_GEMV_DISPATCH(3, 1);
  if (bits == 4) return x_terms == 2 ? NB_GEMV_DISPATCH(4, 2) : NB_GEMV_DISPATCH(4, 1);
  return x_terms == 2 ? NB_GEMV_DISPATCH(2, 2) : NB_GEMV_DISPATCH(2, 1);
#undef NB_GEMV_DISPATCH
}

extern "C" int nb_gemv(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                       int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
                       size_t workspace_bytes, void* stream) {
  return gemv_impl(Prologue{}, x, x_dtype, M, packed, codebook, cb_dtype, bits, block_size, N, K, y, y_dtype, workspace,
                   workspace_bytes, stream);
}

extern "C" int nb_gemv_ordered(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                               int bits, int block_size, int N, int K, void* y, int y_dtype, void* workspace,
                               size_t workspace_bytes, void* stream) {
  g_launch_pdl = false;
  const int rc = gemv_impl(Prologue{}, x, x_dtype, M, packed, codebook, cb_dtype, bits, block_size, N, K, y, y_dtype, workspace,
                           workspace_bytes, stream);
  g_launch_pdl = true;
  return rc;
}

extern "C" int nb_gemv_fused(int prologue, const float* x, const float* delta, const float* norm_weight, float eps, float* x_out,
                             int M, const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size, int N,
                             int K, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  Prologue pro;
  pro.kind = prologue;
  if (prologue == NB_PRO_ADD_RMSNORM) { pro.delta = delta; pro.weight = norm_weight; pro.x_out = x_out; pro.eps = eps; }
  return gemv_impl(pro, x, NB_F32, M, packed, codebook, cb_dtype, bits, block_size, N, K, y, y_dtype, workspace, workspace_bytes,
                   stream);
}

extern "C" size_t nb_exchange_buffer_bytes(int world, int max_count) {
  if (world < 1 || world > 8 || max_count < 4 || (max_count & 3)) return 0;
  return xchg_bytes(world, max_count);
}

extern "C" int nb_exchange_init(void* exchange, const uint64_t* peer_bufs, int world, int rank, int max_count) {
  if (!exchange || !peer_bufs || world < 1 || world > 8 || rank < 0 || rank >= world) return NB_ERR_ARG;
  if (max_count < 4 || (max_count & 3)) return NB_ERR_ARG;
  unsigned long long table[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int q = 0; q < world; ++q) {
    if (!peer_bufs[q] || peer_bufs[q] % 16) return NB_ERR_ALIGN;
    table[q] = peer_bufs[q];
  }
  if (peer_bufs[rank] != (uint64_t)(uintptr_t)exchange) return NB_ERR_ARG;
  return record_cuda_error(cudaMemcpy(xchg_table(reinterpret_cast<const uint8_t*>(exchange), world, max_count), table, sizeof(table),
                                      cudaMemcpyHostToDevice));
}

extern "C" int nb_gemv_tp(int prologue, const float* x, const float* delta, const float* norm_weight, float eps, float* x_out, int M,
                          const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size, int N, int K, void* y,
                          int y_dtype, void* workspace, size_t workspace_bytes, void* exchange, int world, int rank, int max_count,
                          int gather, int push, uint32_t spin_limit, void* stream) {
  Prologue pro;
  pro.kind = prologue;
  if (prologue == NB_PRO_ADD_RMSNORM) { pro.delta = gather ? nullptr : delta; pro.weight = norm_weight; pro.x_out = x_out; pro.eps = eps; }
  pro.exchange = exchange; pro.world = world; pro.rank = rank; pro.max_count = max_count;
  pro.gather = gather ? 1 : 0; pro.push = push ? 1 : 0; pro.spin_limit = spin_limit;
  return gemv_impl(pro, x, NB_F32, M, packed, codebook, cb_dtype, bits, block_size, N, K, y, push ? NB_F32 : y_dtype, workspace,
                   workspace_bytes, stream);
}

extern "C" int nb_exchange_gather(float* out, int count, const void* exchange, int world, int rank, int max_count,
                                  uint32_t spin_limit, int* status, void* stream) {
  if (!out || !exchange || world < 1 || world > 8 || rank < 0 || rank >= world) return NB_ERR_ARG;
  if (count < 4 || (count & 3) || count > max_count || (max_count & 3)) return NB_ERR_SHAPE;
  if ((uintptr_t)out % 16 || (uintptr_t)exchange % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(std::max(1, std::min(8, count / 4 / 256)));
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return record_cuda_error(cudaLaunchKernelEx(&cfg, exchange_gather_kernel, out, count, reinterpret_cast<const uint8_t*>(exchange),
                                              world, max_count, spin_limit ? spin_limit : kXchgSpinLimit, status));
}

// ------------------------------------------------------------------------------------------------
// nb_gemv_static — the same fused GEMV for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand nb_gemv a workspace: code running inside a CUDA-graph
// capture or inside another framework's allocator-owned region, plugins whose interface gives
// them input and output buffers and nothing else, and processes that run with a frozen memory
// budget.  For them the split-K scratch lives in a fixed array in this module's device image
// (4 MiB, resident on every GPU that loads the library until the process exits).  In host code
// the array's name is only a handle, not a device pointer, so its address is looked up once per
// device with cudaGetSymbolAddress while that device is current.
// ------------------------------------------------------------------------------------------------
namespace nb {
constexpr size_t kStaticWsBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];
static std::mutex g_static_mu;
static void* g_static_ptr[64];
static bool g_static_ready[64];
}  // namespace nb

extern "C" int nb_gemv_static(const void* x, int x_dtype, int M, const uint8_t* packed, const void* codebook, int cb_dtype,
                              int bits, int block_size, int N, int K, void* y, int y_dtype, void* stream) {
  if (!x || !packed || !codebook || !y) return NB_ERR_ARG;
  if (int rc = gemv_check_shape(M, N, K, bits, block_size)) return rc;
  // the scratch need of a shape is the largest over codebook and activation types (as
  // nb_gemv_workspace_bytes reports it), from the plan cache
  size_t need = 0;
  for (int cb = NB_F32; cb <= NB_F16; ++cb)
    for (int xt = 1; xt <= 2; ++xt) need = std::max(need, plan_workspace(cached_plan(M, N, K, bits, cb, xt, sm_count()), M));
  if (need > kStaticWsBytes) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "nb_gemv_static: M=%d N=%d K=%d needs %zu bytes of scratch, the built-in array holds %zu",
                  M, N, K, need, (size_t)kStaticWsBytes);
    set_last_error(msg);
    return NB_ERR_WORKSPACE;
  }
  int dev = -1;
  if (cudaError_t e = cudaGetDevice(&dev)) return record_cuda_error(e);
  if (dev < 0 || dev >= 64) return NB_ERR_ARG;
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ready[dev]) {  // set-up, once per device, with that device current
      void* ptr = nullptr;
      if (cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_ws)) return record_cuda_error(e);
      g_static_ptr[dev] = ptr;
      g_static_ready[dev] = true;
    }
    ws = g_static_ptr[dev];
  }
  // The array keeps whatever the previous call left.  Only the ticket counters have to start at
  // zero; partial sums are always written before they are read, and the status word (the last int of
  // the head) is left alone so that a timeout stays visible to nb_gemv_static_status.
  if (cudaError_t e = cudaMemsetAsync(ws, 0, (size_t)(kCounterInts - 1) * sizeof(int), (cudaStream_t)stream)) return record_cuda_error(e);
  return nb_gemv(x, x_dtype, M, packed, codebook, cb_dtype, bits, block_size, N, K, y, y_dtype, ws, kStaticWsBytes, stream);
}

extern "C" int nb_gemv_static_status(int* host_out, int clear) {
  if (!host_out) return NB_ERR_ARG;
  int dev = -1;
  if (cudaError_t e = cudaGetDevice(&dev)) return record_cuda_error(e);
  if (dev < 0 || dev >= 64) return NB_ERR_ARG;
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ready[dev]) { *host_out = 0; return NB_OK; }  // never used on this device
    ws = g_static_ptr[dev];
  }
  int* word = reinterpret_cast<int*>(ws) + (kCounterInts - 1);
  if (cudaError_t e = cudaMemcpy(host_out, word, sizeof(int), cudaMemcpyDeviceToHost)) return record_cuda_error(e);
  if (clear && *host_out != 0)
    if (cudaError_t e = cudaMemset(word, 0, sizeof(int))) return record_cuda_error(e);
  return NB_OK;
}

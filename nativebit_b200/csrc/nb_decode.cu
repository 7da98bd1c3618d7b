// Small fused kernels of the decode step around the packed GEMVs (one new token per sequence):
// residual add + RMSNorm, RoPE + KV-cache write, single-query attention over the valid prefix of
// the cache, and SiLU(gate) * up.  All activations are fp32, as in the reference's cached path
// (inference/generate_torch.py:29-38 RMSNorm, :41-60 RoPE on interleaved pairs, :86-97 cache write
// and masked attention, :116-117 SwiGLU).  The position is read from device memory so that the
// step can be replayed from a CUDA graph.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cooperative_groups.h>

#include <algorithm>
#include <cfloat>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

namespace cg = cooperative_groups;

// Every kernel of the decode chain is launched with programmatic stream serialization: it may be
// scheduled while its predecessor still runs and waits for the predecessor's results before it
// touches memory.  It releases its own successor only AFTER that wait: a successor may then read,
// ahead of its own wait, anything written two or more launches back (the attention kernel does).
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
}

template <typename... KArgs, typename... Args>
static int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return record_cuda_error(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// x[b] += delta[b] (if delta); out[b] = x[b] / sqrt(mean(x[b]^2) + eps) * w.  One CTA per row; the
// row lives in registers (up to 16 elements per thread), so global memory is read exactly once.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                          const float* __restrict__ w, float eps, float* __restrict__ out, int C) {
  __shared__ float red[8];
  constexpr int kPer = 16;
  pdl_enter();
  float* xr = x + (size_t)blockIdx.x * C;
  const float* dr = delta ? delta + (size_t)blockIdx.x * C : nullptr;
  float v[kPer], wv[kPer];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int i = threadIdx.x + k * 256;
    v[k] = 0.f; wv[k] = 0.f;
    if (i < C) {
      v[k] = xr[i];
      wv[k] = w[i];
      if (dr) v[k] += dr[i];
    }
  }
#pragma unroll
  for (int k = 0; k < kPer; ++k) ss += v[k] * v[k];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot / (float)C + eps);
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < C) {
      if (dr) xr[i] = v[k];
      out[(size_t)blockIdx.x * C + i] = v[k] * inv * wv[k];
    }
  }
}

// qkv (B, 3*H*hd) = [q | k | v]; rotates q and k pairs (2i, 2i+1) by the position's angle, writes
// k and v into the caches (B, H, ctx, hd) at `pos`, q into q_out (B, H, hd).  grid (H, B).
__global__ void rope_kv_kernel(const float* __restrict__ qkv, const float* __restrict__ cos2, const float* __restrict__ sin2,
                               const long long* __restrict__ pos_ptr, float* __restrict__ k_cache, float* __restrict__ v_cache,
                               float* __restrict__ q_out, int H, int hd, int ctx) {
  const int h = blockIdx.x, b = blockIdx.y;
  pdl_enter();                                             // releases after the wait: the attention kernel behind reads the cache early
  const long long pos = *pos_ptr;
  if (pos < 0 || pos >= ctx) return;
  const float* base = qkv + (size_t)b * 3 * H * hd;
  const float* q = base + h * hd;
  const float* k = base + H * hd + h * hd;
  const float* v = base + 2 * H * hd + h * hd;
  const size_t crow = (((size_t)b * H + h) * ctx + pos) * hd;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    const float c = cos2[pos * hd + i], s = sin2[pos * hd + i];
    const int j = i ^ 1;                       // partner of the pair
    const float sign = (i & 1) ? 1.f : -1.f;   // rot = (-x2, x1)
    q_out[((size_t)b * H + h) * hd + i] = q[i] * c + sign * q[j] * s;
    k_cache[crow + i] = k[i] * c + sign * k[j] * s;
    v_cache[crow + i] = v[i];
  }
}

// Single-query attention for one (head, batch): scores over keys 0..pos, softmax, weighted sum of
// values; out[b, out_offset + h*hd + d].  grid (H, B, S) in clusters of S CTAs along z: the CTAs of
// a cluster split the keys of one head into S contiguous ranges (the whole GPU works on the 32
// heads of a batch-1 step instead of 32 SMs), each forms the softmax numerator and denominator of
// its range, and rank 0 merges them through distributed shared memory.  Inside a CTA a warp takes
// 8 keys per iteration: for the scores four lanes share a key (16-byte loads, two shuffles), for
// the values a lane owns four head dimensions of all 8 keys.  The values of the first iteration
// are requested before the scores are computed, so a context of up to 64*S keys costs one memory
// round trip.  head_dim a multiple of 4, <= 128.  Dynamic smem: see attn_smem_floats.
//
// When `qkv` is given (B, 3*H*hd = [q|k|v]) the kernel first does the work of rope_kv_kernel for its
// head: it rotates q and k by the position's angle, the CTA that owns key `pos` writes k and v into
// the caches, and all attend with the rotated q, so the step needs one launch instead of two.
constexpr int kAttnWarps = 8;
constexpr int kAttnKeysPerIter = kAttnWarps * 8;
static int attn_per_max(int ctx, int S) { return (((ctx + S - 1) / S) + 7) & ~7; }
static size_t attn_smem_floats(int ctx, int hd, int S) { return (size_t)attn_per_max(ctx, S) + (size_t)(2 + kAttnWarps) * hd + 4; }

__global__ void __launch_bounds__(kAttnWarps * 32) decode_attention_kernel(
    const float* __restrict__ q, float* k_cache, float* v_cache, const long long* __restrict__ pos_ptr, float* __restrict__ out,
    int H, int hd, int ctx, int out_stride, int out_offset, const float* __restrict__ qkv, const float* __restrict__ cos2,
    const float* __restrict__ sin2) {
  extern __shared__ __align__(16) float sm[];  // scores of this CTA's keys | q | per-warp outputs | exchange (o, max, sum)
  __shared__ float red[kAttnWarps];
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  asm volatile("griddepcontrol.launch_dependents;");
  // The position was written at the end of the step before, and the cache rows below it in earlier steps: neither
  // depends on the launch before this one, so this CTA's first keys and values are requested BEFORE the dependency
  // wait and arrive while the qkv matvec drains.  Only the row this step writes (position pos) is fetched after it.
  long long pos = *pos_ptr;
  if (pos < 0) return;  // the same for every CTA of the cluster
  if (pos >= ctx) pos = ctx - 1;
  const int n = (int)pos + 1, hd4 = hd >> 2;
  const int per = (((n + S - 1) / S) + 7) & ~7;
  const int k0 = rank * per;
  const int cnt = max(0, min(n, k0 + per) - k0);
  float* sc = sm;
  float* qs = sc + ((((ctx + S - 1) / S) + 7) & ~7);
  float* part = qs + hd;
  float* xch = part + kAttnWarps * hd;
  const size_t head = ((size_t)b * H + h);
  float* kb = k_cache + head * ctx * hd;
  float* vb = v_cache + head * ctx * hd;
  const int kq = lane >> 2, t = lane & 3;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 kfirst[8], vfirst[8];  // keys and values of iteration 0
  {
    const int jl = warp * 8 + kq;
    const bool ld = jl < cnt && k0 + jl != (int)pos;
    const float4* krow = reinterpret_cast<const float4*>(kb + (size_t)(k0 + jl) * hd);
#pragma unroll
    for (int i = 0; i < 8; ++i) kfirst[i] = (ld && t + 4 * i < hd4) ? krow[t + 4 * i] : zero4;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int ju = warp * 8 + u;
      vfirst[u] = (ju < cnt && k0 + ju != (int)pos && lane < hd4) ? *reinterpret_cast<const float4*>(vb + (size_t)(k0 + ju) * hd + 4 * lane)
                                                                   : zero4;
    }
  }
  float c_pre = 0.f, s_pre = 0.f;  // this thread's entry of the rotary tables (head_dim <= 128 < threads per CTA)
  if (qkv && tid < hd) { c_pre = cos2[pos * hd + tid]; s_pre = sin2[pos * hd + tid]; }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (qkv) {
    const float* base = qkv + (size_t)b * 3 * H * hd;
    const float* qh = base + h * hd;
    const float* kh = base + H * hd + h * hd;
    const float* vh = base + 2 * H * hd + h * hd;
    const bool owner = pos >= k0 && pos < k0 + cnt;
    for (int i = tid; i < hd; i += blockDim.x) {
      const float c = c_pre, s = s_pre;
      const int j = i ^ 1;
      const float sign = (i & 1) ? 1.f : -1.f;   // rot = (-x2, x1) on interleaved pairs
      qs[i] = (qh[i] * c + sign * qh[j] * s) * rsqrtf((float)hd);
      if (owner) {
        kb[(size_t)pos * hd + i] = kh[i] * c + sign * kh[j] * s;
        vb[(size_t)pos * hd + i] = vh[i];
      }
    }
  } else {
    for (int i = tid; i < hd; i += blockDim.x) qs[i] = q[head * hd + i] * rsqrtf((float)hd);
  }
  __syncthreads();  // also orders the cache row written above before the reads below (same CTA)

  const int iters = (cnt + kAttnKeysPerIter - 1) / kAttnKeysPerIter;
  {  // the row written in this step (by this CTA above, or by the launch before): now it can be read
    const int jl = warp * 8 + kq;
    if (jl < cnt && k0 + jl == (int)pos) {
      const float4* krow = reinterpret_cast<const float4*>(kb + (size_t)pos * hd);
#pragma unroll
      for (int i = 0; i < 8; ++i) kfirst[i] = (t + 4 * i < hd4) ? krow[t + 4 * i] : zero4;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int ju = warp * 8 + u;
      if (ju < cnt && k0 + ju == (int)pos && lane < hd4) vfirst[u] = *reinterpret_cast<const float4*>(vb + (size_t)pos * hd + 4 * lane);
    }
  }
  float mx = -FLT_MAX;
  for (int it = 0; it < iters; ++it) {
    const int jl = (it * kAttnWarps + warp) * 8 + kq;
    float s = 0.f;
    if (jl < cnt) {
      const float4* krow = reinterpret_cast<const float4*>(kb + (size_t)(k0 + jl) * hd);
      float4 kv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) kv[i] = it == 0 ? kfirst[i] : ((t + 4 * i < hd4) ? krow[t + 4 * i] : zero4);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (t + 4 * i < hd4) {
          const float4 qv = reinterpret_cast<const float4*>(qs)[t + 4 * i];
          s += qv.x * kv[i].x + qv.y * kv[i].y + qv.z * kv[i].z + qv.w * kv[i].w;
        }
      }
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (jl < cnt) {
      if (t == 0) sc[jl] = s;
      mx = fmaxf(mx, s);
    }
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < kAttnWarps; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < cnt; j += blockDim.x) {
    const float e = __expf(sc[j] - mx);
    sc[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kAttnWarps; ++i) tot += red[i];

  float4 acc = zero4;
  for (int it = 0; it < iters; ++it) {
    const int j0 = (it * kAttnWarps + warp) * 8;
    float4 vv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (it == 0) vv[u] = vfirst[u];
      else vv[u] = (j0 + u < cnt && lane < hd4) ? *reinterpret_cast<const float4*>(vb + (size_t)(k0 + j0 + u) * hd + 4 * lane) : zero4;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float pj = (j0 + u < cnt) ? sc[j0 + u] : 0.f;
      acc.x += pj * vv[u].x; acc.y += pj * vv[u].y; acc.z += pj * vv[u].z; acc.w += pj * vv[u].w;
    }
  }
  if (lane < hd4) reinterpret_cast<float4*>(part + warp * hd)[lane] = acc;
  __syncthreads();
  for (int d = tid; d < hd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int wi = 0; wi < kAttnWarps; ++wi) o += part[wi * hd + d];
    xch[d] = o;
  }
  if (tid == 0) { xch[hd] = mx; xch[hd + 1] = tot; }
  cluster.sync();
  if (rank == 0) {
    for (int d = tid; d < hd; d += blockDim.x) {
      float m_all = -FLT_MAX;
      for (int r = 0; r < S; ++r) m_all = fmaxf(m_all, cluster.map_shared_rank(xch, r)[hd]);
      float num = 0.f, den = 0.f;
      for (int r = 0; r < S; ++r) {  // a rank without keys has max -FLT_MAX: its weight is exp(-inf) = 0
        const float* rx = cluster.map_shared_rank(xch, r);
        const float w = __expf(rx[hd] - m_all);
        num += w * rx[d];
        den += w * rx[hd + 1];
      }
      out[(size_t)b * out_stride + out_offset + h * hd + d] = num / den;
    }
  }
  cluster.sync();  // the exchange buffers stay alive until rank 0 has read them
}

// Cluster size: enough CTAs for a few waves of the GPU, at most 8 per head.
static int attn_split(int B, int H) {
  const int want = 592 / std::max(1, B * H);
  return want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;
}

template <typename... Args>
static int launch_attention(int B, int H, int hd, int ctx, cudaStream_t st, Args... args) {
  const int S = attn_split(B, H);
  const size_t smem = attn_smem_floats(ctx, hd, S) * sizeof(float);
  if (smem > 48 * 1024) return NB_ERR_SHAPE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(H, B, S);
  cfg.blockDim = dim3(kAttnWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = S;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return record_cuda_error(cudaLaunchKernelEx(&cfg, decode_attention_kernel, args...));
}

// Causal attention of a prompt (or a chunk of one that continues a cache of pos0 keys) in ONE launch per layer:
// RoPE on q and k, cache write, softmax(q k^T / sqrt(hd)) v over keys 0 .. pos0 + t for query t
// (inference/generate_torch.py:41-60 RoPE, :86-97 cache write and masked attention).  grid (ceil(T / 16), H, B):
// a CTA owns 16 queries of one head; it walks the keys in chunks of 32, staging a chunk of K and V in shared
// memory — from the cache below pos0, from qkv (rotating k on the way) from pos0 on, so no CTA reads what
// another one writes in this launch — and keeps a running maximum, denominator and numerator per query.  The
// CTA whose queries sit at positions [q0, q0 + 16) is the one that writes those positions' k and v to the cache.
// Eight threads share a query: for the scores each takes every eighth key of the chunk, for the values four head
// dimensions out of every 32.  Everything is fp32.  head_dim a multiple of 4, <= 128.
constexpr int kPQ = 16, kPK = 32, kPThreads = 128;

__global__ void __launch_bounds__(kPThreads) prefill_attention_kernel(
    const float* __restrict__ qkv, const float* __restrict__ cos2, const float* __restrict__ sin2, float* __restrict__ k_cache,
    float* __restrict__ v_cache, float* __restrict__ out, int T, int H, int hd, int ctx, int pos0, int out_stride, int out_offset,
    float scale) {
  extern __shared__ __align__(16) float psm[];
  const int hdp = hd + 4;                       // row stride: 16-byte aligned, eight consecutive rows on different banks
  float* q_s = psm;                             // [kPQ][hdp]
  float* k_s = q_s + kPQ * hdp;                 // [kPK][hdp]
  float* v_s = k_s + kPK * hdp;                 // [kPK][hdp]
  float* p_s = v_s + kPK * hdp;                 // [kPQ][kPK + 1]
  const int tid = threadIdx.x, q0 = blockIdx.x * kPQ, h = blockIdx.y, b = blockIdx.z;
  const int row3 = 3 * H * hd, half = hd >> 1, quarter = hd >> 2;
  const size_t cbase = ((size_t)b * H + h) * (size_t)ctx * hd;

  // this tile's queries, rotated (rows past the prompt's end repeat its last query and are not written)
  for (int i = tid; i < kPQ * half; i += kPThreads) {
    const int r = i / half, d = (i - r * half) * 2;
    const int t = min(q0 + r, T - 1);
    const float2 x = *reinterpret_cast<const float2*>(qkv + (size_t)(b * T + t) * row3 + h * hd + d);
    const size_t ri = (size_t)(pos0 + t) * hd + d;
    const float c = cos2[ri], s = sin2[ri];
    q_s[r * hdp + d] = x.x * c - x.y * s;
    q_s[r * hdp + d + 1] = x.y * c + x.x * s;
  }

  const int qi = tid >> 3, sub = tid & 7;
  const int my_pos = pos0 + min(q0 + qi, T - 1);
  const int kmax = pos0 + min(q0 + kPQ - 1, T - 1);      // last key any query of this tile may see
  float m = -INFINITY, l = 0.f;
  float4 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);

  for (int kc = 0; kc <= kmax; kc += kPK) {
    for (int i = tid; i < kPK * half; i += kPThreads) {
      const int j = i / half, d = (i - j * half) * 2, p = kc + j;
      float2 r = make_float2(0.f, 0.f);
      if (p <= kmax) {
        if (p < pos0) {
          r = *reinterpret_cast<const float2*>(k_cache + cbase + (size_t)p * hd + d);
        } else {
          const int t = p - pos0;
          const float2 x = *reinterpret_cast<const float2*>(qkv + (size_t)(b * T + t) * row3 + (H + h) * hd + d);
          const size_t ri = (size_t)p * hd + d;
          const float c = cos2[ri], s = sin2[ri];
          r.x = x.x * c - x.y * s;
          r.y = x.y * c + x.x * s;
          if (t >= q0) *reinterpret_cast<float2*>(k_cache + cbase + (size_t)p * hd + d) = r;
        }
      }
      k_s[j * hdp + d] = r.x;
      k_s[j * hdp + d + 1] = r.y;
    }
    for (int i = tid; i < kPK * quarter; i += kPThreads) {
      const int j = i / quarter, d = (i - j * quarter) * 4, p = kc + j;
      float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p <= kmax) {
        if (p < pos0) {
          r = *reinterpret_cast<const float4*>(v_cache + cbase + (size_t)p * hd + d);
        } else {
          const int t = p - pos0;
          r = *reinterpret_cast<const float4*>(qkv + (size_t)(b * T + t) * row3 + (2 * H + h) * hd + d);
          if (t >= q0) *reinterpret_cast<float4*>(v_cache + cbase + (size_t)p * hd + d) = r;
        }
      }
      *reinterpret_cast<float4*>(v_s + j * hdp + d) = r;
    }
    __syncthreads();

    // scores of keys sub, sub + 8, sub + 16, sub + 24 of the chunk against query qi
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const float4* qr = reinterpret_cast<const float4*>(q_s + qi * hdp);
      const float4* kr = reinterpret_cast<const float4*>(k_s + sub * hdp);
      const int kstep = 8 * hdp / 4;
      for (int d4 = 0; d4 < quarter; ++d4) {
        const float4 x = qr[d4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 y = kr[i * kstep + d4];
          sc[i] += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
        }
      }
    }
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sc[i] = (kc + sub + 8 * i <= my_pos) ? sc[i] * scale : -INFINITY;
      cm = fmaxf(cm, sc[i]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
    const float m_new = fmaxf(m, cm);           // finite from the first chunk on: key 0 is visible to every query
    const float corr = expf(m - m_new);
    float ps = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pr = expf(sc[i] - m_new);
      p_s[qi * (kPK + 1) + sub + 8 * i] = pr;
      ps += pr;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * corr + ps;
    m = m_new;
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc[i].x *= corr; acc[i].y *= corr; acc[i].z *= corr; acc[i].w *= corr; }
    __syncwarp();                               // the eight threads of a query are lanes of one warp

    // numerator: head dimensions sub*4 + 32*i of query qi
    const float* pr = p_s + qi * (kPK + 1);
#pragma unroll 4
    for (int j = 0; j < kPK; ++j) {
      const float w = pr[j];
      const float* vr = v_s + j * hdp + sub * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (sub * 4 + 32 * i < hd) {
          const float4 v = *reinterpret_cast<const float4*>(vr + 32 * i);
          acc[i].x += w * v.x; acc[i].y += w * v.y; acc[i].z += w * v.z; acc[i].w += w * v.w;
        }
      }
    }
    __syncthreads();                            // before the next chunk overwrites K, V and the weights
  }
  if (q0 + qi < T) {
    const float inv = 1.f / l;
    float* o = out + (size_t)(b * T + q0 + qi) * out_stride + out_offset + h * hd + sub * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (sub * 4 + 32 * i < hd)
        *reinterpret_cast<float4*>(o + 32 * i) = make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv);
  }
}

// The tied LM head of one sequence as a matvec over the bf16 embedding table, with the final residual add + RMSNorm
// in front and the soft-cap + arg-max behind it (inference/generate_torch.py:155-160 and :300-310): logits[v] =
// cap * tanh(dot(table[v], norm(x + delta) * w) / cap).  HBM-bound (164 MB per token at V = 32000, C = 2560): CTA b
// owns the table rows [V*b/G, V*(b+1)/G); a warp takes every tenth of them through its own ring of 16-byte
// asynchronous copies (up to four slots of one row: three rows are in flight while one is multiplied, 150 KB per SM
// on the way — plain loads were sunk to their uses by the compiler, four in flight per lane) and multiplies them
// with the activations staged once in shared memory as fp32 (bf16 x fp32 products are exact in fp32).  The
// norm's scale is one factor on the dot products.  Every CTA leaves its best (value, index) as a candidate;
// lm_head_finish_kernel picks the token (largest capped logit, lowest index among equals) and advances the
// position.  C = 256 * NC: a lane owns eight values of every 256.
constexpr int kHeadWarps = 10;
constexpr int kHeadThreads = kHeadWarps * 32;
constexpr int kHeadMaxCtas = 1024;
constexpr int kHeadMaxNC = 12;                               // C <= 3072
constexpr size_t kHeadSmemBudget = 216 * 1024;               // activations + the warps' rings

__device__ __forceinline__ void head_cp_async16(void* dst, const void* src) {   // 16 bytes global -> shared, past L1
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kHeadThreads, 1) lm_head_kernel(const float* __restrict__ x, const float* __restrict__ delta,
                                                                  const float* __restrict__ w, float eps,
                                                                  const __nv_bfloat16* __restrict__ table, int V, int NC, int slots,
                                                                  float cap, float* __restrict__ logits_out,
                                                                  float* __restrict__ cand_val, int* __restrict__ cand_idx) {
  extern __shared__ __align__(16) uint8_t head_smem[];
  __shared__ float s_red[kHeadWarps];
  __shared__ int s_ci[kHeadWarps];
  __shared__ float s_scale;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = NC * 256, row_bytes = C * 2;
  float* hs = reinterpret_cast<float*>(head_smem);                                   // C floats
  uint8_t* ring = head_smem + (size_t)C * 4 + (size_t)warp * slots * row_bytes;     // [slots][row_bytes]
  const int G = gridDim.x, b = blockIdx.x;
  const int row0 = (int)((long long)V * b / G), row1 = (int)((long long)V * (b + 1) / G);
  // row i of this warp: row0 + warp + 10 i, copied into ring slot i % slots
  int rq = 0, rq_slot = 0;
  auto request = [&]() {
    const int r = row0 + warp + kHeadWarps * rq;
    if (r < row1) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(table) + (size_t)r * row_bytes;
      uint8_t* dst = ring + (size_t)rq_slot * row_bytes;
      for (int j = 0; j < NC; ++j) head_cp_async16(dst + (j * 32 + lane) * 16, src + (j * 32 + lane) * 16);
    }
    ++rq;
    if (++rq_slot == slots) rq_slot = 0;
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  asm volatile("griddepcontrol.launch_dependents;");
  for (int i = 0; i < slots - 1; ++i) request();             // the table does not depend on the launch before
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float ss = 0.f;
  for (int i4 = tid; i4 < C / 4; i4 += kHeadThreads) {
    float4 v = __ldcg(reinterpret_cast<const float4*>(x) + i4);
    if (delta) {
      const float4 d = __ldcg(reinterpret_cast<const float4*>(delta) + i4);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (w) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(w) + i4);
      v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
    }
    reinterpret_cast<float4*>(hs)[i4] = v;
  }
  ss = warp_sum(ss);
  if (lane == 0) s_red[warp] = ss;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int i = 0; i < kHeadWarps; ++i) tot += s_red[i];
    s_scale = w ? 1.0f / sqrtf(tot / (float)C + eps) : 1.0f;
  }
  __syncthreads();
  const float scale = s_scale;
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  int use_slot = 0;
#pragma unroll 1
  for (int r = row0 + warp; r < row1; r += kHeadWarps) {
    request();                                               // (past the end: an empty group)
    if (slots == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else if (slots == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    const uint8_t* pr = ring + (size_t)use_slot * row_bytes;
    float acc = 0.f;
#pragma unroll 2
    for (int j = 0; j < NC; ++j) {
      const float4 x0 = *reinterpret_cast<const float4*>(hs + (j * 32 + lane) * 8);
      const float4 x1 = *reinterpret_cast<const float4*>(hs + (j * 32 + lane) * 8 + 4);
      const uint4 t = *reinterpret_cast<const uint4*>(pr + (j * 32 + lane) * 16);
      // a word holds elements 2e (low half) and 2e + 1
      acc += __uint_as_float(t.x << 16) * x0.x + __uint_as_float(t.x & 0xffff0000u) * x0.y;
      acc += __uint_as_float(t.y << 16) * x0.z + __uint_as_float(t.y & 0xffff0000u) * x0.w;
      acc += __uint_as_float(t.z << 16) * x1.x + __uint_as_float(t.z & 0xffff0000u) * x1.y;
      acc += __uint_as_float(t.w << 16) * x1.z + __uint_as_float(t.w & 0xffff0000u) * x1.w;
    }
    if (++use_slot == slots) use_slot = 0;
    __syncwarp();                                            // every lane is done with this slot before it is requested again
    acc = warp_sum(acc);
    if (lane == 0) {
      const float y = cap * tanhf(acc * scale / cap);
      logits_out[r] = y;
      if (y > best || (y == best && r < best_i)) { best = y; best_i = r; }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                           // s_red is reused
  if (lane == 0) { s_red[warp] = best; s_ci[warp] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < kHeadWarps; ++i)
      if (s_red[i] > best || (s_red[i] == best && s_ci[i] < best_i)) { best = s_red[i]; best_i = s_ci[i]; }
    cand_val[b] = best;
    cand_idx[b] = best_i;
  }
}

__global__ void __launch_bounds__(256) lm_head_finish_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx, int G,
                                                             long long* __restrict__ token, long long* __restrict__ pos) {
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  pdl_enter();
  const int tid = threadIdx.x;
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = tid; i < G; i += 256) {
    const float v = cand_val[i];
    const int vi = cand_idx[i];
    if (v > best || (v == best && vi < best_i)) { best = v; best_i = vi; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((tid & 31) == 0) { s_val[tid >> 5] = best; s_idx[tid >> 5] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < 8; ++i)
      if (s_val[i] > best || (s_val[i] == best && s_idx[i] < best_i)) { best = s_val[i]; best_i = s_idx[i]; }
    token[0] = best_i == 0x7fffffff ? 0 : best_i;
    if (pos) *pos += 1;
  }
}


// h[b, i] = silu(gu[b, i]) * gu[b, F + i]
__global__ void silu_mul_kernel(const float* __restrict__ gu, float* __restrict__ hmid, int F, int total) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_enter();
  if (i >= total) return;
  const int b = i / F, c = i - b * F;
  const float g = gu[(size_t)b * 2 * F + c], u = gu[(size_t)b * 2 * F + F + c];
  hmid[i] = g / (1.0f + __expf(-g)) * u;
}

// out[b, :] = float(table[token[b], :]) for a bf16 (V, C) embedding table; one CTA per sequence.
__global__ void embed_rows_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ token, float* __restrict__ out,
                                  int C, int V) {
  pdl_enter();
  long long t = token[blockIdx.x];
  t = t < 0 ? 0 : (t >= V ? V - 1 : t);
  const __nv_bfloat16* row = table + (size_t)t * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) out[(size_t)blockIdx.x * C + i] = __bfloat162float(row[i]);
}

// The end of a decode step for one sequence per CTA: logits_out[b, v] = cap * tanh(float(logits[b, v]) / cap),
// token[b] = index of the largest capped logit (the lowest index among equals), and CTA 0 advances the
// position.  logits are bf16 (the LM-head product) or fp32.
constexpr int kFinishThreads = 1024;
__global__ void __launch_bounds__(kFinishThreads) softcap_argmax_kernel(const void* __restrict__ logits, int is_bf16, int V, float cap,
                                                                        float* __restrict__ logits_out, long long* __restrict__ token,
                                                                        long long* __restrict__ pos) {
  __shared__ float s_val[kFinishThreads / 32];
  __shared__ int s_idx[kFinishThreads / 32];
  pdl_enter();
  const int b = blockIdx.x, tid = threadIdx.x;
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i0 = tid; i0 < V; i0 += 8 * kFinishThreads) {  // eight loads in flight per thread
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * kFinishThreads;
      x[j] = 0.f;
      if (i < V)
        x[j] = is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[(size_t)b * V + i])
                       : reinterpret_cast<const float*>(logits)[(size_t)b * V + i];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * kFinishThreads;
      if (i < V) {
        const float y = cap * tanhf(x[j] / cap);
        logits_out[(size_t)b * V + i] = y;
        if (y > best || (y == best && i < best_i)) { best = y; best_i = i; }   // NaN never wins, as in a max-reduction that skips it
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((tid & 31) == 0) { s_val[tid >> 5] = best; s_idx[tid >> 5] = best_i; }
  __syncthreads();
  if (tid < 32) {
    best = s_val[tid]; best_i = s_idx[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (tid == 0) {
      token[b] = best_i == 0x7fffffff ? 0 : best_i;
      if (b == 0 && pos) *pos += 1;
    }
  }
}

}  // namespace nb

using namespace nb;

extern "C" int nb_embed_rows(const void* table_bf16, const int64_t* token, int B, int V, int C, float* out, void* stream) {
  if (!table_bf16 || !token || !out || B < 1 || V < 1 || C < 1) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  return launch_pdl(embed_rows_kernel, dim3(B), dim3(1024), 0, (cudaStream_t)stream, reinterpret_cast<const __nv_bfloat16*>(table_bf16),
                    reinterpret_cast<const long long*>(token), out, C, V);
}

extern "C" int nb_softcap_argmax(const void* logits, int logits_dtype, int B, int V, float cap, float* logits_out, int64_t* token,
                                 int64_t* pos, void* stream) {
  if (!logits || !logits_out || !token || B < 1 || V < 1 || !(cap > 0.f)) return NB_ERR_ARG;
  if (logits_dtype != NB_BF16 && logits_dtype != NB_F32) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  return launch_pdl(softcap_argmax_kernel, dim3(B), dim3(kFinishThreads), 0, (cudaStream_t)stream, logits,
                    logits_dtype == NB_BF16 ? 1 : 0, V, cap, logits_out, reinterpret_cast<long long*>(token),
                    reinterpret_cast<long long*>(pos));
}

extern "C" int nb_add_rmsnorm(float* x, const float* delta, const float* w, float eps, float* out, int B, int C, void* stream) {
  if (!x || !w || !out || B < 1 || C < 1) return NB_ERR_ARG;
  if (C > 16 * 256) return NB_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  return launch_pdl(add_rmsnorm_kernel, dim3(B), dim3(256), 0, (cudaStream_t)stream, x, delta, w, eps, out, C);
}

extern "C" int nb_rope_kv_write(const float* qkv, int B, int H, int hd, const float* cos2, const float* sin2, const int64_t* pos,
                                float* k_cache, float* v_cache, int ctx, float* q_out, void* stream) {
  if (!qkv || !cos2 || !sin2 || !pos || !k_cache || !v_cache || !q_out || B < 1 || H < 1 || hd < 2 || (hd & 1) || ctx < 1)
    return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  return launch_pdl(rope_kv_kernel, dim3(H, B), dim3(128), 0, (cudaStream_t)stream, qkv, cos2, sin2,
                    reinterpret_cast<const long long*>(pos), k_cache, v_cache, q_out, H, hd, ctx);
}

extern "C" int nb_decode_attention_rope(const float* qkv, const float* cos2, const float* sin2, const int64_t* pos, float* k_cache,
                                        float* v_cache, int B, int H, int hd, int ctx, float* out, int out_stride, int out_offset,
                                        void* stream) {
  if (!qkv || !cos2 || !sin2 || !k_cache || !v_cache || !pos || !out || B < 1 || H < 1 || hd < 2 || (hd & 1) || ctx < 1)
    return NB_ERR_ARG;
  if (hd > 128 || hd % 4 != 0) return NB_ERR_SHAPE;
  if ((uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  return launch_attention(B, H, hd, ctx, (cudaStream_t)stream, (const float*)nullptr, k_cache, v_cache,
                          reinterpret_cast<const long long*>(pos), out, H, hd, ctx, out_stride, out_offset, qkv, cos2, sin2);
}

extern "C" int nb_decode_attention(const float* q, const float* k_cache, const float* v_cache, const int64_t* pos, int B, int H,
                                   int hd, int ctx, float* out, int out_stride, int out_offset, void* stream) {
  if (!q || !k_cache || !v_cache || !pos || !out || B < 1 || H < 1 || hd < 1 || ctx < 1) return NB_ERR_ARG;
  if (hd > 128 || hd % 4 != 0) return NB_ERR_SHAPE;
  if ((uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16) return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  return launch_attention(B, H, hd, ctx, (cudaStream_t)stream, q, const_cast<float*>(k_cache), const_cast<float*>(v_cache),
                          reinterpret_cast<const long long*>(pos), out, H, hd, ctx, out_stride, out_offset, (const float*)nullptr,
                          (const float*)nullptr, (const float*)nullptr);
}

extern "C" int nb_prefill_attention(const float* qkv, int B, int T, int H, int hd, const float* cos2, const float* sin2, int pos0,
                                    float* k_cache, float* v_cache, int ctx, float* out, int out_stride, int out_offset,
                                    void* stream) {
  if (!qkv || !cos2 || !sin2 || !k_cache || !v_cache || !out || B < 1 || T < 1 || H < 1 || hd < 4 || ctx < 1 || pos0 < 0 ||
      out_stride < 1 || out_offset < 0)
    return NB_ERR_ARG;
  if (hd > 128 || hd % 4 != 0 || pos0 + T > ctx || out_offset + H * hd > out_stride) return NB_ERR_SHAPE;
  if ((uintptr_t)qkv % 16 || (uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16 || (uintptr_t)out % 16 || out_stride % 4 ||
      out_offset % 4)
    return NB_ERR_ALIGN;
  if (H > 65535 || B > 65535) return NB_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  const int hdp = hd + 4;
  const size_t smem = (size_t)((kPQ + 2 * kPK) * hdp + kPQ * (kPK + 1)) * sizeof(float);      // <= 44 KB
  prefill_attention_kernel<<<dim3((T + kPQ - 1) / kPQ, H, B), kPThreads, smem, (cudaStream_t)stream>>>(
      qkv, cos2, sin2, k_cache, v_cache, out, T, H, hd, ctx, pos0, out_stride, out_offset, 1.0f / sqrtf((float)hd));
  return record_cuda_error(cudaGetLastError());
}

extern "C" size_t nb_lm_head_scratch_bytes(void) { return (size_t)kHeadMaxCtas * 8; }

extern "C" int nb_lm_head(const float* x, const float* delta, const float* norm_weight, float eps, const void* table_bf16, int V, int C,
                          float cap, float* logits_out, int64_t* token, int64_t* pos, void* scratch, void* stream) {
  if (!x || !table_bf16 || !logits_out || !token || !scratch || V < 1 || C < 1 || !(cap > 0.f)) return NB_ERR_ARG;
  if (C % 256 != 0 || C / 256 > kHeadMaxNC) return NB_ERR_SHAPE;
  if ((uintptr_t)x % 16 || (uintptr_t)delta % 16 || (uintptr_t)norm_weight % 16 || (uintptr_t)table_bf16 % 16 || (uintptr_t)scratch % 16)
    return NB_ERR_ALIGN;
  if (int rc = check_device()) return rc;
  const int G = std::min(std::min(sm_count(), kHeadMaxCtas), V);
  float* cv = reinterpret_cast<float*>(scratch);
  int* ci = reinterpret_cast<int*>(cv + kHeadMaxCtas);
  cudaStream_t st = (cudaStream_t)stream;
  // ring slots per warp: as many rows in flight as the shared memory holds (4 at C = 2560, 3 at C = 3072)
  const size_t ring_row = (size_t)kHeadWarps * C * 2;
  const int slots = (int)std::min<size_t>(4, (kHeadSmemBudget - (size_t)C * 4) / ring_row);
  if (slots < 2) return NB_ERR_SHAPE;
  const size_t smem = (size_t)C * 4 + (size_t)slots * ring_row;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    if (cudaError_t e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHeadSmemBudget)) return record_cuda_error(e);
    attr_done[dev & 63] = true;
  }
  if (int rc = launch_pdl(lm_head_kernel, dim3(G), dim3(kHeadThreads), smem, st, x, delta, norm_weight, eps,
                          reinterpret_cast<const __nv_bfloat16*>(table_bf16), V, C / 256, slots, cap, logits_out, cv, ci))
    return rc;
  return launch_pdl(lm_head_finish_kernel, dim3(1), dim3(256), 0, st, (const float*)cv, (const int*)ci, G,
                    reinterpret_cast<long long*>(token), reinterpret_cast<long long*>(pos));
}

extern "C" int nb_silu_mul(const float* gu, int B, int F, float* hmid, void* stream) {
  if (!gu || !hmid || B < 1 || F < 1) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  const int total = B * F;
  return launch_pdl(silu_mul_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, gu, hmid, F, total);
}

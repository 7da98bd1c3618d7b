// Small fused kernels of the decode step around the packed GEMVs (one new token per sequence):
// residual add + RMSNorm, RoPE + KV-cache write, single-query attention over the valid prefix of
// the cache, and SiLU(gate) * up.  All activations are fp32, as in the reference's cached path
// (inference/generate_torch.py:29-38 RMSNorm, :41-60 RoPE on interleaved pairs, :86-97 cache write
// and masked attention, :116-117 SwiGLU).  The position is read from device memory so that the
// step can be replayed from a CUDA graph.
#include <cuda_runtime.h>

#include <cfloat>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

// Every kernel of the decode chain is launched with programmatic stream serialization: it may be
// scheduled while its predecessor still runs, lets its own successor do the same, and waits for
// the predecessor's results before it touches memory.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
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
  pdl_enter();
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
// values.  out[b, out_offset + h*hd + d].  grid (H, B), 256 threads.  Warps take keys round robin,
// lanes run over the head dimension (rows of the cache are contiguous), four keys per iteration so
// that a dozen loads per lane are in flight; head_dim <= 128.  Dynamic smem: ctx + 9*hd floats.
constexpr int kAttnWarps = 8;
// When `qkv` is given (B, 3*H*hd = [q|k|v]) the kernel first does the work of rope_kv_kernel for its
// head: it rotates q and k by the position's angle, writes k and v into the caches at `pos` and
// attends with the rotated q, so the step needs one launch instead of two.
__global__ void __launch_bounds__(kAttnWarps * 32) decode_attention_kernel(
    const float* __restrict__ q, float* __restrict__ k_cache, float* __restrict__ v_cache,
    const long long* __restrict__ pos_ptr, float* __restrict__ out, int H, int hd, int ctx, int out_stride, int out_offset,
    const float* __restrict__ qkv, const float* __restrict__ cos2, const float* __restrict__ sin2) {
  extern __shared__ float sc[];  // ctx scores | hd query values | kAttnWarps x hd partial outputs
  __shared__ float red[kAttnWarps];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_enter();
  long long pos = *pos_ptr;
  if (pos < 0) return;
  if (pos >= ctx) pos = ctx - 1;
  const int n = (int)pos + 1;
  float* qs = sc + ctx;
  float* part = qs + hd;
  const size_t head = ((size_t)b * H + h);
  if (qkv) {
    const float* base = qkv + (size_t)b * 3 * H * hd;
    const float* qh = base + h * hd;
    const float* kh = base + H * hd + h * hd;
    const float* vh = base + 2 * H * hd + h * hd;
    const size_t crow = (head * ctx + pos) * hd;
    for (int i = tid; i < hd; i += blockDim.x) {
      const float c = cos2[pos * hd + i], s = sin2[pos * hd + i];
      const int j = i ^ 1;
      const float sign = (i & 1) ? 1.f : -1.f;   // rot = (-x2, x1) on interleaved pairs
      qs[i] = (qh[i] * c + sign * qh[j] * s) * rsqrtf((float)hd);
      k_cache[crow + i] = kh[i] * c + sign * kh[j] * s;
      v_cache[crow + i] = vh[i];
    }
  } else {
    for (int i = tid; i < hd; i += blockDim.x) qs[i] = q[head * hd + i] * rsqrtf((float)hd);
  }
  __syncthreads();
  const float* kb = k_cache + head * ctx * hd;
  const float* vb = v_cache + head * ctx * hd;
  float qv[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) qv[e] = (lane + 32 * e < hd) ? qs[lane + 32 * e] : 0.f;

  float mx = -FLT_MAX;
  for (int j0 = warp; j0 < n; j0 += 4 * kAttnWarps) {
    float s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kAttnWarps;
      s[u] = 0.f;
      if (j < n) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (lane + 32 * e < hd) s[u] += qv[e] * kb[(size_t)j * hd + lane + 32 * e];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kAttnWarps;
      const float t = warp_sum(s[u]);
      if (j < n) {
        if (lane == 0) sc[j] = t;
        mx = fmaxf(mx, t);
      }
    }
  }
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < kAttnWarps; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < n; j += blockDim.x) {
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
  const float inv = 1.0f / tot;

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = warp; j0 < n; j0 += 4 * kAttnWarps) {
    float vv[4][4], pj[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * kAttnWarps;
      pj[u] = (j < n) ? sc[j] : 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        vv[u][e] = (j < n && lane + 32 * e < hd) ? vb[(size_t)j * hd + lane + 32 * e] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] += pj[u] * vv[u][e];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (lane + 32 * e < hd) part[warp * hd + lane + 32 * e] = acc[e];
  __syncthreads();
  for (int d = tid; d < hd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int wi = 0; wi < kAttnWarps; ++wi) o += part[wi * hd + d];
    out[(size_t)b * out_stride + out_offset + h * hd + d] = o * inv;
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

}  // namespace nb

using namespace nb;

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
  if (hd > 128 || (size_t)(ctx + 9 * hd) * sizeof(float) > 48 * 1024) return NB_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  return launch_pdl(decode_attention_kernel, dim3(H, B), dim3(kAttnWarps * 32), (size_t)(ctx + 9 * hd) * sizeof(float),
                    (cudaStream_t)stream, (const float*)nullptr, k_cache, v_cache, reinterpret_cast<const long long*>(pos), out, H,
                    hd, ctx, out_stride, out_offset, qkv, cos2, sin2);
}

extern "C" int nb_decode_attention(const float* q, const float* k_cache, const float* v_cache, const int64_t* pos, int B, int H,
                                   int hd, int ctx, float* out, int out_stride, int out_offset, void* stream) {
  if (!q || !k_cache || !v_cache || !pos || !out || B < 1 || H < 1 || hd < 1 || ctx < 1) return NB_ERR_ARG;
  if (hd > 128 || (size_t)(ctx + 9 * hd) * sizeof(float) > 48 * 1024) return NB_ERR_SHAPE;
  if (int rc = check_device()) return rc;
  return launch_pdl(decode_attention_kernel, dim3(H, B), dim3(kAttnWarps * 32), (size_t)(ctx + 9 * hd) * sizeof(float),
                    (cudaStream_t)stream, q, const_cast<float*>(k_cache), const_cast<float*>(v_cache),
                    reinterpret_cast<const long long*>(pos), out, H, hd, ctx, out_stride, out_offset, (const float*)nullptr,
                    (const float*)nullptr, (const float*)nullptr);
}

extern "C" int nb_silu_mul(const float* gu, int B, int F, float* hmid, void* stream) {
  if (!gu || !hmid || B < 1 || F < 1) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  const int total = B * F;
  return launch_pdl(silu_mul_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, gu, hmid, F, total);
}

// Bit-unpack, bit-pack and whole-weight dequantisation kernels (integer / gather work, HBM bound).
//
// All three treat the packed buffer as one LSB-first bit stream: index i occupies bits
// [i*bits, (i+1)*bits).  That is what the reference's three packers produce
// (nativebit/pack.py:21-41, 75-82, 97-116).
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint32_t stream_index(const uint8_t* __restrict__ p, int64_t n_bytes, int64_t i, int bits) {
  const int64_t bit = i * bits;
  const int64_t byte = bit >> 3;
  uint32_t v = p[byte];
  if (((int)(bit & 7) + bits > 8) && byte + 1 < n_bytes) v |= (uint32_t)p[byte + 1] << 8;
  return (v >> (bit & 7)) & ((1u << bits) - 1u);
}

__host__ __device__ inline int64_t packed_bytes(int64_t count, int bits) {
  return bits == 3 ? 3 * ((count + 7) / 8) : (count * bits + 7) / 8;
}

// ---- unpack -------------------------------------------------------------------------------
// Fast path: one thread turns `BITS` aligned 32-bit words into 32 indices (two 16-byte stores).
template <int BITS>
__global__ void unpack32_kernel(const uint32_t* __restrict__ packed, int64_t n_chunks, uint4* __restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  uint32_t w[BITS];
#pragma unroll
  for (int i = 0; i < BITS; ++i) w[i] = packed[c * BITS + i];
  uint32_t o[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    uint32_t v = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int bit = (4 * r + j) * BITS;
      const int wi = bit >> 5, sh = bit & 31;
      uint32_t f = w[wi] >> sh;
      if (sh + BITS > 32 && wi + 1 < BITS) f |= w[wi + 1] << (32 - sh);
      v |= (f & ((1u << BITS) - 1u)) << (8 * j);
    }
    o[r] = v;
  }
  out[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
  out[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

__global__ void unpack_generic_kernel(const uint8_t* __restrict__ packed, int64_t n_bytes, int bits, int64_t first,
                                      int64_t count, uint8_t* __restrict__ out) {
  const int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  out[i] = (uint8_t)stream_index(packed, n_bytes, i, bits);
}

// ---- pack ---------------------------------------------------------------------------------
// One thread writes one output byte: it ORs the (at most 5) indices that overlap the byte.
__global__ void pack_kernel(const uint8_t* __restrict__ idx, int64_t count, int bits, int64_t n_bytes,
                            uint8_t* __restrict__ out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_bytes) return;
  const int64_t lo_bit = b * 8, hi_bit = lo_bit + 8;
  const uint32_t mask = (1u << bits) - 1u;
  uint32_t v = 0;
  for (int64_t i = lo_bit / bits; i * bits < hi_bit; ++i) {
    const uint32_t f = (i < count) ? (idx[i] & mask) : 0u;
    const int64_t sh = i * bits - lo_bit;
    v |= sh >= 0 ? (f << sh) : (f >> (-sh));
  }
  out[b] = (uint8_t)v;
}

// ---- dequant ------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T from_half_bits(uint32_t h16);
template <> __device__ __forceinline__ __half from_half_bits<__half>(uint32_t h) { return __ushort_as_half((unsigned short)h); }
template <> __device__ __forceinline__ float from_half_bits<float>(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
template <> __device__ __forceinline__ __nv_bfloat16 from_half_bits<__nv_bfloat16>(uint32_t h) {
  return __float2bfloat16_rn(__half2float(__ushort_as_half((unsigned short)h)));
}

// Fast path (fp16 codebook, block_size % 32 == 0, aligned): one thread dequantises 32
// consecutive weights of one block.  The 2^BITS entry table lives in registers as a low-byte
// plane and a high-byte plane; each lookup is two byte-permutes.
template <int BITS, typename OutT>
__global__ void dequant32_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ codebook,
                                 int64_t n_chunks, int block_size, OutT* __restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  uint32_t w[BITS];
#pragma unroll
  for (int i = 0; i < BITS; ++i) w[i] = packed[c * BITS + i];
  const int64_t block = (c * 32) / block_size;
  uint32_t lo0, lo1, hi0, hi1;
  if (BITS == 3) {
    const uint4 e = *reinterpret_cast<const uint4*>(codebook + block * 8);
    lo0 = prmt(e.x, e.y, 0x6420); lo1 = prmt(e.z, e.w, 0x6420);
    hi0 = prmt(e.x, e.y, 0x7531); hi1 = prmt(e.z, e.w, 0x7531);
  } else {
    const uint2 e = *reinterpret_cast<const uint2*>(codebook + block * 4);
    lo0 = prmt(e.x, e.y, 0x6420); hi0 = prmt(e.x, e.y, 0x7531);
    lo1 = 0; hi1 = 0;
  }
  alignas(16) OutT v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int bit = j * BITS;
    const int wi = bit >> 5, sh = bit & 31;
    uint32_t f = w[wi] >> sh;
    if (sh + BITS > 32 && wi + 1 < BITS) f |= w[wi + 1] << (32 - sh);
    f &= (1u << BITS) - 1u;
    const uint32_t h = (prmt(lo0, lo1, f) & 0xFFu) | ((prmt(hi0, hi1, f) & 0xFFu) << 8);
    v[j] = from_half_bits<OutT>(h);
  }
  // 16-byte stores (out + 32*c is 16-byte aligned for 2- and 4-byte element types)
  const uint4* src = reinterpret_cast<const uint4*>(v);
  uint4* dst = reinterpret_cast<uint4*>(out + c * 32);
#pragma unroll
  for (int j = 0; j < (int)(32 * sizeof(OutT) / 16); ++j) dst[j] = src[j];
}

template <typename CbT, typename OutT>
__global__ void dequant_generic_kernel(const uint8_t* __restrict__ packed, int64_t n_bytes, const CbT* __restrict__ codebook,
                                       int bits, int block_size, int64_t first, int64_t total, OutT* __restrict__ out) {
  const int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const uint32_t e = stream_index(packed, n_bytes, i, bits);
  const float v = (float)codebook[(i / block_size) * (1 << bits) + e];
  out[i] = (OutT)v;
}

// ---- quantise: nearest codebook entry per weight (the exporter's argmin) ------------------------
// idx[i] = argmin_e |w[i] - codebook[i / block_size][e]|, first minimum on ties; weights past `total`
// (padding of the last block) count as 0, as in the reference's zero-padded argmin.
template <typename CbT>
__global__ void quantize_kernel(const float* __restrict__ w, int64_t total, int64_t padded, const CbT* __restrict__ codebook,
                                int n_entries, int block_size, uint8_t* __restrict__ idx) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= padded) return;
  const float v = i < total ? w[i] : 0.f;
  const CbT* cb = codebook + (i / block_size) * n_entries;
  float best = fabsf(v - (float)cb[0]);
  int arg = 0;
  for (int e = 1; e < n_entries; ++e) {
    const float d = fabsf(v - (float)cb[e]);
    if (d < best) { best = d; arg = e; }
  }
  idx[i] = (uint8_t)arg;
}

template <typename OutT>
static int dequant_dispatch(const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size,
                            int64_t total, OutT* out, cudaStream_t st) {
  const int64_t n_blocks = (total + block_size - 1) / block_size;
  const int64_t n_bytes = packed_bytes(n_blocks * block_size, bits);
  int64_t done = 0;
  const bool aligned = ((uintptr_t)packed % 4 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)codebook % 16 == 0);
  if (cb_dtype == NB_F16 && (bits == 2 || bits == 3) && block_size % 32 == 0 && aligned) {
    const int64_t chunks = total / 32;
    if (chunks > 0) {
      const unsigned grid = (unsigned)((chunks + 127) / 128);
      if (bits == 3)
        dequant32_kernel<3, OutT><<<grid, 128, 0, st>>>((const uint32_t*)packed, (const __half*)codebook, chunks, block_size, out);
      else
        dequant32_kernel<2, OutT><<<grid, 128, 0, st>>>((const uint32_t*)packed, (const __half*)codebook, chunks, block_size, out);
      done = chunks * 32;
    }
  }
  if (done < total) {
    const int64_t rest = total - done;
    const unsigned grid = (unsigned)((rest + 255) / 256);
    if (cb_dtype == NB_F16)
      dequant_generic_kernel<__half, OutT><<<grid, 256, 0, st>>>(packed, n_bytes, (const __half*)codebook, bits, block_size, done, total, out);
    else
      dequant_generic_kernel<float, OutT><<<grid, 256, 0, st>>>(packed, n_bytes, (const float*)codebook, bits, block_size, done, total, out);
  }
  return check_launch();
}

}  // namespace nb

using namespace nb;

extern "C" int nb_unpack(const uint8_t* packed, int bits, int64_t count, uint8_t* idx_out, void* stream) {
  if (!packed || !idx_out || count < 0 || (bits != 2 && bits != 3 && bits != 4)) return NB_ERR_ARG;
  if (count == 0) return NB_OK;
  if (int rc = check_device()) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n_bytes = packed_bytes(count, bits);
  int64_t done = 0;
  if ((uintptr_t)packed % 4 == 0 && (uintptr_t)idx_out % 16 == 0) {
    const int64_t chunks = count / 32;
    if (chunks > 0) {
      const unsigned grid = (unsigned)((chunks + 255) / 256);
      if (bits == 2) unpack32_kernel<2><<<grid, 256, 0, st>>>((const uint32_t*)packed, chunks, (uint4*)idx_out);
      if (bits == 3) unpack32_kernel<3><<<grid, 256, 0, st>>>((const uint32_t*)packed, chunks, (uint4*)idx_out);
      if (bits == 4) unpack32_kernel<4><<<grid, 256, 0, st>>>((const uint32_t*)packed, chunks, (uint4*)idx_out);
      done = chunks * 32;
    }
  }
  if (done < count) {
    const unsigned grid = (unsigned)((count - done + 255) / 256);
    unpack_generic_kernel<<<grid, 256, 0, st>>>(packed, n_bytes, bits, done, count, idx_out);
  }
  return check_launch();
}

extern "C" int nb_pack(const uint8_t* idx, int bits, int64_t count, uint8_t* packed_out, void* stream) {
  if (!idx || !packed_out || count < 0 || (bits != 2 && bits != 3 && bits != 4)) return NB_ERR_ARG;
  if (count == 0) return NB_OK;
  if (int rc = check_device()) return rc;
  const int64_t n_bytes = packed_bytes(count, bits);
  const unsigned grid = (unsigned)((n_bytes + 255) / 256);
  pack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(idx, count, bits, n_bytes, packed_out);
  return check_launch();
}

extern "C" int nb_dequant(const uint8_t* packed, const void* codebook, int cb_dtype, int bits, int block_size,
                          int64_t n_rows, int64_t n_cols, void* w_out, int w_dtype, void* stream) {
  if (!packed || !codebook || !w_out || n_rows <= 0 || n_cols <= 0 || block_size <= 0) return NB_ERR_ARG;
  if (bits != 2 && bits != 3 && bits != 4) return NB_ERR_ARG;
  if (cb_dtype != NB_F16 && cb_dtype != NB_F32) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  const int64_t total = n_rows * n_cols;
  cudaStream_t st = (cudaStream_t)stream;
  switch (w_dtype) {
    case NB_F32: return dequant_dispatch<float>(packed, codebook, cb_dtype, bits, block_size, total, (float*)w_out, st);
    case NB_F16: return dequant_dispatch<__half>(packed, codebook, cb_dtype, bits, block_size, total, (__half*)w_out, st);
    case NB_BF16: return dequant_dispatch<__nv_bfloat16>(packed, codebook, cb_dtype, bits, block_size, total, (__nv_bfloat16*)w_out, st);
    default: return NB_ERR_ARG;
  }
}

extern "C" int nb_quantize(const float* w, int64_t total, const void* codebook, int cb_dtype, int n_entries, int block_size,
                           uint8_t* idx_out, void* stream) {
  if (!w || !codebook || !idx_out || total <= 0 || block_size <= 0 || n_entries < 2 || n_entries > 256) return NB_ERR_ARG;
  if (cb_dtype != NB_F16 && cb_dtype != NB_F32) return NB_ERR_ARG;
  if (int rc = check_device()) return rc;
  const int64_t padded = (total + block_size - 1) / block_size * block_size;
  const unsigned grid = (unsigned)((padded + 255) / 256);
  if (cb_dtype == NB_F16)
    quantize_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(w, total, padded, (const __half*)codebook, n_entries, block_size, idx_out);
  else
    quantize_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(w, total, padded, (const float*)codebook, n_entries, block_size, idx_out);
  return check_launch();
}

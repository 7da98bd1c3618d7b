// Shared definitions for the NativeBit B200 kernels: status codes, dtype tags and the
// in-register index-unpack scheme used by the decode GEMV and the prefill GEMM.
//
// Packed layout consumed here is exactly what the reference's packer writes
// (nativebit/pack.py:21-41 for 3-bit: index j of a group of 8 sits at bits [3j,3j+3) of a
// little-endian 24-bit word; nativebit/pack.py:97-116 for 2-bit: LSB-first bit stream, so
// index j of a byte sits at bits [2j,2j+2); nativebit/pack.py:75-82 for 4-bit: low nibble first).
// A codebook block covers 128 consecutive weights = 48 bytes (3-bit), 32 bytes (2-bit) or 64 bytes (4-bit).
#pragma once
#include <cstdint>
#include <cstddef>

#include "../../include/nativebit_b200.h"

#if defined(__CUDACC__)
#define NB_HD __host__ __device__ __forceinline__
#else
#define NB_HD inline
#endif

namespace nb {

constexpr int kBlock = 128;  // weights per codebook block handled by the fast kernels

template <int BITS> struct Fmt;
template <> struct Fmt<3> { static constexpr int kWords = 12; static constexpr int kEntries = 8; };
template <> struct Fmt<2> { static constexpr int kWords = 8;  static constexpr int kEntries = 4; };
template <> struct Fmt<4> { static constexpr int kWords = 16; static constexpr int kEntries = 16; };

NB_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, int s) {
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, s);
#else
  return (uint32_t)(((((uint64_t)hi) << 32) | lo) >> s);
#endif
}

// ---------------------------------------------------------------------------------------
// Selector words.  A "selector word" holds eight codebook indices, one per nibble, with bit 3
// of every nibble clear, i.e. it is directly usable (16 bits at a time) as the control operand
// of a byte-permute that gathers four table bytes.  A block is processed in 4 groups; a group
// is 32 indices and yields 4 selector words.
//
// 3-bit: a group is three 32-bit words (96 bits, fields f0..f31 at bit 3f).  Fields whose bit
// position plus a left shift of 0..3 is a multiple of 4 are moved to their nibble with one
// mask each (left shifts are multiplies, which keeps them off the logic pipe); f10 and f21
// straddle a word boundary and come from a funnel shift, f31 from a plain right shift.
// field3(u, k) is the field that ends up in nibble k of selector word u.
// ---------------------------------------------------------------------------------------
NB_HD void selectors3(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t (&U)[4]) {
  const uint32_t a1 = w0 * 2u, a2 = w0 * 4u, a3 = w0 * 8u;
  const uint32_t b1 = w1 * 2u, b2 = w1 * 4u, b3 = w1 * 8u;
  const uint32_t c1 = w2 * 2u, c2 = w2 * 4u, c3 = w2 * 8u;
  U[0] = (w0 & 0x07007007u) | (a1 & 0x70070070u) | (a2 & 0x00700700u);
  U[1] = (funnel_r(w0, w1, 30) & 0x7u) | (w1 & 0x70070070u) | (b1 & 0x00700700u) | (b2 & 0x07007000u);
  U[2] = (funnel_r(w1, w2, 31) & 0x7u) | (c2 & 0x70070070u) | (w2 & 0x00700700u) | (c1 & 0x07007000u);
  U[3] = (w2 >> 29) | (b3 & 0x70070070u) | (c3 & 0x00700700u) | (a3 & 0x07007000u);
}
// One byte per nibble, nibble 0 in the low byte.
NB_HD int field3(int u, int k) {
  const uint64_t c = u == 0 ? 0x0908060504020100ull   // {0,1,2,4,5,6,8,9}
                   : u == 1 ? 0x141211100E0D0C0Aull   // {10,12,13,14,16,17,18,20}
                   : u == 2 ? 0x1E1D1C1A19181615ull   // {21,22,24,25,26,28,29,30}
                            : 0x13071B0F03170B1Full;  // {31,11,23,3,15,27,7,19}
  return (int)((c >> (8 * k)) & 0xFFu);
}

// 2-bit: a group is two 32-bit words of 16 fields; even fields are already nibble aligned,
// odd fields after a right shift by 2.
NB_HD void selectors2(uint32_t w0, uint32_t w1, uint32_t (&U)[4]) {
  U[0] = w0 & 0x33333333u;
  U[1] = (w0 >> 2) & 0x33333333u;
  U[2] = w1 & 0x33333333u;
  U[3] = (w1 >> 2) & 0x33333333u;
}

// Position inside the 128-weight block of the index that nibble k (0..7) of selector word u
// (0..3) of group q (0..3) holds.
template <int BITS> NB_HD int slot_position(int q, int u, int k);
template <> NB_HD int slot_position<3>(int q, int u, int k) { return 32 * q + field3(u, k); }
template <> NB_HD int slot_position<2>(int q, int u, int k) { return 32 * q + 16 * (u >> 1) + 2 * k + (u & 1); }
// 4-bit (nativebit/pack.py:75-82: low nibble first): a packed word already holds eight indices in
// order, one per nibble; bit 3 of a nibble is part of the index, so the lookup splits it off.
template <> NB_HD int slot_position<4>(int q, int u, int k) { return 32 * q + 8 * u + k; }

template <int BITS> NB_HD void group_selectors(const uint32_t* w, int q, uint32_t (&U)[4]);
template <> NB_HD void group_selectors<3>(const uint32_t* w, int q, uint32_t (&U)[4]) {
  selectors3(w[3 * q], w[3 * q + 1], w[3 * q + 2], U);
}
template <> NB_HD void group_selectors<2>(const uint32_t* w, int q, uint32_t (&U)[4]) {
  selectors2(w[2 * q], w[2 * q + 1], U);
}

template <> NB_HD void group_selectors<4>(const uint32_t* w, int q, uint32_t (&U)[4]) {
  U[0] = w[4 * q]; U[1] = w[4 * q + 1]; U[2] = w[4 * q + 2]; U[3] = w[4 * q + 3];
}

// A contraction "step" consumes four weights of a block: step s = 8q + 2u + h uses nibbles
// 4h..4h+3 of selector word u of group q.  slot = 4*s + i is the order in which the kernels
// see the weights of a block; the activation tile is staged in the same order.
template <int BITS> NB_HD int slot_to_position(int slot) {
  const int s = slot >> 2, i = slot & 3;
  return slot_position<BITS>(s >> 3, (s >> 1) & 3, 4 * (s & 1) + i);
}

}  // namespace nb

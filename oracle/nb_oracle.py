"""CPU oracle for the NativeBit packed-inference path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy (and, for the timed CPU baseline, in CPU torch ops
that mirror the reference op for op), the algorithm of the reference's packed
linear: bit-unpack -> per-block codebook gather -> contraction with activations.
It is the checker that the CUDA path is compared with.  Nothing in the product
package may import it: only the tests, the smoke check and the benchmark's CPU
baseline leg do.

Parity status: PINNED.  Every function here is checked against golden vectors
that were produced by importing the reference's own Python functions (the
generator script sits next to the vectors in tests/golden/).

Reference locations each function follows (paths are inside the reference repo):
  pack_3bit / unpack_3bit        nativebit/pack.py:21-41, 44-68
  pack_4bit / unpack_4bit        nativebit/pack.py:75-82, 85-90
  pack_nbits / unpack_nbits      nativebit/pack.py:97-116, 119-138 (bit-serial, LSB first)
  reconstruct_weight             nativebit/pack.py:145-169
  inference_linear_forward       nativebit/inference.py:42-46
  packed_linear_forward          inference/triton_kernel.py:258-275 (batched path)
  fused_matvec_3bit              inference/cuda_kernel.py:38-82 (scalar loop order)
  pack_indices_to_3bit           inference/triton_kernel.py:199-220, inference/pack.py:38-57
"""
from __future__ import annotations

import math

import numpy as np

BS = 128  # weights per codebook block (inference/triton_kernel.py:18)
NE = 8    # codebook entries per block for 3-bit (inference/triton_kernel.py:19)


# --------------------------------------------------------------------------- packing
def pack_3bit(indices: np.ndarray) -> np.ndarray:
    """8 indices -> 3 bytes; index j occupies bits [3j, 3j+3) of a little-endian
    24-bit word.  Input is zero-padded to a multiple of 8 (nativebit/pack.py:21-41)."""
    idx = np.asarray(indices, dtype=np.uint8).reshape(-1)
    pad = (-idx.size) % 8
    if pad:
        idx = np.concatenate([idx, np.zeros(pad, np.uint8)])
    g = idx.reshape(-1, 8).astype(np.uint32)
    bits24 = np.zeros(g.shape[0], np.uint32)
    for j in range(8):
        bits24 |= (g[:, j] & 7) << (3 * j)
    out = np.empty((g.shape[0], 3), np.uint8)
    out[:, 0] = bits24 & 0xFF
    out[:, 1] = (bits24 >> 8) & 0xFF
    out[:, 2] = (bits24 >> 16) & 0xFF
    return out.reshape(-1)


def unpack_3bit(packed: np.ndarray, count: int) -> np.ndarray:
    """Inverse of pack_3bit (nativebit/pack.py:44-68)."""
    p = np.asarray(packed, dtype=np.uint8).reshape(-1, 3).astype(np.uint32)
    bits24 = p[:, 0] | (p[:, 1] << 8) | (p[:, 2] << 16)
    out = np.empty((p.shape[0], 8), np.uint8)
    for j in range(8):
        out[:, j] = (bits24 >> (3 * j)) & 7
    return out.reshape(-1)[:count]


def pack_4bit(indices: np.ndarray) -> np.ndarray:
    """Two indices per byte, low nibble first (nativebit/pack.py:75-82)."""
    idx = np.asarray(indices, dtype=np.uint8).reshape(-1)
    if idx.size % 2:
        idx = np.concatenate([idx, np.zeros(1, np.uint8)])
    g = idx.reshape(-1, 2)
    return (g[:, 0] | (g[:, 1] << 4)).astype(np.uint8)


def unpack_4bit(packed: np.ndarray, count: int) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8).reshape(-1)
    return np.stack([p & 0xF, (p >> 4) & 0xF], axis=1).reshape(-1)[:count]


def pack_nbits(indices: np.ndarray, bits: int) -> np.ndarray:
    """Generic LSB-first bit stream (nativebit/pack.py:97-116), vectorised: bit b of
    index i lands at stream position i*bits+b; stream position p is bit p%8 of byte p//8."""
    if bits == 3:
        return pack_3bit(indices)
    if bits == 4:
        return pack_4bit(indices)
    idx = np.asarray(indices).reshape(-1).astype(np.uint32)
    n_bytes = math.ceil(idx.size * bits / 8)
    stream = ((idx[:, None] >> np.arange(bits, dtype=np.uint32)[None, :]) & 1).astype(np.uint8).reshape(-1)
    stream = np.concatenate([stream, np.zeros(n_bytes * 8 - stream.size, np.uint8)])
    return np.packbits(stream.reshape(-1, 8), axis=1, bitorder="little").reshape(-1)


def unpack_nbits(packed: np.ndarray, count: int, bits: int) -> np.ndarray:
    if bits == 3:
        return unpack_3bit(packed, count)
    if bits == 4:
        return unpack_4bit(packed, count)
    p = np.asarray(packed, dtype=np.uint8).reshape(-1)
    stream = np.unpackbits(p, bitorder="little")[: count * bits].reshape(count, bits).astype(np.uint32)
    return (stream << np.arange(bits, dtype=np.uint32)[None, :]).sum(axis=1).astype(np.uint8)


def pack_indices_to_3bit(indices_uint8: np.ndarray) -> np.ndarray:
    """The loader-side packer (inference/triton_kernel.py:199-220) produces the same
    bytes as pack_3bit."""
    return pack_3bit(indices_uint8)


# --------------------------------------------------------------------------- quantise
def quantize_weight(weight: np.ndarray, codebook: np.ndarray, block_size: int) -> np.ndarray:
    """Nearest codebook entry per weight, first minimum on ties, the zero-padded tail included
    (nativebit/pack.py:176-199; the same argmin as nativebit/layers.py:84-86 and
    nativebit/inference.py:60-67).  Returns (num_blocks * block_size,) uint8."""
    nb = codebook.shape[0]
    w = np.zeros(nb * block_size, np.float32)
    w[:weight.size] = np.asarray(weight, np.float32).reshape(-1)
    d = np.abs(w.reshape(nb, block_size, 1) - np.asarray(codebook, np.float32)[:, None, :])
    return d.argmin(-1).astype(np.uint8).reshape(-1)


# --------------------------------------------------------------------------- dequant
def reconstruct_weight(indices: np.ndarray, codebook: np.ndarray, shape, block_size: int,
                       total_weights: int) -> np.ndarray:
    """W.flat[b*block_size + t] = codebook[b, idx[b, t]], truncated to total_weights
    (nativebit/pack.py:145-169).  Returns an array of codebook's dtype."""
    nb = codebook.shape[0]
    idx = np.asarray(indices).reshape(nb, block_size).astype(np.int64)
    w = np.take_along_axis(codebook, idx, axis=1)
    return w.reshape(-1)[:total_weights].reshape(shape)


def dequant_packed(packed: np.ndarray, codebook: np.ndarray, n_rows: int, n_cols: int,
                   bits: int = 3, block_size: int = BS) -> np.ndarray:
    """unpack + reconstruct for a whole (n_rows, n_cols) weight."""
    nb = codebook.shape[0]
    idx = unpack_nbits(packed, nb * block_size, bits)
    return reconstruct_weight(idx, codebook, (n_rows, n_cols), block_size, n_rows * n_cols)


# --------------------------------------------------------------------------- linear
def inference_linear_forward(x: np.ndarray, indices: np.ndarray, codebook: np.ndarray,
                             out_features: int, in_features: int, block_size: int = BS,
                             acc_dtype=np.float32) -> np.ndarray:
    """gather + F.linear (nativebit/inference.py:42-46).  acc_dtype float64 gives the
    'exact' value used to separate the CUDA path's error from the fp32 oracle's own."""
    w = reconstruct_weight(indices, codebook.astype(acc_dtype), (out_features, in_features),
                           block_size, out_features * in_features)
    xf = np.asarray(x, dtype=acc_dtype).reshape(-1, in_features)
    y = xf @ w.T
    return y.reshape(*np.shape(x)[:-1], out_features)


def packed_linear_forward(x: np.ndarray, packed: np.ndarray, codebook: np.ndarray,
                          out_features: int, in_features: int, bits: int = 3,
                          block_size: int = BS, acc_dtype=np.float32) -> np.ndarray:
    """The reference's batched packed-linear path: unpack every call, gather, x @ W.T
    (inference/triton_kernel.py:258-275)."""
    nb = codebook.shape[0]
    idx = unpack_nbits(packed, nb * block_size, bits)
    return inference_linear_forward(x, idx, codebook, out_features, in_features, block_size, acc_dtype)


def fused_matvec_3bit(x: np.ndarray, packed: np.ndarray, codebook: np.ndarray, n: int, k: int) -> np.ndarray:
    """Scalar restatement of the reference's only native kernel
    (inference/cuda_kernel.py:38-82): one output row at a time, blocks in order,
    16 groups of 3 bytes per block, 8 indices per group, fp32 accumulate in that order.
    Pure-Python loops: small cases only."""
    bpr = k // BS
    xf = np.asarray(x, np.float32).reshape(-1)
    cb = np.asarray(codebook, np.float32).reshape(-1, NE)
    pk = np.asarray(packed, np.uint8).reshape(-1)
    y = np.zeros(n, np.float32)
    for row in range(n):
        acc = np.float32(0.0)
        for kb in range(bpr):
            block = row * bpr + kb
            for g in range(16):
                o = block * 48 + g * 3
                bits24 = int(pk[o]) | (int(pk[o + 1]) << 8) | (int(pk[o + 2]) << 16)
                for j in range(8):
                    acc = np.float32(acc + cb[block, (bits24 >> (3 * j)) & 7] * xf[kb * BS + g * 8 + j])
        y[row] = acc
    return y


# --------------------------------------------------------------------------- synthetic inputs
def make_codebook(num_blocks: int, n_entries: int, seed: int, block_size: int = BS) -> np.ndarray:
    """Synthetic per-block codebook with the value distribution the benchmark configs name:
    evenly spaced quantiles (0..1, n_entries points; the percentile initialiser of
    nativebit/codebook_utils.py:6-22) of block_size N(0,1) draws, times a per-block
    scale ~U(0.01, 0.05), stored as fp16.  Sorted ascending by construction."""
    rng = np.random.default_rng(seed)
    z = rng.standard_normal((num_blocks, block_size)).astype(np.float32)
    q = np.quantile(z, np.linspace(0.0, 1.0, n_entries), axis=1).T.astype(np.float32)
    scale = rng.uniform(0.01, 0.05, size=(num_blocks, 1)).astype(np.float32)
    return np.ascontiguousarray((q * scale).astype(np.float16))


def make_packed_linear(out_features: int, in_features: int, bits: int, seed: int, block_size: int = BS):
    """(packed uint8 bytes, fp16 codebook (nb, 2**bits), uint8 indices (nb, block_size))."""
    assert (out_features * in_features) % block_size == 0
    nb = out_features * in_features // block_size
    rng = np.random.default_rng(seed + 7919)
    idx = rng.integers(0, 1 << bits, size=(nb, block_size), dtype=np.uint8)
    cb = make_codebook(nb, 1 << bits, seed, block_size)
    return pack_nbits(idx.reshape(-1), bits), cb, idx


def make_activation(m: int, k: int, seed: int) -> np.ndarray:
    """N(0,1) activations as fp32 values that are exactly representable in bf16."""
    rng = np.random.default_rng(seed + 104729)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return round_to_bf16(x)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 -> fp32, in integer arithmetic."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return (((u + r) >> 16) << 16).astype(np.uint32).view(np.float32).reshape(np.shape(x))


def algorithmic_bytes(m: int, n: int, k: int, bits: int, block_size: int = BS,
                      cb_bytes: int = 2, act_bytes: int = 2) -> int:
    """Compulsory traffic of one packed matvec/GEMM: packed indices + codebooks + x + y."""
    return n * k * bits // 8 + (n * k // block_size) * (1 << bits) * cb_bytes + m * k * act_bytes + m * n * act_bytes


# --------------------------------------------------------------------------- timed CPU baseline
def torch_reference_forward(x_t, packed_t, codebook_t, out_features: int, in_features: int):
    """The reference's CPU PyTorch path restated op for op with CPU torch tensors
    (unpack to int64, advanced-index gather, x @ W.T — inference/triton_kernel.py:258-275).
    Used only as the timed CPU baseline; numerically equal to packed_linear_forward."""
    import torch

    n_groups = packed_t.shape[0] // 3
    p = packed_t.reshape(n_groups, 3).to(torch.int32)
    bits24 = p[:, 0] | (p[:, 1] << 8) | (p[:, 2] << 16)
    indices = torch.zeros(n_groups, 8, dtype=torch.int64)
    for j in range(8):
        indices[:, j] = (bits24 >> (j * 3)) & 0x7
    nb = codebook_t.shape[0]
    indices = indices.reshape(-1)[: nb * BS].reshape(nb, BS)
    block_idx = torch.arange(nb).unsqueeze(1)
    w = codebook_t[block_idx, indices].reshape(-1)[: out_features * in_features]
    w = w.reshape(out_features, in_features)
    return x_t.reshape(-1, in_features) @ w.T


def torch_gather_forward(x_t, indices_t, codebook_t, out_features: int, in_features: int):
    """nativebit/inference.py:42-46 with pre-unpacked int64 indices (gather + F.linear)."""
    import torch
    import torch.nn.functional as F

    nb = codebook_t.shape[0]
    block_idx = torch.arange(nb).unsqueeze(1)
    w = codebook_t[block_idx, indices_t].reshape(-1)[: out_features * in_features]
    return F.linear(x_t, w.view(out_features, in_features))

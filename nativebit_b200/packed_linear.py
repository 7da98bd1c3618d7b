"""Packed linear module and free functions with the reference's names and argument meaning.

Mirrors inference/triton_kernel.py (BS/NE/TILE_N :18-20, dequant_matvec :119-140,
dequant_matvec_3bit :186-196, pack_indices_to_3bit :199-220, PackedLinear :223-286) and
inference/cuda_kernel.py (dequant_matvec_3bit_cuda :133-136).  Differences, all deliberate:
every batch size runs a fused kernel (the reference re-materialises the whole weight for
M > 1), errors are raised instead of being swallowed into a second backend, launches go to
torch's current stream, and 2-bit (K=4) codebooks are accepted as well as 3-bit.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops

BS = 128      # weights per codebook block
NE = 8        # codebook entries per block at 3 bits
TILE_N = 32   # kept for signature compatibility; the B200 kernels pick their own tiling
GEMV_MAX_M = 16
FUSED_MAX_ROWS = 1024   # up to this many activation rows the weights are dequantised inside the GEMM kernel


def pack_indices_to_3bit(indices_uint8: torch.Tensor) -> torch.Tensor:
    """uint8 indices (0..7) -> flat 3-bit packed bytes, on the GPU (inference/triton_kernel.py:199-220)."""
    return ops.pack(indices_uint8.contiguous().reshape(-1), 3)


def dequant_matvec_3bit(x, packed_indices, codebook, N, K, tile_n=TILE_N):
    """y (N,) fp32 = W @ x for one activation vector, 3-bit packed indices
    (inference/triton_kernel.py:186-196)."""
    # the caller may have produced packed_indices on this stream a moment ago (dequant_matvec packs per
    # call): the launch is fully stream-ordered
    y = ops.gemv(x.reshape(1, int(K)).contiguous(), packed_indices, codebook.contiguous(), 3, BS, int(N), int(K),
                 out_dtype=torch.float32, ordered=True)
    return y.reshape(int(N))


def dequant_matvec_3bit_cuda(x, packed, codebook, N, K):
    """Same contract as inference/cuda_kernel.py:133-136."""
    return dequant_matvec_3bit(x, packed.view(-1), codebook, N, K)


def dequant_matvec(x, indices, codebook, N, K, tile_n=TILE_N):
    """y (N,) fp32 = W @ x with unpacked uint8 indices of shape (num_blocks, BS)
    (inference/triton_kernel.py:119-140).  The indices are packed on the device first."""
    packed = ops.pack(indices.contiguous().reshape(-1), 3)
    return dequant_matvec_3bit(x, packed, codebook, N, K)


class PackedLinear(torch.nn.Module):
    """Drop-in for nn.Linear over NativeBit packed weights (inference/triton_kernel.py:223-286).

    Buffers keep the reference's names: `packed_indices` (flat uint8 in the nativebit/pack.py
    layout) and `codebook` ((num_blocks, 2**bits), fp16 or fp32).  forward accepts any leading
    dims; the result has x's dtype.
    """

    def __init__(self, packed_indices, codebook, out_features, in_features, bits: int = 3, block_size: int = BS):
        super().__init__()
        self.register_buffer("packed_indices", packed_indices)
        self.register_buffer("codebook", codebook)
        self.out_features = int(out_features)
        self.in_features = int(in_features)
        self.bits = int(bits)
        self.block_size = int(block_size)
        # The buffers may have been written by kernels still in flight (from_packed / pack_linear pack on
        # the device): the first fused launch is fully stream-ordered, later ones may start early.
        self._fresh = True

    def forward(self, x):
        shape = x.shape
        x_flat = x.reshape(-1, self.in_features)
        if not x_flat.is_contiguous():
            x_flat = x_flat.contiguous()
        m = x_flat.shape[0]
        if self.block_size != BS or self.bits not in (2, 3, 4):
            # shapes outside the fused kernels (small codebook blocks): gather kernel + matmul
            w = ops.dequant(self.packed_indices, self.codebook, self.bits, self.block_size,
                            (self.out_features, self.in_features),
                            dtype=x_flat.dtype if x_flat.dtype in (torch.float16, torch.bfloat16) else torch.float32)
            y = x_flat @ w.T
        elif m <= GEMV_MAX_M:
            y = ops.gemv(x_flat, self.packed_indices, self.codebook, self.bits, self.block_size,
                         self.out_features, self.in_features, ordered=self._fresh)
            self._fresh = False
        else:
            y = self._forward_many(x_flat)
        return y.reshape(*shape[:-1], self.out_features)

    def stream_weight(self, row_mode: int = 0):
        """Tile-major copy of the packed weight for the fused tensor-core kernel and the many-matrix / decode-chain
        kernels (built on first use, kept with the module).  row_mode 1: this is a fused [gate | up] matrix and every
        16-row tile holds 8 gate channels and the matching 8 up channels (for a SwiGLU epilogue)."""
        attr = "_wstream" if row_mode == 0 else "_wstream_rm1"
        w = getattr(self, attr, None)
        if w is None:
            from .stream import stream_pack
            w = stream_pack(self.packed_indices, self.codebook, self.bits, self.out_features, self.in_features, row_mode)
            setattr(self, attr, w)
        return w

    def _forward_many(self, x_flat):
        """M > 16 rows on the tcgen05 kernels (exact fp16 weights; bf16 and fp16 activations as given, fp32
        carried as two fp16 terms; fp32 accumulation; result in x's dtype): one pass over the packed weights,
        dequantised inside the kernel, up to FUSED_MAX_ROWS rows; dequantise-once + GEMM beyond."""
        if self.in_features % BS == 0 and self.bits in (2, 3, 4):
            rows = x_flat.shape[0] * (2 if x_flat.dtype == torch.float32 else 1)
            if rows > FUSED_MAX_ROWS:
                # long inputs: dequantising W once into a scratch copy (12 us for 6912 x 2560) and running the plain
                # tensor-core kernel measures faster than dequantising every weight tile once per 256 rows
                return ops.gemm_prefill(x_flat, self.packed_indices, self.codebook, self.bits, self.block_size,
                                        self.out_features, self.in_features, out_dtype=x_flat.dtype)
            return ops.gemm_prefill_fused(x_flat, self.stream_weight(), self.bits, self.out_features, self.in_features,
                                          out_dtype=x_flat.dtype)
        wdt = x_flat.dtype if x_flat.dtype in (torch.float16, torch.bfloat16) else torch.float32
        w = ops.dequant(self.packed_indices, self.codebook, self.bits, self.block_size,
                        (self.out_features, self.in_features), dtype=wdt)
        return x_flat @ w.T

    def dequantized_weight(self, dtype=torch.float32):
        """The dense (out_features, in_features) weight; bit-exact gather of the codebook values."""
        return ops.dequant(self.packed_indices, self.codebook, self.bits, self.block_size,
                           (self.out_features, self.in_features), dtype=dtype)

    @staticmethod
    def from_packed(indices_np, codebook_np, weight_shape, device="cuda", bits: int = 3):
        """From unpacked uint8 numpy indices + codebook as stored in .nbpack.npz
        (inference/triton_kernel.py:277-286): indices are packed on the GPU."""
        indices_uint8 = torch.from_numpy(np.ascontiguousarray(indices_np)).to(device)
        packed = ops.pack(indices_uint8.reshape(-1), bits)
        codebook = torch.from_numpy(np.ascontiguousarray(codebook_np)).to(device)
        return PackedLinear(packed, codebook, weight_shape[0], weight_shape[1], bits=bits)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}"

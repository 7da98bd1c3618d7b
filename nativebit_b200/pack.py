"""Bit-packing and weight reconstruction with the reference's function names
(nativebit/pack.py:21-169), executed by the CUDA kernels on device tensors.

The byte layout is the reference's, unchanged; these functions exist so that code written
against nativebit.pack keeps working on GPU-resident tensors.
"""
from __future__ import annotations

import torch

from . import ops

FORMAT_VERSION = 1


def pack_3bit(indices: torch.Tensor) -> torch.Tensor:
    return ops.pack(indices.to(torch.uint8).reshape(-1).contiguous(), 3)


def unpack_3bit(packed: torch.Tensor, count: int) -> torch.Tensor:
    return ops.unpack(packed.reshape(-1).contiguous(), 3, count)


def pack_4bit(indices: torch.Tensor) -> torch.Tensor:
    return ops.pack(indices.to(torch.uint8).reshape(-1).contiguous(), 4)


def unpack_4bit(packed: torch.Tensor, count: int) -> torch.Tensor:
    return ops.unpack(packed.reshape(-1).contiguous(), 4, count)


def pack_nbits(indices: torch.Tensor, bits: int) -> torch.Tensor:
    if bits not in (2, 3, 4):
        raise RuntimeError(f"{bits}-bit packing is not part of the accelerated path (2, 3 and 4 are)")
    return ops.pack(indices.to(torch.uint8).reshape(-1).contiguous(), bits)


def unpack_nbits(packed: torch.Tensor, count: int, bits: int) -> torch.Tensor:
    if bits not in (2, 3, 4):
        raise RuntimeError(f"{bits}-bit unpacking is not part of the accelerated path (2, 3 and 4 are)")
    return ops.unpack(packed.reshape(-1).contiguous(), bits, count)


def reconstruct_weight(indices: torch.Tensor, codebook: torch.Tensor, shape, block_size: int,
                       total_weights: int) -> torch.Tensor:
    """Gather from unpacked indices (nativebit/pack.py:145-169).  The indices are packed on the
    device and dequantised by the same kernel that serves packed weights."""
    n_entries = codebook.shape[1]
    bits = max(1, (n_entries - 1).bit_length())
    if bits not in (2, 3, 4):
        raise RuntimeError(f"codebooks of {n_entries} entries are not supported")
    if total_weights != int(shape[0]) * int(shape[1]):
        raise RuntimeError("total_weights must equal shape[0]*shape[1]")
    packed = ops.pack(indices.to(torch.uint8).reshape(-1).contiguous(), bits)
    return ops.dequant(packed, codebook.contiguous(), bits, block_size, shape, dtype=codebook.dtype)

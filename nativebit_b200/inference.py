"""Gather-only inference linear with the reference's constructor (nativebit/inference.py:15-46),
running the fused packed kernels instead of gather + F.linear."""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .packed_linear import PackedLinear


class NativeBitInferenceLinear(nn.Module):
    """Same constructor as the reference: unpacked (num_blocks, block_size) indices and a
    (num_blocks, n_entries) codebook.  The indices are packed once on the device."""

    def __init__(self, in_features: int, out_features: int, codebook: torch.Tensor, indices: torch.Tensor,
                 block_size: int, bias: torch.Tensor = None):
        super().__init__()
        self.in_features, self.out_features, self.block_size = in_features, out_features, block_size
        bits = max(1, (codebook.shape[1] - 1).bit_length())
        packed = ops.pack(indices.to(torch.uint8).reshape(-1).contiguous(), bits)
        self.linear = PackedLinear(packed, codebook.contiguous(), out_features, in_features, bits=bits,
                                   block_size=block_size)
        self.bias = nn.Parameter(bias) if bias is not None else None
        self.total_weights = out_features * in_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.linear(x)
        return y if self.bias is None else y + self.bias.to(y.dtype)

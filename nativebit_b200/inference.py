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


def convert_to_inference(model: nn.Module) -> nn.Module:
    """Replace every trainable NativeBit linear of a model by a NativeBitInferenceLinear
    (nativebit/inference.py:49-85).  A module qualifies by its attributes (latent `weight`, per-block
    `codebook`, `block_size`, `in_features`, `out_features`), so the reference's NativeBitLinear is
    accepted without importing it.  The nearest-entry search runs once, on the device."""
    targets = [(name, m) for name, m in model.named_modules()
               if not isinstance(m, (NativeBitInferenceLinear, PackedLinear))
               and all(hasattr(m, a) for a in ("weight", "codebook", "block_size", "in_features", "out_features"))
               and getattr(m.codebook, "dim", lambda: 0)() == 2]
    for name, m in targets:
        w, cb = m.weight.data, m.codebook.data
        if not w.is_cuda:
            raise RuntimeError("convert_to_inference needs the model on a CUDA device")
        idx = ops.quantize(w.contiguous().float(), cb.contiguous().float(), int(m.block_size))
        fast = NativeBitInferenceLinear(m.in_features, m.out_features, cb.clone(), idx.reshape(cb.shape[0], int(m.block_size)),
                                        int(m.block_size), bias=m.bias.data.clone() if getattr(m, "bias", None) is not None else None)
        parent = model
        parts = name.split(".")
        for part in parts[:-1]:
            parent = getattr(parent, part)
        setattr(parent, parts[-1], fast)
    model.requires_grad_(False)
    return model

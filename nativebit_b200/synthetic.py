"""Seeded synthetic packed weights generated on the device (no checkpoint or dataset is needed).

Value distributions follow the benchmark configuration: uniform indices in [0, 2**bits), a
per-block codebook made of evenly spaced quantiles of block_size N(0,1) draws (the reference's
percentile initialiser, nativebit/codebook_utils.py:6-22) times a per-block scale ~U(0.01, 0.05),
stored as fp16; activations ~N(0,1) in bf16.
"""
from __future__ import annotations

import torch

from . import ops


def synthetic_codebook(num_blocks: int, n_entries: int, gen: torch.Generator, device, block_size: int = 128):
    z, _ = torch.randn(num_blocks, block_size, device=device, generator=gen).sort(dim=1)
    pos = torch.linspace(0, 1, n_entries, device=device) * (block_size - 1)
    lo = pos.floor().long()
    hi = pos.ceil().long()
    frac = (pos - lo).unsqueeze(0)
    q = z[:, lo] * (1 - frac) + z[:, hi] * frac
    scale = torch.empty(num_blocks, 1, device=device).uniform_(0.01, 0.05, generator=gen)
    return (q * scale).half().contiguous()


def synthetic_packed(out_features: int, in_features: int, bits: int, seed: int, device, block_size: int = 128):
    """(packed uint8 bytes in the nativebit/pack.py layout, fp16 codebook (num_blocks, 2**bits))."""
    total = out_features * in_features
    assert total % block_size == 0
    gen = torch.Generator(device=device).manual_seed(seed)
    idx = torch.randint(0, 1 << bits, (total,), dtype=torch.uint8, device=device, generator=gen)
    packed = ops.pack(idx, bits)
    cb = synthetic_codebook(total // block_size, 1 << bits, gen, device, block_size)
    return packed, cb


def synthetic_activation(m: int, k: int, seed: int, device, dtype=torch.bfloat16):
    gen = torch.Generator(device=device).manual_seed(seed + 104729)
    return torch.randn(m, k, device=device, generator=gen).to(dtype)

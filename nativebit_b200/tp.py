"""Tensor-parallel partitioning of packed linears (Megatron style): q/k/v/gate/up are split by
output rows, out_proj/down by input columns in whole codebook blocks, one all-reduce after each
row-sharded projection.  Pure index arithmetic on packed bytes; no arithmetic on weights."""
from __future__ import annotations

import torch


def split_even(n_items: int, world: int) -> list[int]:
    """Sizes of `world` contiguous shares of n_items, larger shares first (e.g. 54 -> 14,14,13,13)."""
    base, rem = divmod(n_items, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def share(n_items: int, world: int, rank: int) -> tuple[int, int]:
    """(start, size) of `rank`'s share."""
    sizes = split_even(n_items, world)
    return sum(sizes[:rank]), sizes[rank]


def block_bytes(bits: int, block_size: int = 128) -> int:
    assert (block_size * bits) % 8 == 0
    return block_size * bits // 8


def slice_rows(packed: torch.Tensor, codebook: torch.Tensor, out_features: int, in_features: int, bits: int,
               row_start: int, n_rows: int, block_size: int = 128):
    """Column-parallel shard: rows [row_start, row_start + n_rows) of a packed (out, in) weight.
    A row is in_features/block_size whole blocks, so the shard is a contiguous byte range."""
    bpr = in_features // block_size
    bb = block_bytes(bits, block_size)
    p = packed.reshape(out_features, bpr * bb)[row_start:row_start + n_rows].reshape(-1).contiguous()
    c = codebook.reshape(out_features, bpr, -1)[row_start:row_start + n_rows].reshape(n_rows * bpr, -1).contiguous()
    return p, c


def slice_cols(packed: torch.Tensor, codebook: torch.Tensor, out_features: int, in_features: int, bits: int,
               block_start: int, n_blocks: int, block_size: int = 128):
    """Row-parallel shard: input columns [block_start*block_size, (block_start+n_blocks)*block_size)
    of every row, i.e. n_blocks whole codebook blocks per row, re-laid out row-major."""
    bpr = in_features // block_size
    bb = block_bytes(bits, block_size)
    p = packed.reshape(out_features, bpr, bb)[:, block_start:block_start + n_blocks].reshape(-1).contiguous()
    c = codebook.reshape(out_features, bpr, -1)[:, block_start:block_start + n_blocks]
    return p, c.reshape(out_features * n_blocks, -1).contiguous()


def ffn_shard_plan(ffn_hidden: int, world: int, rank: int, block_size: int = 128) -> tuple[int, int]:
    """(first hidden channel, number of hidden channels) of `rank`: whole codebook blocks of the
    down projection's input, so gate/up rows and down columns use the same channel range."""
    start_b, n_b = share(ffn_hidden // block_size, world, rank)
    return start_b * block_size, n_b * block_size

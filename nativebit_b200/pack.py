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


def _compute_indices(weight: torch.Tensor, codebook: torch.Tensor, block_size: int, total_weights: int,
                     active_mask=None) -> torch.Tensor:
    """Quantisation indices of a weight on the device (nativebit/pack.py:176-199).  active_mask is not
    supported by the kernel."""
    if active_mask is not None:
        raise RuntimeError("active_mask is not supported by the device quantiser")
    if total_weights != weight.numel():
        raise RuntimeError("total_weights must equal weight.numel()")
    return ops.quantize(weight.contiguous().float(), codebook.contiguous(), block_size)


def pack_linear(weight: torch.Tensor, codebook: torch.Tensor, block_size: int = 128):
    """Dense (out, in) weight + (num_blocks, n_entries) codebook -> PackedLinear with an fp16 codebook: the
    per-layer work of the reference's export_packed (nativebit/pack.py:238-253: indices, bit-pack, codebook.half())."""
    from .packed_linear import PackedLinear
    bits = max(1, (codebook.shape[1] - 1).bit_length())
    if bits not in (2, 3, 4):
        raise RuntimeError(f"codebooks of {codebook.shape[1]} entries are not supported")
    idx = _compute_indices(weight, codebook, block_size, weight.numel())
    return PackedLinear(ops.pack(idx, bits), codebook.half().contiguous(), weight.shape[0], weight.shape[1], bits=bits,
                        block_size=block_size)


def load_packed_layers(path: str, device="cuda"):
    """Read a torch .nbpack file written by the reference's export_packed (schema nativebit/pack.py:256-291:
    format_version, config, bits, n_entries, quantized_layers[name] = {packed_indices, codebook (fp16), shape,
    block_size, n_entries, num_blocks, total_weights[, bias]}, float_params) straight into device-resident packed
    linears: the bytes and fp16 codebooks are uploaded as stored, nothing is unpacked or materialised (the reference's
    load_packed reconstructs dense fp32 nn.Linear weights instead, nativebit/pack.py:343-415).

    Returns (config dict, {layer name: PackedLinear}, {layer name: bias tensor}, {param name: fp16 tensor})."""
    from .packed_linear import PackedLinear
    blob = torch.load(path, map_location="cpu", weights_only=False)
    if blob.get("format_version") != FORMAT_VERSION:
        raise RuntimeError(f"unsupported .nbpack format_version {blob.get('format_version')!r}")
    bits = int(blob["bits"])
    if bits not in (2, 3, 4):
        raise RuntimeError(f"{bits}-bit checkpoints are not supported (2, 3 and 4 are)")
    dev = torch.device(device)
    layers, biases = {}, {}
    for name, d in blob["quantized_layers"].items():
        out_f, in_f = (int(v) for v in d["shape"])
        if int(d["total_weights"]) != out_f * in_f:
            raise RuntimeError(f"{name}: total_weights does not match its shape")
        layers[name] = PackedLinear(d["packed_indices"].contiguous().to(dev), d["codebook"].contiguous().to(dev), out_f, in_f,
                                    bits=bits, block_size=int(d["block_size"]))
        if "bias" in d:
            biases[name] = d["bias"].to(dev)
    floats = {k: v.to(dev) for k, v in blob["float_params"].items()}
    return dict(blob["config"]), layers, biases, floats

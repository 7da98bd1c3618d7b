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


# ---------------------------------------------------------------------------------------------------
# Whole-checkpoint export / load / verify with the reference's names (nativebit/pack.py:202,343,422)
# ---------------------------------------------------------------------------------------------------

def _checkpoint_layers(sd: dict):
    """Names of the quantised linears of a training state dict: every module that owns a 2-D `weight`
    and a 2-D `codebook` (the reference finds them by module type, nativebit/pack.py:222-225, 267-269)."""
    names = [k[:-len(".codebook")] for k, v in sd.items() if k.endswith(".codebook") and v.dim() == 2]
    return [n for n in names if n + ".weight" in sd and sd[n + ".weight"].dim() == 2]


def _read_checkpoint(ckpt_path: str):
    ckpt = torch.load(ckpt_path, map_location="cpu", weights_only=False)
    sd = {k.replace("_orig_mod.", ""): v for k, v in ckpt["model_state_dict"].items()}   # nativebit/generate.py:89-90
    names = _checkpoint_layers(sd)
    if not names:
        raise ValueError("No NativeBitLinear layers found — this is a float model, nothing to pack")
    return ckpt.get("config", {}), sd, names


def _full_config(cfg: dict, sd: dict, names) -> dict:
    """The eight keys the reference writes (nativebit/pack.py:232-245), read off the tensors; the head count
    is not recoverable from shapes and comes from the checkpoint's config (default 4, nativebit/generate.py:112)."""
    first = names[0]
    n_entries = sd[first + ".codebook"].shape[1]
    block_size = -(-sd[first + ".weight"].numel() // sd[first + ".codebook"].shape[0])
    return {
        "vocab_size": sd["tok_emb.weight"].shape[0],
        "n_embd": sd["tok_emb.weight"].shape[1],
        "n_layers": len([k for k in sd if k.startswith("blocks.") and k.endswith(".attn.qkv.weight")]),
        "n_head": int(cfg.get("n_head", 4)),
        "ffn_hidden": sd["blocks.0.ffn.w_gate.weight"].shape[0],
        "context_len": int(cfg.get("context_len", 512)),
        "block_size": int(cfg.get("block_size") or block_size),
        "n_codebook": n_entries,
    }


def export_packed(ckpt_path: str, output_path: str, device: str = "cuda") -> dict:
    """Training checkpoint ({"model_state_dict", "config"}) -> .nbpack file in the reference's schema, with
    the nearest-entry search and the bit-packing done by the device kernels (nativebit/pack.py:202-340).
    The file is byte-for-byte what the reference's exporter stores for the same checkpoint: same keys, same
    index bytes, fp16 codebooks and fp16 float parameters.  Returns the reference's statistics dict."""
    import math
    from pathlib import Path
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("export_packed quantises and packs on the GPU: pass a CUDA device")
    cfg, sd, names = _read_checkpoint(ckpt_path)
    config = _full_config(cfg, sd, names)
    n_entries = config["n_codebook"]
    bits = math.ceil(math.log2(n_entries))
    state = {"format_version": FORMAT_VERSION, "config": config, "bits": bits, "n_entries": n_entries,
             "quantized_layers": {}, "float_params": {}}
    q_bytes = cb_bytes = f_bytes = 0
    for name in names:
        w, cb = sd[name + ".weight"], sd[name + ".codebook"]
        block_size = config["block_size"]
        if cb.shape[0] != -(-w.numel() // block_size):
            raise RuntimeError(f"{name}: {cb.shape[0]} codebook blocks do not cover {w.numel()} weights at block size {block_size}")
        idx = _compute_indices(w.to(dev), cb.to(dev).float(), block_size, w.numel())
        packed = pack_nbits(idx, bits).cpu()
        layer = {"packed_indices": packed, "codebook": cb.half(), "shape": (w.shape[0], w.shape[1]), "block_size": block_size,
                 "n_entries": n_entries, "num_blocks": cb.shape[0], "total_weights": w.numel()}
        if name + ".bias" in sd:
            layer["bias"] = sd[name + ".bias"].half()
        state["quantized_layers"][name] = layer
        q_bytes += packed.numel()
        cb_bytes += cb.numel() * 2
    owned = tuple(n + "." for n in names)
    seen = set()
    for key, v in sd.items():
        # parameters only, each once: buffers (utilisation counters), the tied lm_head and the other names of the
        # token table (value embeddings share it) stay out, as with named_parameters (nativebit/pack.py:300-311)
        if key.startswith(owned) or key == "lm_head.weight" or not v.is_floating_point() or v.data_ptr() in seen:
            continue
        seen.add(v.data_ptr())
        state["float_params"][key] = v.half()
        f_bytes += v.numel() * 2
    out = Path(output_path)
    out.parent.mkdir(parents=True, exist_ok=True)
    torch.save(state, out)
    size, orig = out.stat().st_size, Path(ckpt_path).stat().st_size
    return {"packed_indices_bytes": q_bytes, "codebook_bytes": cb_bytes, "float_param_bytes": f_bytes, "file_size_bytes": size,
            "original_size_bytes": orig, "compression_ratio": orig / size, "bits": bits,
            "n_quantized_layers": len(state["quantized_layers"])}


def load_packed(path: str, device: str = "cuda"):
    """.nbpack file -> decoder ready for inference (nativebit/pack.py:343-415).  Where the reference rebuilds
    dense fp32 nn.Linear weights, this keeps every quantised layer packed on the device: model(idx) -> logits
    runs the fused dequant kernels."""
    from .gpt import NativeBitGPT
    config, layers, biases, floats = load_packed_layers(path, device)
    return NativeBitGPT(config, layers, floats, biases)


def verify_packed(ckpt_path: str, packed_path: str, device: str = "cuda") -> dict:
    """Logits of the packed file against the checkpoint it came from (nativebit/pack.py:422-459): same
    seeded 32-token input, same 0.1 gate.  The checkpoint side is the training forward restated: each linear
    uses codebook[argmin] of its latent weight with the fp32 codebook (nativebit/layers.py:77-104)."""
    from .gpt import NativeBitGPT
    dev = torch.device(device)
    cfg, sd, names = _read_checkpoint(ckpt_path)
    config = _full_config(cfg, sd, names)
    dense = {}
    for name in names:
        w, cb = sd[name + ".weight"].to(dev).float(), sd[name + ".codebook"].to(dev).float()
        idx = _compute_indices(w, cb, config["block_size"], w.numel())
        dense[name] = reconstruct_weight(idx, cb, tuple(w.shape), config["block_size"], w.numel())
    owned = tuple(n + "." for n in names)
    floats = {k: v.to(dev) for k, v in sd.items() if not k.startswith(owned) and v.is_floating_point() and k != "lm_head.weight"}
    biases = {n: sd[n + ".bias"].to(dev) for n in names if n + ".bias" in sd}
    orig = NativeBitGPT(config, dense, floats, biases)
    packed = load_packed(packed_path, device)
    gen = torch.Generator().manual_seed(42)
    test_input = torch.randint(0, config["vocab_size"], (1, min(32, config["context_len"])), generator=gen).to(dev)
    diff = (orig(test_input).float() - packed(test_input).float()).abs()
    max_diff, mean_diff = diff.max().item(), diff.mean().item()
    return {"max_diff": max_diff, "mean_diff": mean_diff, "passed": max_diff < 0.1}

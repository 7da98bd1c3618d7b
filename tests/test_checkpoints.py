"""Loaders for the reference's two packed checkpoint formats, on files written by the reference's own
exporters (tests/golden/make_golden_checkpoints.py).  CPU part: structure and bytes; GPU part: logits
of the loaded decoder against what the reference's own loader + PackedGPT computed, and bit-exact
dequantisation of every layer of the torch-format files."""
import os

import numpy as np
import pytest
import torch

from oracle import nb_oracle as o

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class _Cfg:
    vocab_size, n_layers, n_embd, n_head, ffn_hidden, context_len = 128, 2, 256, 4, 512, 32


def test_npz_loader_structure_on_cpu():
    from nativebit_b200 import generate as G
    model = G.load_packed_model(os.path.join(GOLD, "tiny.nbpack.npz"), _Cfg, device="cpu")
    assert len(model.blocks) == 2 and model.embedding.shape == (128, 256)
    raw = np.load(os.path.join(GOLD, "tiny.nbpack.npz"))
    blk = model.blocks[0]
    assert blk.qkv.out_features == 768 and blk.qkv.in_features == 256
    assert blk.gate_up.out_features == 1024 and blk.down.in_features == 512
    # the packed bytes are the file's bytes, untouched
    key = "params.block_0.CausalSelfAttention_0.NativeBitDense_1"
    assert np.array_equal(blk.out_proj.packed_indices.numpy(), raw[f"idx.{key}"])
    assert blk.out_proj.codebook.dtype == torch.float32          # .nbpack.npz stores fp32 codebooks
    # and decode to the indices the reference's quantiser produced
    idx = o.unpack_3bit(raw[f"idx.{key}"], 256 * 256).reshape(tuple(raw[f"idxshape.{key}"]))
    w = o.reconstruct_weight(idx.reshape(-1), raw[f"cb.{key}"], (256, 256), 128, 256 * 256)
    assert w.shape == (256, 256)
    assert not torch.equal(blk.ln1, torch.ones(256))             # norm weights were read from the file


@pytest.mark.parametrize("name,bs", [("tiny.nbpack", 128), ("tiny_bs8.nbpack", 8)])
def test_torch_nbpack_loader_structure_on_cpu(name, bs):
    from nativebit_b200.pack import load_packed_layers
    cfg, layers, biases, floats = load_packed_layers(os.path.join(GOLD, name), device="cpu")
    assert cfg["block_size"] == bs and cfg["n_codebook"] == 8 and len(layers) == 10
    lin = layers["blocks.0.attn.qkv"]
    assert lin.bits == 3 and lin.block_size == bs and lin.codebook.dtype == torch.float16
    n_w = lin.out_features * lin.in_features
    assert lin.packed_indices.numel() == 3 * ((n_w + 7) // 8)
    assert "tok_emb.weight" in floats and floats["tok_emb.weight"].dtype == torch.float16


@pytest.mark.gpu
def test_npz_checkpoint_decodes_like_the_reference(built_lib):
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    exp = np.load(os.path.join(GOLD, "tiny_nbpack_npz_expected.npz"))
    model = G.load_packed_model(os.path.join(GOLD, "tiny.nbpack.npz"), _Cfg, device=dev)
    caches = G.init_kv_cache(model, 1, dev)
    logits, caches = model(torch.from_numpy(exp["prompt"]).to(dev), kv_caches=caches)
    ref = exp["logits"]
    assert np.abs(logits[0].cpu().numpy() - ref).max() <= 2e-3 * np.abs(ref).max()
    logits2, caches = model(torch.from_numpy(exp["more"]).to(dev), kv_caches=caches)
    assert np.abs(logits2[0].cpu().numpy() - exp["logits2"]).max() <= 2e-3 * np.abs(ref).max()
    assert (logits[0].argmax(-1).cpu().numpy() == ref.argmax(-1)).all()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny.nbpack", "tiny_bs8.nbpack"])
def test_torch_nbpack_layers_bit_exact_and_forward(built_lib, name):
    from nativebit_b200.pack import load_packed_layers
    dev = torch.device("cuda:0")
    cfg, layers, biases, floats = load_packed_layers(os.path.join(GOLD, name), device=dev)
    blob = torch.load(os.path.join(GOLD, name), map_location="cpu", weights_only=False)
    for lname, lin in layers.items():
        d = blob["quantized_layers"][lname]
        n, k = lin.out_features, lin.in_features
        idx = o.unpack_3bit(d["packed_indices"].numpy(), d["num_blocks"] * d["block_size"])
        ref = o.reconstruct_weight(idx, d["codebook"].float().numpy(), (n, k), d["block_size"], n * k)
        assert np.array_equal(lin.dequantized_weight().cpu().numpy(), ref), lname
        x = o.make_activation(3, k, seed=1)
        y = lin(torch.from_numpy(x).to(dev)).double().cpu().numpy()
        yr = x.astype(np.float64) @ ref.T.astype(np.float64)
        assert np.abs(y - yr).max() <= 2e-5 * max(np.abs(yr).max(), 1e-6), lname

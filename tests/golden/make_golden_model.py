"""Golden logits of a tiny packed decoder from the reference's own PackedGPT class.

    python tests/golden/make_golden_model.py /path/to/reference

The reference model (inference/generate_torch.py:135) is built with plain nn.Linear layers that
hold the dense weights reconstructed by the reference's reconstruct_weight from seeded packed
indices and fp16 codebooks — the reference's own materialise recipe (inference/compare.py:260-288).
Stored: the packed weights, the embedding, a prompt, and fp32 logits of the prompt pass and of
four cached decode steps fed with fixed tokens.
"""
import os
import sys

import numpy as np
import torch


def main(ref_root):
    sys.path.insert(0, ref_root)
    from inference.generate_torch import PackedGPT, init_kv_cache
    from nativebit.pack import pack_3bit, unpack_3bit, reconstruct_weight
    from nativebit.codebook_utils import init_codebook_percentile

    V, L, C, H, Fh, ctx = 128, 2, 256, 4, 512, 32
    g = torch.Generator().manual_seed(0)
    out = {"cfg": np.array([V, L, C, H, Fh, ctx])}
    model = PackedGPT(V, L, C, H, Fh, ctx, lambda o, i: torch.nn.Linear(i if i != 3 * C else C, o, bias=False))
    emb = (torch.randn(V, C, generator=g) * 0.02).bfloat16().float()
    model.embedding.weight.data = emb
    out["embedding"] = emb.numpy()

    def make(name, n, k):
        nb = n * k // 128
        z = torch.randn(nb, 128, generator=g)
        # larger scale than the benchmark's so that a 2-layer model produces logits with structure
        cb = (torch.stack([init_codebook_percentile(z[b], 8) for b in range(nb)]) *
              torch.empty(nb, 1).uniform_(0.05, 0.25, generator=g)).half()
        idx = torch.randint(0, 8, (nb * 128,), dtype=torch.uint8, generator=g)
        packed = pack_3bit(idx)
        w = reconstruct_weight(unpack_3bit(packed, nb * 128), cb.float(), (n, k), 128, n * k)
        out[f"p_{name}"], out[f"c_{name}"], out[f"s_{name}"] = packed.numpy(), cb.numpy(), np.array([n, k])
        return w

    for l, blk in enumerate(model.blocks):
        blk.attn.qkv = torch.nn.Linear(C, 3 * C, bias=False)
        blk.attn.qkv.weight.data = make(f"qkv{l}", 3 * C, C)
        blk.attn.out_proj = torch.nn.Linear(C, C, bias=False)
        blk.attn.out_proj.weight.data = make(f"out{l}", C, C)
        blk.ffn.gate.weight.data = make(f"gate{l}", Fh, C)
        blk.ffn.up.weight.data = make(f"up{l}", Fh, C)
        blk.ffn.down.weight.data = make(f"down{l}", C, Fh)
    model.requires_grad_(False)

    prompt = torch.randint(0, V, (1, 8), generator=g)
    forced = torch.randint(0, V, (4,), generator=g)
    caches = init_kv_cache(model, device="cpu")
    logits, caches = model(prompt, kv_caches=caches)
    steps = []
    for t in forced.tolist():
        lg, caches = model(torch.tensor([[t]]), kv_caches=caches)
        steps.append(lg[0, -1].numpy())
    out["prompt"], out["forced"] = prompt.numpy(), forced.numpy()
    out["logits_prompt"] = logits[0].numpy()
    out["logits_steps"] = np.stack(steps)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_model.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes; logits range", float(logits.min()), float(logits.max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} <path of the NativeBit reference checkout>")
    main(sys.argv[1])

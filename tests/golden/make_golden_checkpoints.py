"""Golden packed checkpoints in the reference's two on-disk formats, written by the reference's own
exporters, plus what the reference itself computes from them.

    python tests/golden/make_golden_checkpoints.py /path/to/reference

1. tiny.nbpack.npz  — inference/pack.py:pack_checkpoint on a tiny JAX-style parameter file (keys
   params/block_i/CausalSelfAttention_0/NativeBitDense_{0,1}/{weight,codebook}, .../SwiGLU_0/NativeBitDense_{0,1,2},
   params/embedding, RMSNorm weights); golden logits come from the reference's own
   inference/generate_torch.py:load_packed_model + PackedGPT run on CPU (prompt of 8 tokens, batched path).
2. tiny.nbpack      — nativebit/pack.py:export_packed on a tiny NativeBitGPT training checkpoint
   (block_size 128) and, for the generic path, one with block_size 8 as in the reference's tests; beside each
   the checkpoint it was exported from (*_ckpt.pt) and *_nbpack_expected.npz: logits of the reference's training
   forward and of its load_packed model on one seeded input, verify_packed's max_diff and the exporter's statistics.
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, ref_root)
    from inference.pack import pack_checkpoint
    from inference.generate_torch import load_packed_model, init_kv_cache
    from nativebit.codebook_utils import init_codebook_percentile
    from nativebit.model import NativeBitGPT
    from nativebit.pack import export_packed, load_packed, verify_packed

    # ---------------------------------------------------------------- 1. .nbpack.npz
    V, L, C, H, Fh, ctx = 128, 2, 256, 4, 512, 32
    g = torch.Generator().manual_seed(1)
    ck = {"params/embedding": (torch.randn(V, C, generator=g) * 0.02).numpy()}
    ck["params/ln_f/weight"] = (1 + 0.1 * torch.randn(C, generator=g)).numpy()

    def layer(prefix, n, k):
        nb = n * k // 128
        z = torch.randn(nb, 128, generator=g)
        cb = torch.stack([init_codebook_percentile(z[b], 8) for b in range(nb)]) * torch.empty(nb, 1).uniform_(0.05, 0.25, generator=g)
        cb = cb.half().float()          # fp16-representable, distinct entries
        idx = torch.randint(0, 8, (nb, 128), generator=g)
        w = torch.gather(cb, 1, idx).reshape(n, k)
        ck[f"{prefix}/weight"], ck[f"{prefix}/codebook"] = w.numpy(), cb.numpy()

    for l in range(L):
        b = f"params/block_{l}"
        layer(f"{b}/CausalSelfAttention_0/NativeBitDense_0", 3 * C, C)
        layer(f"{b}/CausalSelfAttention_0/NativeBitDense_1", C, C)
        layer(f"{b}/SwiGLU_0/NativeBitDense_0", Fh, C)
        layer(f"{b}/SwiGLU_0/NativeBitDense_1", Fh, C)
        layer(f"{b}/SwiGLU_0/NativeBitDense_2", C, Fh)
        for j in range(2):
            ck[f"{b}/RMSNorm_{j}/weight"] = (1 + 0.1 * torch.randn(C, generator=g)).numpy()
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "tiny_params.npz")
        np.savez(src, **ck)
        out = os.path.join(HERE, "tiny.nbpack.npz")
        pack_checkpoint(src, out, 128, 8)

    class Cfg:
        vocab_size, n_layers, n_embd, n_head, ffn_hidden, context_len = V, L, C, H, Fh, ctx
    model = load_packed_model(out, Cfg, device="cpu")
    model.requires_grad_(False)
    prompt = torch.randint(0, V, (1, 8), generator=g)
    caches = init_kv_cache(model, device="cpu")
    logits, caches = model(prompt, kv_caches=caches)
    more = torch.randint(0, V, (1, 2), generator=g)          # two more tokens at once: still the batched path
    logits2, caches = model(more, kv_caches=caches)
    np.savez_compressed(os.path.join(HERE, "tiny_nbpack_npz_expected.npz"), cfg=np.array([V, L, C, H, Fh, ctx]),
                        prompt=prompt.numpy(), more=more.numpy(), logits=logits[0].numpy(), logits2=logits2[0].numpy())
    print("npz checkpoint", os.path.getsize(out), "bytes; logits range", float(logits.min()), float(logits.max()))

    # ---------------------------------------------------------------- 2. torch .nbpack
    for tag, (n_embd, ffn, bs) in {"tiny": (128, 256, 128), "tiny_bs8": (32, 64, 8)}.items():
        torch.manual_seed(3)
        m = NativeBitGPT(vocab_size=256, n_layers=2, n_embd=n_embd, n_head=2, ffn_hidden=ffn, context_len=32,
                         block_size=bs, n_entries=8, use_nativebit=True)
        _ = m(torch.randint(0, 256, (1, 16)))
        m.update_all_utilization()
        with tempfile.TemporaryDirectory() as tmp:
            ckp = os.path.join(tmp, "ckpt.pt")
            torch.save({"model_state_dict": m.state_dict(),
                        "config": {"vocab_size": 256, "n_layers": 2, "n_embd": n_embd, "n_head": 2, "ffn_hidden": ffn,
                                   "context_len": 32, "block_size": bs, "n_codebook": 8}}, ckp)
            stats = export_packed(ckp, os.path.join(HERE, f"{tag}.nbpack"))
            # the checkpoint itself (for the device exporter, which must write the same file) and what the
            # reference computes from both sides: the training forward and its load_packed model
            import shutil
            shutil.copy(ckp, os.path.join(HERE, f"{tag}_ckpt.pt"))
            idx = torch.randint(0, 256, (1, 16), generator=torch.Generator().manual_seed(5))
            m.train(False)
            with torch.no_grad():
                lo = m(idx).float()
                lp = load_packed(os.path.join(HERE, f"{tag}.nbpack"), "cpu")(idx).float()
            ver = verify_packed(ckp, os.path.join(HERE, f"{tag}.nbpack"), "cpu")
            np.savez_compressed(os.path.join(HERE, f"{tag}_nbpack_expected.npz"), idx=idx.numpy(), logits_checkpoint=lo.numpy(),
                                logits_packed=lp.numpy(), verify_max_diff=np.float64(ver["max_diff"]),
                                stats=np.array([stats[k] for k in ("packed_indices_bytes", "codebook_bytes", "float_param_bytes",
                                                                   "n_quantized_layers", "bits")]))
        print(tag, ".nbpack", stats["file_size_bytes"], "bytes,", stats["n_quantized_layers"], "layers; verify", ver)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} <path of the NativeBit reference checkout>")
    main(sys.argv[1])

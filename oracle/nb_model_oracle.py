"""CPU oracle of the packed decoder.  TEST INFRASTRUCTURE ONLY (see nb_oracle.py).

Dense fp32 restatement of the reference's PackedGPT forward with a KV cache
(inference/generate_torch.py:29-162): every packed linear is materialised to a dense fp32 matrix
with reconstruct_weight — the reference's own recipe for a dense oracle (inference/compare.py:260-288)
— and the block math is restated with torch CPU ops.  Parity status: PINNED against logits
produced by the reference's PackedGPT class itself (tests/golden/make_golden_model.py).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from . import nb_oracle as o


def rms_norm(x, w, eps=1e-6):
    # inference/generate_torch.py:35-38
    return x.float() / torch.sqrt(x.float().pow(2).mean(-1, keepdim=True) + eps) * w.float()


def rope_tables(head_dim, max_len, theta=10000.0):
    # inference/generate_torch.py:41-45
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    f = torch.outer(torch.arange(max_len, dtype=torch.float32), freqs)
    return torch.cos(f), torch.sin(f)


def apply_rope(x, cos, sin, pos):
    # inference/generate_torch.py:48-60 (interleaved pairs)
    T = x.shape[2]
    c = cos[pos:pos + T].repeat_interleave(2, dim=-1)[None, None]
    s = sin[pos:pos + T].repeat_interleave(2, dim=-1)[None, None]
    x1, x2 = x[..., ::2], x[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).reshape(x.shape)
    return x * c + rot * s


class DenseModel:
    """weights: dict with 'embedding' (V, C) and per layer l: qkv{l} (3C, C), out{l} (C, C), gate{l}, up{l} (F, C),
    down{l} (C, F), ln1_{l}, ln2_{l}, and ln_f — all fp32 torch tensors."""

    def __init__(self, weights: dict, n_layers: int, n_head: int, context_len: int):
        self.w, self.L, self.H, self.ctx = weights, n_layers, n_head, context_len
        C = weights["embedding"].shape[1]
        self.hd = C // n_head
        # the same torch ops run wherever the weights live (CPU here; a GPU for the full-size model,
        # with TF32 off, so that every product is fp32)
        self.dev = weights["embedding"].device
        cos, sin = rope_tables(self.hd, context_len)
        self.cos, self.sin = cos.to(self.dev), sin.to(self.dev)

    def init_cache(self, batch=1):
        z = lambda: torch.zeros(batch, self.H, self.ctx, self.hd, device=self.dev)
        return [[z(), z(), 0] for _ in range(self.L)]

    @torch.no_grad()
    def forward(self, idx: torch.Tensor, caches):
        """idx (B, T) -> logits (B, T, V) fp32; caches updated in place (inference/generate_torch.py:72-106,150-162)."""
        w = self.w
        B, T = idx.shape
        x = w["embedding"][idx].float()
        for l in range(self.L):
            h = rms_norm(x, w[f"ln1_{l}"])
            qkv = h @ w[f"qkv{l}"].T
            q, k, v = qkv.chunk(3, dim=-1)
            q, k, v = (t.reshape(B, T, self.H, self.hd).transpose(1, 2) for t in (q, k, v))
            kb, vb, n = caches[l]
            q, k = apply_rope(q, self.cos, self.sin, n), apply_rope(k, self.cos, self.sin, n)
            kb[:, :, n:n + T] = k
            vb[:, :, n:n + T] = v
            new = n + T
            att = torch.einsum("bhqd,bhkd->bhqk", q * self.hd ** -0.5, kb)
            qp = n + torch.arange(T, device=self.dev)
            kp = torch.arange(self.ctx, device=self.dev)
            mask = (kp[None, :] <= qp[:, None]) & (kp[None, :] < new)
            att = att.masked_fill(~mask[None, None], torch.finfo(att.dtype).min)
            out = torch.einsum("bhqk,bhkd->bhqd", F.softmax(att, dim=-1), vb)
            caches[l][2] = new
            x = x + out.transpose(1, 2).reshape(B, T, -1) @ w[f"out{l}"].T
            h = rms_norm(x, w[f"ln2_{l}"])
            x = x + (F.silu(h @ w[f"gate{l}"].T) * (h @ w[f"up{l}"].T)) @ w[f"down{l}"].T
        x = rms_norm(x, w["ln_f"])
        logits = x.to(w["embedding"].dtype) @ w["embedding"].T
        return 30.0 * torch.tanh(logits.float() / 30.0)


def dense_weights_from_packed(packed_layers: dict, embedding: np.ndarray, n_layers: int, bits: int = 3) -> dict:
    """packed_layers[name] = (packed bytes, fp16/fp32 codebook, (N, K)); names qkv{l}, out{l}, gate{l}, up{l}, down{l}."""
    w = {"embedding": torch.from_numpy(np.asarray(embedding, np.float32))}
    C = embedding.shape[1]
    for name, (packed, cb, (n, k)) in packed_layers.items():
        w[name] = torch.from_numpy(o.dequant_packed(packed, np.asarray(cb, np.float32), n, k, bits))
    for l in range(n_layers):
        w[f"ln1_{l}"] = torch.ones(C)
        w[f"ln2_{l}"] = torch.ones(C)
    w["ln_f"] = torch.ones(C)
    return w

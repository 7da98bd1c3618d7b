"""Inference-only restatement of the reference's training-side decoder (nativebit/model.py:60-230:
RoPE over interleaved pairs, RMSNorm, SwiGLU, token-table value embeddings gated into V on odd layers,
tied LM head, tanh soft-cap at 30), built over packed linears.

This is what the torch-format .nbpack files describe (nativebit/pack.py:343-415 loads them into the
same architecture with dense nn.Linear weights).  Every quantised linear here is a PackedLinear, so the
forward pass runs the fused dequant kernels; the rest is host-side torch glue.  A `dense=True` build
holds fp32 matrices instead and serves as the "original checkpoint" side of verify_packed.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

QUANTIZED = ("attn.qkv", "attn.out_proj", "ffn.w_gate", "ffn.w_up", "ffn.w_down")


def _rms(x, w, eps=1e-6):
    # nativebit/model.py:23-25
    xf = x.float()
    return (xf * xf.pow(2).mean(-1, keepdim=True).add(eps).rsqrt()).type_as(x) * w


def _rope(q, k, cos, sin):
    # nativebit/model.py:39-57: positions 0..T-1, tables tiled (not interleaved) along the head dim
    T = q.shape[2]
    c = cos[:T][None, None].repeat(1, 1, 1, 2)
    s = sin[:T][None, None].repeat(1, 1, 1, 2)

    def rot(x):
        return torch.stack((-x[..., 1::2], x[..., ::2]), dim=-1).flatten(-2)
    return q * c + rot(q) * s, k * c + rot(k) * s


class NativeBitGPT(torch.nn.Module):
    """linears[name] is a PackedLinear (or any callable module) or, for a dense build, an fp32 (out, in)
    matrix; floats holds tok_emb.weight, ln_f.weight, blocks.i.ln{1,2}.weight and, on odd layers,
    blocks.i.attn.ve_gate.weight."""

    def __init__(self, config: dict, linears: dict, floats: dict, biases: dict | None = None):
        super().__init__()
        self.config = dict(config)
        self.context_len = int(config["context_len"])
        self.n_layers, self.n_embd, self.n_head = int(config["n_layers"]), int(config["n_embd"]), int(config["n_head"])
        self.head_dim = self.n_embd // self.n_head
        self.linears = torch.nn.ModuleDict() if all(isinstance(v, torch.nn.Module) for v in linears.values()) else None
        self._lin = {}
        for name, lin in linears.items():
            if self.linears is not None:
                self.linears[name.replace(".", "/")] = lin
            self._lin[name] = lin
        self.floats = {k: v.float() for k, v in floats.items()}
        self.biases = {k: v.float() for k, v in (biases or {}).items()}
        dev = self.floats["tok_emb.weight"].device
        freqs = 1.0 / (10000.0 ** (torch.arange(0, self.head_dim, 2).float() / self.head_dim))
        f = torch.outer(torch.arange(self.context_len).float(), freqs)
        self.rope_cos, self.rope_sin = f.cos().to(dev), f.sin().to(dev)

    def _apply(self, name, x):
        lin = self._lin[name]
        y = lin(x) if isinstance(lin, torch.nn.Module) else F.linear(x, lin)
        b = self.biases.get(name)
        return y if b is None else y + b

    @torch.no_grad()
    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        B, T = idx.shape
        if T > self.context_len:
            raise RuntimeError(f"sequence length {T} > context_len {self.context_len}")
        emb = self.floats["tok_emb.weight"]
        H, hd, C = self.n_head, self.head_dim, self.n_embd
        x = emb[idx]
        for i in range(self.n_layers):
            p = f"blocks.{i}."
            h = _rms(x, self.floats[p + "ln1.weight"])
            q, k, v = self._apply(p + "attn.qkv", h).split(C, dim=-1)
            q, k, v = (t.reshape(B, T, H, hd).transpose(1, 2) for t in (q, k, v))
            if i % 2 == 1:                                     # value embeddings, nativebit/model.py:100-105
                gw = self.floats[p + "attn.ve_gate.weight"]
                ve = emb[idx].reshape(B, T, H, hd).transpose(1, 2)
                gate = 2.0 * torch.sigmoid(F.linear(h[:, :, :gw.shape[1]], gw))
                v = v + gate.transpose(1, 2).unsqueeze(-1) * ve
            q, k = _rope(q, k, self.rope_cos, self.rope_sin)
            att = F.scaled_dot_product_attention(q, k, v.to(q.dtype), is_causal=True)
            x = x + self._apply(p + "attn.out_proj", att.transpose(1, 2).reshape(B, T, C))
            h = _rms(x, self.floats[p + "ln2.weight"])
            x = x + self._apply(p + "ffn.w_down", F.silu(self._apply(p + "ffn.w_gate", h)) * self._apply(p + "ffn.w_up", h))
        x = _rms(x, self.floats["ln_f.weight"])
        logits = F.linear(x, emb)
        return 30.0 * torch.tanh(logits / 30.0)

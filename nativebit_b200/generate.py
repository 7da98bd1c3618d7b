"""Packed LLaMA-style decoder with a static KV cache, built from PackedLinear, tensor-parallel over
1/2/4/8 GPUs.  Mirrors the reference's decode interface (inference/generate_torch.py): PackedGPT
(:135-162: pre-norm blocks, fused qkv chunked [q|k|v] :74-75, interleaved-pair RoPE theta=1e4
:41-60, RMSNorm x/sqrt(mean(x^2)+1e-6)*w :29-38, SwiGLU :109-117, tied LM head with 30*tanh(./30)
soft-cap :157-159), init_kv_cache (:269-277), load_packed_model (:176-266, .nbpack.npz keys) and
benchmark (:280-320, same result keys), plus prefill/step functions shaped like the JAX twin's
(inference/generate.py:163-184).

Differences, all deliberate: packed bytes go straight to the device (no unpack -> repack round
trip); gate and up are one fused packed matrix; the decode step is captured once in a CUDA graph
and replayed with the position and the next token held on the device (the reference syncs with
the host every token); the cache is attended over its valid prefix only in eager mode and under a
position mask in the captured step; ranks of a tensor-parallel group hold row shards of
q/k/v/gate/up and whole-block column shards of out_proj/down and all-reduce after each of the two.
"""
from __future__ import annotations

import math
import re
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from . import ops, synthetic, tp
from .packed_linear import PackedLinear


@dataclass
class ModelConfig:
    """Shape of the packed decoder.  Defaults: the 2.2B benchmark configuration (26 layers, hidden
    2560, 32 heads, SwiGLU 6912, vocab 32000, context 1024, 3-bit block-128 codebooks)."""
    vocab_size: int = 32000
    n_layers: int = 26
    n_embd: int = 2560
    n_head: int = 32
    ffn_hidden: int = 6912
    context_len: int = 1024
    block_size: int = 128
    bits: int = 3
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6
    logit_cap: float = 30.0

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.shape[-1] <= 4096 and weight.dtype == torch.float32:
        out = torch.empty_like(x)                      # one kernel instead of five element-wise launches
        ops.add_rmsnorm(x.view(-1, x.shape[-1]), None, weight, eps, out.view(-1, x.shape[-1]))
        return out
    xf = x.float()
    return xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight


def precompute_rope(head_dim: int, max_len: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(max_len, dtype=torch.float32, device=device)
    f = torch.outer(t, freqs)
    return torch.cos(f).repeat_interleave(2, dim=-1), torch.sin(f).repeat_interleave(2, dim=-1)


def apply_rope(x: torch.Tensor, cos2: torch.Tensor, sin2: torch.Tensor) -> torch.Tensor:
    """x (B, H, T, hd); cos2/sin2 (T, hd) already repeated per pair (interleaved-pair rotation)."""
    x1, x2 = x[..., ::2], x[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).reshape(x.shape)
    return x * cos2 + rot * sin2


class PackedBlock(torch.nn.Module):
    def __init__(self, qkv, out_proj, gate_up, down, ln1, ln2):
        super().__init__()
        self.qkv, self.out_proj, self.gate_up, self.down = qkv, out_proj, gate_up, down
        self.register_buffer("ln1", ln1)
        self.register_buffer("ln2", ln2)


class PackedGPT(torch.nn.Module):
    """Inference-only packed decoder (one tensor-parallel rank's shard)."""

    def __init__(self, config: ModelConfig, embedding: torch.Tensor, blocks: list[PackedBlock], ln_f: torch.Tensor,
                 tp_rank: int = 0, tp_size: int = 1, group=None):
        super().__init__()
        self.config = config
        self.n_layers, self.n_embd, self.n_head, self.context_len = (config.n_layers, config.n_embd, config.n_head,
                                                                     config.context_len)
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        assert config.n_head % tp_size == 0
        self.heads_local = config.n_head // tp_size
        self.register_buffer("embedding", embedding)
        self.blocks = torch.nn.ModuleList(blocks)
        self.register_buffer("ln_f", ln_f)
        cos2, sin2 = precompute_rope(config.head_dim, config.context_len, config.rope_theta, embedding.device)
        self.register_buffer("cos2", cos2)
        self.register_buffer("sin2", sin2)
        # columns of the attention output this rank feeds to out_proj, and the whole codebook blocks covering them
        c0 = self.heads_local * config.head_dim * tp_rank
        c1 = c0 + self.heads_local * config.head_dim
        self.o_col0 = c0 - (c0 // config.block_size) * config.block_size      # offset inside the first block
        self.o_cols = blocks[0].out_proj.in_features if blocks else 0

    # ------------------------------------------------------------------ pieces
    def enable_oneshot_allreduce(self, max_batch: int = 64) -> None:
        """Use the one-shot peer-memory all-reduce (csrc/nb_comm.cu) for decode-sized messages instead of
        NCCL; larger messages (prefill) stay on NCCL."""
        if self.tp_size > 1:
            from .comm import OneShotAllReduce
            self.oneshot = OneShotAllReduce(max_batch * self.n_embd, self.embedding.device, self.group)
            # decode steps of up to 8 sequences also shard the tied LM head by vocabulary rows: every rank multiplies
            # its rows of the table only and the ranks' slices of the logits are put together by one more sum
            # (all other ranks contribute zeros to a slice, so the sum is exact)
            V = self.embedding.shape[0]
            if V % 8 == 0 and self.embedding.dtype == torch.bfloat16:
                self.head_batch = min(8, max_batch)
                self.head_ar = OneShotAllReduce(self.head_batch * V, self.embedding.device, self.group)
                v0, vn = tp.share(V // 8, self.tp_size, self.tp_rank)
                self.head_rows = (8 * v0, 8 * vn)

    def enable_fused_allreduce(self, max_batch: int = 8) -> None:
        """Fold the decode step's all-reduces into the packed GEMVs on both sides of them (nb_gemv_tp):
        the row-sharded projections push their partial results into every rank's exchange buffer and
        the next GEMV sums them while it stages its activations.  Used by DecodeSession for up to 8
        sequences; prefill and larger batches keep the collective."""
        if self.tp_size > 1:
            from .comm import Exchange
            self.exchange = Exchange(max_batch * self.n_embd, self.embedding.device, self.group)

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            ar = getattr(self, "oneshot", None)
            if ar is not None and t.dtype == torch.float32 and t.is_contiguous() and t.numel() <= ar.max_count \
                    and t.numel() % 4 == 0:
                ar(t)
            else:
                torch.distributed.all_reduce(t, group=self.group)
        return t

    def _attn_inputs(self, x, blk, pos0: int | torch.Tensor, T: int):
        B = x.shape[0]
        hd, Hl = self.config.head_dim, self.heads_local
        qkv = blk.qkv(rms_norm(x, blk.ln1, self.config.norm_eps)).float()
        q, k, v = qkv.split(Hl * hd, dim=-1)
        q = q.reshape(B, T, Hl, hd).transpose(1, 2)
        k = k.reshape(B, T, Hl, hd).transpose(1, 2)
        v = v.reshape(B, T, Hl, hd).transpose(1, 2)
        if isinstance(pos0, int):
            cos2, sin2 = self.cos2[pos0:pos0 + T], self.sin2[pos0:pos0 + T]
        else:  # device position (captured decode step, T == 1)
            cos2, sin2 = self.cos2.index_select(0, pos0), self.sin2.index_select(0, pos0)
        return apply_rope(q, cos2, sin2), apply_rope(k, cos2, sin2), v

    @staticmethod
    def _add_norm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float) -> torch.Tensor:
        """x += delta in place (delta may be None); returns RMSNorm(x) * weight: one kernel on the GPU."""
        C = x.shape[-1]
        if (delta is not None and x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and C <= 4096
                and weight.dtype == torch.float32 and delta.dtype == torch.float32 and delta.is_contiguous()):
            out = torch.empty_like(x)
            ops.add_rmsnorm(x.view(-1, C), delta.view(-1, C), weight, eps, out.view(-1, C))
            return out
        if delta is not None:
            x.add_(delta)
        return rms_norm(x, weight, eps)

    def _finish_block(self, x, blk, attn_out):
        """attn_out (B, T, Hl*hd) -> residual adds of out_proj and the SwiGLU FFN."""
        if attn_out.shape[-1] != self.o_cols:  # pad to the whole codebook blocks covering this rank's columns
            padded = attn_out.new_zeros(*attn_out.shape[:-1], self.o_cols)
            padded[..., self.o_col0:self.o_col0 + attn_out.shape[-1]] = attn_out
            attn_out = padded
        x = x + self._all_reduce(blk.out_proj(attn_out).float())
        gu = blk.gate_up(rms_norm(x, blk.ln2, self.config.norm_eps)).float()
        if gu.is_cuda and gu.is_contiguous():
            act = torch.empty(*gu.shape[:-1], gu.shape[-1] // 2, dtype=torch.float32, device=gu.device)
            ops.silu_mul(gu.view(-1, gu.shape[-1]), act.view(-1, act.shape[-1]))
        else:
            gate, up = gu.split(gu.shape[-1] // 2, dim=-1)
            act = F.silu(gate) * up
        return x + self._all_reduce(blk.down(act).float())

    def _head(self, x: torch.Tensor, rows: tuple[int, int] | None = None) -> torch.Tensor:
        """x (..., C) fp32 @ embedding.T with fp32 accumulation and an fp32 result.  A bf16 table is
        multiplied by the activations split into two bf16 terms (16 significant bits) stacked into one
        operand, so the table is read once and neither the activations nor the logits are rounded to 8 bits.
        rows = (first, count): only those rows of the table (a vocabulary shard)."""
        emb = self.embedding if rows is None else self.embedding[rows[0]:rows[0] + rows[1]]
        shape = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).float()
        if emb.dtype != torch.bfloat16:
            return (x2 @ emb.float().T).reshape(*shape, -1)
        hi = x2.bfloat16()
        lo = (x2 - hi.float()).bfloat16()
        y = torch.mm(torch.cat((hi, lo)), emb.T, out_dtype=torch.float32)
        m = x2.shape[0]
        return (y[:m] + y[m:]).reshape(*shape, -1)

    def _logits(self, x):
        logits = self._head(rms_norm(x, self.ln_f, self.config.norm_eps))
        cap = self.config.logit_cap
        return cap * torch.tanh(logits / cap)

    # ------------------------------------------------------------------ eager forward (prefill, tests)
    @torch.no_grad()
    def forward(self, idx: torch.Tensor, kv_caches=None, last_only: bool = False):
        """idx (B, T) int64 -> logits (B, T, V) fp32 [, new caches].  kv_caches: list of
        (k_buf, v_buf, cache_len) as returned by init_kv_cache.  last_only: logits of the last position
        only, (B, 1, V) (what a decode loop needs from its prompt)."""
        B, T = idx.shape
        x = self.embedding[idx].float()
        new_caches = []
        delta = None                                   # a residual update that the next norm kernel will add
        for i, blk in enumerate(self.blocks):
            if kv_caches is not None and x.is_cuda and kv_caches[i][0].shape[0] == B:
                # RoPE, cache write and causal attention in one launch (the rotary tables and the caches are fp32); the
                # residual adds ride in the norm kernels, the last one of a block is still pending when the block ends
                k_buf, v_buf, cache_len = kv_caches[i]
                eps = self.config.norm_eps
                qkv = blk.qkv(self._add_norm(x, delta, blk.ln1, eps)).float().contiguous()
                cols = self.heads_local * self.config.head_dim
                out = (x.new_empty if cols == self.o_cols else x.new_zeros)(B, T, self.o_cols)
                ops.prefill_attention(qkv.view(B * T, -1), T, self.cos2, self.sin2, int(cache_len), k_buf, v_buf,
                                      out.view(B * T, -1), self.o_col0 if cols != self.o_cols else 0)
                new_caches.append((k_buf, v_buf, cache_len + T))
                d1 = self._all_reduce(blk.out_proj(out).float())
                gu = blk.gate_up(self._add_norm(x, d1, blk.ln2, eps)).float().contiguous()
                act = torch.empty(B, T, gu.shape[-1] // 2, dtype=torch.float32, device=gu.device)
                ops.silu_mul(gu.view(B * T, -1), act.view(B * T, -1))
                delta = self._all_reduce(blk.down(act).float())
                continue
            if delta is not None:
                x, delta = x + delta, None
            if kv_caches is not None:
                k_buf, v_buf, cache_len = kv_caches[i]
                q, k, v = self._attn_inputs(x, blk, cache_len, T)
                k_buf[:, :, cache_len:cache_len + T] = k
                v_buf[:, :, cache_len:cache_len + T] = v
                new_len = cache_len + T
                kk, vv = k_buf[:, :, :new_len], v_buf[:, :, :new_len]
                q_pos = cache_len + torch.arange(T, device=x.device)
                mask = torch.arange(new_len, device=x.device)[None, :] <= q_pos[:, None]
                out = F.scaled_dot_product_attention(q, kk, vv, attn_mask=mask[None, None])
                new_caches.append((k_buf, v_buf, new_len))
            else:
                q, k, v = self._attn_inputs(x, blk, 0, T)
                out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = self._finish_block(x, blk, out.transpose(1, 2).reshape(B, T, -1))
        if last_only:
            x = x[:, -1:, :] if delta is None else x[:, -1:, :] + delta[:, -1:, :]
        elif delta is not None:
            x = x + delta
        logits = self._logits(x.contiguous())
        return (logits, new_caches) if kv_caches is not None else logits

    # ------------------------------------------------------------------ construction
    @staticmethod
    def random_init(config: ModelConfig, seed: int = 0, device="cuda", tp_rank: int = 0, tp_size: int = 1, group=None):
        """Seeded random-init model: every rank generates the same global packed weights (per-layer
        seeds seed*1000 + layer*10 + j) and keeps its shard; embedding ~N(0, 0.02) in bf16, norms 1."""
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)
        emb = (torch.randn(config.vocab_size, config.n_embd, device=dev, generator=g) * 0.02).bfloat16()
        C, Fh, bits = config.n_embd, config.ffn_hidden, config.bits
        blocks = []
        for l in range(config.n_layers):
            s = seed * 1000 + l * 10
            full = {"qkv": synthetic.synthetic_packed(3 * C, C, bits, s + 0, dev),
                    "out_proj": synthetic.synthetic_packed(C, C, bits, s + 1, dev),
                    "gate": synthetic.synthetic_packed(Fh, C, bits, s + 2, dev),
                    "up": synthetic.synthetic_packed(Fh, C, bits, s + 3, dev),
                    "down": synthetic.synthetic_packed(C, Fh, bits, s + 4, dev)}
            ones = torch.ones(C, device=dev)
            blocks.append(shard_block(config, full, ones, ones.clone(), tp_rank, tp_size))
            del full
        return PackedGPT(config, emb, blocks, torch.ones(C, device=dev), tp_rank, tp_size, group)


def shard_block(config: ModelConfig, full: dict, ln1, ln2, tp_rank: int, tp_size: int) -> PackedBlock:
    """Global packed (bytes, codebook) pairs of one layer -> this rank's PackedBlock."""
    C, Fh, bits, bs, hd = config.n_embd, config.ffn_hidden, config.bits, config.block_size, config.head_dim
    Hl = config.n_head // tp_size
    rows = Hl * hd
    r0 = tp_rank * rows
    # q, k, v rows of this rank's heads out of the fused [q|k|v] row order
    parts = [tp.slice_rows(*full["qkv"], 3 * C, C, bits, j * C + r0, rows, bs) for j in range(3)]
    qkv = PackedLinear(torch.cat([p for p, _ in parts]), torch.cat([c for _, c in parts]), 3 * rows, C, bits, bs)
    # out_proj: the whole codebook blocks that cover columns [r0, r0 + rows)
    b0, b1 = r0 // bs, (r0 + rows + bs - 1) // bs
    p, c = tp.slice_cols(*full["out_proj"], C, C, bits, b0, b1 - b0, bs)
    out_proj = PackedLinear(p, c, C, (b1 - b0) * bs, bits, bs)
    # FFN: whole blocks of hidden channels; gate rows then up rows in one matrix
    ch0, chn = tp.ffn_shard_plan(Fh, tp_size, tp_rank, bs)
    gp, gc = tp.slice_rows(*full["gate"], Fh, C, bits, ch0, chn, bs)
    up, uc = tp.slice_rows(*full["up"], Fh, C, bits, ch0, chn, bs)
    gate_up = PackedLinear(torch.cat([gp, up]), torch.cat([gc, uc]), 2 * chn, C, bits, bs)
    dp, dc = tp.slice_cols(*full["down"], C, Fh, bits, ch0 // bs, chn // bs, bs)
    down = PackedLinear(dp, dc, C, chn, bits, bs)
    return PackedBlock(qkv, out_proj, gate_up, down, ln1, ln2)


def init_kv_cache(model: PackedGPT, batch_size: int = 1, device="cuda"):
    """fp32 (B, local heads, context_len, head_dim) key and value buffers per layer and a length
    (inference/generate_torch.py:269-277)."""
    hd = model.config.head_dim
    caches = []
    for _ in range(model.n_layers):
        k = torch.zeros(batch_size, model.heads_local, model.context_len, hd, device=device, dtype=torch.float32)
        caches.append((k, torch.zeros_like(k), 0))
    return caches


def prefill(model: PackedGPT, x: torch.Tensor, caches):
    """(logits[:, -1, :], caches) for a prompt (inference/generate.py:169-175)."""
    logits, caches = model(x, kv_caches=caches)
    return logits[:, -1, :], caches


def step(model: PackedGPT, x: torch.Tensor, caches):
    """(logits[:, -1, :], caches) for one new token per sequence (inference/generate.py:177-183)."""
    logits, caches = model(x, kv_caches=caches)
    return logits[:, -1, :], caches


class DecodeSession:
    """Greedy decoding with the whole step in one CUDA graph: token, position and caches live on the
    device, the next token is the argmax written back into the token buffer, so N steps are N graph
    replays without a host round trip.  Attention in the captured step covers the full context
    buffer under a position mask (static shapes), as the reference's cached path does
    (inference/generate_torch.py:91-97)."""

    def __init__(self, model: PackedGPT, batch_size: int = 1, use_graph: bool = True, fused: bool = True,
                 batch_gemm: bool = False, stream: bool | None = None, tile_gemv: bool | None = None, hand_head: bool = True):
        self.model, self.B = model, batch_size
        self.hand_head = hand_head            # False: the LM head of a single sequence stays a library GEMM (comparison)
        self.residual_in_matvec = False       # True: out_proj and down add into the residual stream themselves (flag 4 of
                                              # nb_gemv_stream) instead of the next norm prologue: bit-identical, measured neutral
        self.single_term = False              # True: activations enter the matvecs as one fp16 term: 7 % faster, but 4e-3 of
                                              # max |logit| away from the two-term step at 26 layers (the gate is 2e-3)
        self.swiglu_epilogue = True           # SwiGLU in gate_up's epilogue: down stages F values instead of 2F (costs a
                                              # second stream-layout copy of gate_up, rows interleaved gate / up per tile)
        self.fused = fused
        # one sequence: the packed linears of the step run on the kernel that reads the tile-major copy of the weights
        # (nb_gemv_stream: teams of warps per row tile, no workspace); tile_gemv=False keeps nb_gemv_fused
        blk0 = model.blocks[0] if len(model.blocks) else None
        fits = (blk0 is not None and model.config.block_size == 128 and model.config.bits in (2, 3, 4)
                and all(l.in_features % 128 == 0 and l.in_features <= 7168 for l in (blk0.qkv, blk0.out_proj, blk0.gate_up, blk0.down)))
        self.tile_gemv = bool(fits and batch_size == 1 and fused) if tile_gemv is None else bool(tile_gemv and fits and batch_size == 1)
        # 2 .. 8 sequences: the same kernel family with the rows in the MMA columns a single row leaves empty
        # (nb_gemv_stream_rows): one pass over the weights for all rows, as many rows per launch as shared memory holds
        self.tile_rows = bool(fits and 2 <= batch_size <= 8 and fused and tile_gemv is not False
                              and getattr(model, "exchange", None) is None)
        # stream=True (one sequence on one GPU): the whole step is ONE launch of the persistent kernel
        # (stream.py).  The default is the chain of fused kernels, which measures faster: inside one launch
        # every operation pays a device-wide flag wait and the staging of its activations in full.
        self.stream_step = bool(stream)
        if self.stream_step:
            from . import stream as _stream
            if not _stream.stream_supported(model, batch_size):
                raise RuntimeError("the one-launch decode step needs batch 1, one rank, bf16 embeddings and block-128 codebooks")
        self.prog = None
        self.batch_gemm = batch_gemm          # kept for compatibility: batches above 16 rows always take the tensor-core kernel
        dev = model.embedding.device
        self.dev = dev
        self.caches = init_kv_cache(model, batch_size, dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.pos_host = 0                     # the same position, tracked on the host: steps past the context are refused
        self.token = torch.zeros(batch_size, 1, dtype=torch.long, device=dev)
        self.logits = torch.zeros(batch_size, model.config.vocab_size, dtype=torch.float32, device=dev)
        self.k_idx = torch.arange(model.context_len, device=dev)
        self.use_graph = use_graph
        self.graph = None
        self._prefill_graphs = {}             # prompt length -> (captured prefill, its static input)
        self.stream = torch.cuda.Stream(device=dev)
        if fused:  # static activation buffers of the fused step
            cfg, B = model.config, batch_size
            f32 = dict(dtype=torch.float32, device=dev)
            blk = model.blocks[0]
            self.bx = torch.zeros(B, cfg.n_embd, **f32)
            self.bx2 = torch.zeros(B, cfg.n_embd, **f32)
            self.bh = torch.zeros(B, cfg.n_embd, **f32)
            self.bqkv = torch.zeros(B, blk.qkv.out_features, **f32)
            self.bq = torch.zeros(B, model.heads_local, cfg.head_dim, **f32)
            self.batt = torch.zeros(B, model.o_cols, **f32)      # columns outside this rank's heads stay zero
            self.bo = torch.zeros(B, cfg.n_embd, **f32)
            self.bgu = torch.zeros(B, blk.gate_up.out_features, **f32)
            self.bhm = torch.zeros(B, blk.down.in_features, **f32)
            self.bd = torch.zeros(B, cfg.n_embd, **f32)

    def _linear_into(self, lin: PackedLinear, x: torch.Tensor, out: torch.Tensor) -> None:
        """out = lin(x) for a batch of rows: up to 16 through the fused GEMV, more through the tensor-core
        kernel that dequantises inside (one pass over the weights, exact fp16 weights, fp32 activations as
        two fp16 terms)."""
        if x.shape[0] > 16 and lin.in_features % 128 == 0:
            ops.gemm_prefill_fused(x, lin.stream_weight(), lin.bits, lin.out_features, lin.in_features, out=out)
            return
        for r in range(0, x.shape[0], 16):
            ops.gemv(x[r:r + 16], lin.packed_indices, lin.codebook, lin.bits, lin.block_size, lin.out_features,
                     lin.in_features, out=out[r:r + 16])

    @torch.no_grad()
    def _step_body_fused(self):
        """The decode step on the fused kernels.  Up to 8 sequences: 5 launches per layer (residual add +
        RMSNorm and SwiGLU are computed inside the packed GEMVs that consume them); more: 8 launches."""
        m, cfg = self.model, self.model.config
        eps = cfg.norm_eps
        fold = self.B <= 8
        xch = getattr(m, "exchange", None) if fold else None     # all-reduces folded into the GEMVs
        xa, xb = self.bx, self.bx2                                # residual stream, ping-pong
        if m.embedding.dtype == torch.bfloat16:
            ops.embed_rows(m.embedding, self.token, xa)
        else:
            xa.copy_(m.embedding[self.token[:, 0]])
        delta = None
        pending = False                                           # a pushed vector waits to be gathered
        # one sequence on one rank: out_proj and down add their result to the residual stream themselves
        inplace = self.tile_gemv and m.tp_size == 1 and xch is None and self.residual_in_matvec

        def norm_linear(lin, delta, w, out, swiglu=False):
            nonlocal xa, xb, pending
            args = (lin.packed_indices, lin.codebook, lin.bits, lin.block_size, lin.out_features, lin.in_features)
            if pending:
                ops.gemv_tp(ops.PRO_ADD_RMSNORM, xa, *args, xch, out=out, gather=True, norm_weight=w, eps=eps, x_out=xb)
                xa, xb = xb, xa
                pending = False
            elif self.tile_gemv and inplace:                      # the residual stream was updated by the matvec before
                ops.gemv_stream(ops.PRO_ADD_RMSNORM, xa, lin.stream_weight(1 if swiglu else 0), lin.bits, lin.out_features,
                                lin.in_features, out, norm_weight=w, eps=eps, swiglu=swiglu, single_term=self.single_term)
            elif self.tile_gemv:
                ops.gemv_stream(ops.PRO_ADD_RMSNORM, xa, lin.stream_weight(1 if swiglu else 0), lin.bits, lin.out_features,
                                lin.in_features, out, delta=delta, norm_weight=w, eps=eps, x_out=xb, swiglu=swiglu,
                                single_term=self.single_term)
                xa, xb = xb, xa
            elif self.tile_rows:
                ops.gemv_stream_rows(ops.PRO_ADD_RMSNORM, xa, lin.stream_weight(1 if swiglu else 0), lin.bits, lin.out_features,
                                     lin.in_features, out, delta=delta, norm_weight=w, eps=eps, x_out=xb, swiglu=swiglu)
                xa, xb = xb, xa
            elif fold:
                ops.gemv_fused(ops.PRO_ADD_RMSNORM, xa, *args, out, delta=delta, norm_weight=w, eps=eps, x_out=xb)
                xa, xb = xb, xa
            else:
                ops.add_rmsnorm(xa, delta, w, eps, self.bh)
                self._linear_into(lin, self.bh, out)

        def row_parallel(lin, prologue, x, out):
            """out_proj / down: the result is a partial sum over the ranks."""
            nonlocal pending
            args = (lin.packed_indices, lin.codebook, lin.bits, lin.block_size, lin.out_features, lin.in_features)
            if xch is not None:
                ops.gemv_tp(prologue, x, *args, xch, push=True)
                pending = True
                return None
            if self.tile_gemv and inplace:                        # x += W act(...): no delta vector, no add in the next norm
                ops.gemv_stream(prologue, x, lin.stream_weight(), lin.bits, lin.out_features, lin.in_features, xa,
                                single_term=self.single_term, accumulate=True)
                return None
            if self.tile_gemv:
                ops.gemv_stream(prologue, x, lin.stream_weight(), lin.bits, lin.out_features, lin.in_features, out,
                                single_term=self.single_term)
            elif self.tile_rows:
                ops.gemv_stream_rows(prologue, x, lin.stream_weight(), lin.bits, lin.out_features, lin.in_features, out)
            elif prologue == ops.PRO_SILU_MUL and fold:
                ops.gemv_fused(prologue, x, *args, out)
            elif prologue == ops.PRO_SILU_MUL:
                ops.silu_mul(x, self.bhm)
                self._linear_into(lin, self.bhm, out)
            else:
                self._linear_into(lin, x, out)
            return m._all_reduce(out)

        for i, blk in enumerate(m.blocks):
            k_buf, v_buf, _ = self.caches[i]
            norm_linear(blk.qkv, delta, blk.ln1, self.bqkv)
            ops.decode_attention_rope(self.bqkv, m.cos2, m.sin2, self.pos, k_buf, v_buf, self.batt, m.o_col0)
            delta = row_parallel(blk.out_proj, ops.PRO_NONE, self.batt, self.bo)
            # SwiGLU in gate_up's epilogue (nb_gemv_stream's swiglu flag over a row_mode-1 copy): the 2F intermediate is
            # never written and down stages half the bytes (0.897 -> 0.875 ms per token)
            if (self.tile_gemv or self.tile_rows) and self.swiglu_epilogue and xch is None:
                norm_linear(blk.gate_up, delta, blk.ln2, self.bhm[0] if self.tile_gemv else self.bhm, swiglu=True)
                delta = row_parallel(blk.down, ops.PRO_NONE, self.bhm, self.bd)
                continue
            norm_linear(blk.gate_up, delta, blk.ln2, self.bgu)
            delta = row_parallel(blk.down, ops.PRO_SILU_MUL, self.bgu, self.bd)
        if pending:
            ops.exchange_gather(self.bd, xch, xch.status)
            delta = self.bd
        if (self.B == 1 and self.hand_head and getattr(m, "head_ar", None) is None and m.tp_size == 1
                and ops.lm_head_supported(m.embedding)):
            # one sequence on one GPU: final add + norm, the tied head over the bf16 table, soft-cap and arg-max in two launches
            ops.lm_head(xa, delta, m.ln_f, eps, m.embedding, cfg.logit_cap, self.logits, self.token, self.pos)
            return
        ops.add_rmsnorm(xa, delta, m.ln_f, eps, self.bh)
        if getattr(m, "head_ar", None) is not None and self.B <= m.head_batch:
            if getattr(self, "blog_in", None) is None:
                self.blog_in = torch.zeros(self.B, m.embedding.shape[0], dtype=torch.float32, device=self.bh.device)
                self.blog_sum = torch.empty_like(self.blog_in)
            r0, rn = m.head_rows
            self.blog_in[:, r0:r0 + rn].copy_(m._head(self.bh, m.head_rows))   # the rest of blog_in stays zero
            logits = m.head_ar(self.blog_in, out=self.blog_sum)
        else:
            logits = m._head(self.bh)                            # the LM head is a plain library GEMM (bf16 table, 164 MB)
        ops.softcap_argmax(logits, cfg.logit_cap, self.logits, self.token, self.pos)

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """prompt (B, T): fills the caches, sets the position and the first generated token."""
        if prompt.shape[1] > self.model.context_len:
            raise RuntimeError(f"prompt of {prompt.shape[1]} tokens exceeds the context of {self.model.context_len}")
        T = int(prompt.shape[1])
        if not self.use_graph or not prompt.is_cuda:
            self._prefill_body(prompt)
        else:
            # one CUDA graph per prompt length: the eager forward is about thirty small launches per layer and
            # is bound by the host; replayed from a graph only the device time remains
            entry = self._prefill_graphs.get(T)
            cur = torch.cuda.current_stream(self.dev)
            if entry is None:
                static_in = prompt.clone()
                self.stream.wait_stream(cur)
                with torch.cuda.stream(self.stream):
                    self._prefill_body(static_in)            # warms every kernel up and IS this call's result
                    self.stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=self.stream):
                        self._prefill_body(static_in)
                cur.wait_stream(self.stream)
                self._prefill_graphs[T] = (g, static_in)
            else:
                g, static_in = entry
                static_in.copy_(prompt)
                g.replay()
        self.caches = [(k, v, T) for k, v, _ in self.caches]
        self.pos_host = T
        return self.logits

    def _prefill_body(self, prompt: torch.Tensor) -> None:
        caches = [(k, v, 0) for k, v, _ in self.caches]
        logits, _ = self.model(prompt, kv_caches=caches, last_only=True)      # the caches are written in place
        self.pos.fill_(prompt.shape[1])
        self.logits.copy_(logits[:, -1, :])
        self.token.copy_(self.logits.argmax(-1, keepdim=True))

    @torch.no_grad()
    def _step_body(self):
        if self.stream_step:
            if self.prog is None:
                from . import stream as _stream
                self.prog = _stream.build_decode_program(self.model, self)
            return self.prog.run()
        if self.fused:
            return self._step_body_fused()
        m, cfg = self.model, self.model.config
        B = self.B
        x = m.embedding[self.token].float()                      # (B, 1, C)
        mask = (self.k_idx <= self.pos)[None, None, None, :]     # (1, 1, 1, ctx)
        for i, blk in enumerate(m.blocks):
            k_buf, v_buf, _ = self.caches[i]
            q, k, v = m._attn_inputs(x, blk, self.pos, 1)
            k_buf.index_copy_(2, self.pos, k)
            v_buf.index_copy_(2, self.pos, v)
            out = F.scaled_dot_product_attention(q, k_buf, v_buf, attn_mask=mask)
            x = m._finish_block(x, blk, out.transpose(1, 2).reshape(B, 1, -1))
        self.logits.copy_(m._logits(x)[:, -1, :])
        self.token.copy_(self.logits.argmax(-1, keepdim=True))
        self.pos.add_(1)

    def check(self) -> None:
        """Raises if a bounded wait of the step's kernels ever ran out (a copy barrier, or a peer of the
        tensor-parallel exchange that never arrived).  Reads device status words: synchronises."""
        if self.prog is not None and self.prog.status() != 0:
            raise RuntimeError("nb_stream_run: a bounded wait ran out (status NB_ERR_TIMEOUT in the program state)")
        for st in ((self.stream, torch.cuda.current_stream(self.dev)) if self.use_graph else (torch.cuda.current_stream(self.dev),)):
            with torch.cuda.stream(st):          # the workspace of the stream the steps ran on
                ws = ops.workspace(self.model.embedding.device, 0)
            if ops.workspace_status(ws) != 0:
                raise RuntimeError("nb_gemv: a bounded wait ran out (status NB_ERR_TIMEOUT in the workspace)")
        for name in ("oneshot", "head_ar", "exchange"):
            obj = getattr(self.model, name, None)
            if obj is not None and int(obj.status.item()) != 0:
                raise RuntimeError(f"{name}: a peer did not arrive within the bounded wait")

    def step(self) -> None:
        """One decode step for every sequence: consumes self.token, leaves the next token there.
        Raises (before anything is launched) when the cache has no free slot left."""
        ctx = self.model.context_len
        if self.pos_host >= ctx:
            raise RuntimeError(f"decode position {self.pos_host} is past the end of the context ({ctx}): the KV cache is full")
        if not self.use_graph:
            self._step_body()
            self.pos_host += 1
            return
        if self.graph is None:
            # the warm-up and the capture run on the session's stream: it must first see what the caller's
            # stream has written (prefill: caches, position, first token)
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                saved = (self.pos.clone(), self.token.clone(), self.logits.clone())
                for _ in range(min(2, ctx - self.pos_host)):      # warm-up outside capture, inside the context
                    self._step_body()
                self.stream.synchronize()
                self.pos.copy_(saved[0]); self.token.copy_(saved[1]); self.logits.copy_(saved[2])
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=self.stream):
                    self._step_body()
                # the capture does not execute: state is unchanged; stale cache slots past `pos` are masked
            torch.cuda.current_stream().wait_stream(self.stream)
        self.graph.replay()
        self.pos_host += 1

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_generate: int) -> torch.Tensor:
        """Greedy continuation (B, n_generate) of prompt (B, T)."""
        self.prefill(prompt)
        out = [self.token.clone()]
        for _ in range(n_generate - 1):
            self.step()
            out.append(self.token.clone())
        return torch.cat(out, dim=1)


def benchmark(model: PackedGPT, prompt_tokens, n_generate: int = 128, n_runs: int = 3, device="cuda", batch_size: int = 1,
              batch_gemm: bool = False):
    """Decode-speed benchmark with the reference's result keys (inference/generate_torch.py:280-320)
    plus the JAX twin's prefill fields (inference/generate.py:270-280)."""
    dev = model.embedding.device
    prompt = torch.as_tensor(prompt_tokens, dtype=torch.long, device=dev).reshape(1, -1).repeat(batch_size, 1)
    sess = DecodeSession(model, batch_size, batch_gemm=batch_gemm)
    sess.prefill(prompt)
    sess.step()
    torch.cuda.synchronize()
    pre, gen = [], []
    for _ in range(n_runs):
        t0 = time.perf_counter()
        sess.prefill(prompt)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(n_generate):
            sess.step()
        torch.cuda.synchronize()
        pre.append(t1 - t0)
        gen.append(time.perf_counter() - t1)
    sess.check()
    g, p = sum(gen) / len(gen), sum(pre) / len(pre)
    return {"label": f"b{batch_size}", "prompt_len": prompt.shape[1], "n_generate": n_generate, "n_runs": n_runs,
            "prefill_ms": round(p * 1e3, 2), "prefill_tps": round(prompt.numel() / p, 1),
            "generate_ms": round(g * 1e3, 2), "generate_tps": round(n_generate * batch_size / g, 1),
            "per_token_ms": round(g / n_generate * 1e3, 3)}


# ---------------------------------------------------------------------- checkpoints
def _nat_key(s: str):
    return [int(c) if c.isdigit() else c for c in re.split(r"(\d+)", s)]


def load_packed_model(packed_path: str, config, device="cuda", tp_rank: int = 0, tp_size: int = 1, group=None) -> PackedGPT:
    """Load a .nbpack.npz written by the reference's inference/pack.py (keys idx./cb./shape./idxshape./
    param./__metadata__, :110-151) into a PackedGPT.  Layers are matched to the packed keys in natural
    sort order, five per block in the order qkv, out_proj, gate, up, down
    (inference/generate_torch.py:224-241).  Packed bytes are uploaded as stored; fp32 codebooks are
    kept fp32."""
    pack = np.load(packed_path)
    dev = torch.device(device)
    cfg = config if isinstance(config, ModelConfig) else ModelConfig(
        vocab_size=config.vocab_size, n_layers=config.n_layers, n_embd=config.n_embd, n_head=config.n_head,
        ffn_hidden=config.ffn_hidden, context_len=config.context_len,
        block_size=getattr(config, "block_size", 128), bits=int(math.log2(getattr(config, "n_codebook", 8))))
    keys = sorted((k[4:] for k in pack.files if k.startswith("idx.")), key=_nat_key)
    if len(keys) != 5 * cfg.n_layers:
        raise RuntimeError(f"expected {5 * cfg.n_layers} packed layers, found {len(keys)}")

    def get(prefix):
        p = torch.from_numpy(np.ascontiguousarray(pack[f"idx.{prefix}"])).to(dev)
        c = torch.from_numpy(np.ascontiguousarray(pack[f"cb.{prefix}"])).to(dev)
        return p, c

    params = {}
    for k in pack.files:
        if k.startswith("param."):
            arr = pack[k]
            if arr.dtype.kind == "V":
                arr = np.frombuffer(arr.tobytes(), dtype=np.float16).reshape(arr.shape)
            params[k[6:].replace(".", "/")] = arr
    C = cfg.n_embd
    blocks = []
    for l in range(cfg.n_layers):
        names = keys[5 * l:5 * l + 5]
        full = dict(zip(("qkv", "out_proj", "gate", "up", "down"), (get(n) for n in names)))
        ln = []
        for j in range(2):
            w = params.get(f"params/block_{l}/RMSNorm_{j}/weight")
            ln.append(torch.from_numpy(w.astype(np.float32)).to(dev) if w is not None else torch.ones(C, device=dev))
        blocks.append(shard_block(cfg, full, ln[0], ln[1], tp_rank, tp_size))
    emb = params.get("params/embedding")
    if emb is None:
        raise RuntimeError("checkpoint has no params/embedding")
    emb_t = torch.from_numpy(np.ascontiguousarray(emb)).to(dev)
    lnf = params.get("params/ln_f/weight")
    lnf_t = torch.from_numpy(lnf.astype(np.float32)).to(dev) if lnf is not None else torch.ones(C, device=dev)
    return PackedGPT(cfg, emb_t, blocks, lnf_t, tp_rank, tp_size, group)

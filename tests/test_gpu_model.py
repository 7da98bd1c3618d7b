"""The packed decoder on the GPU against the reference's own PackedGPT logits (golden) and the dense
oracle: eager prefill + cached steps, the CUDA-graph decode session, teacher-forced greedy agreement,
and the tensor-parallel block shards evaluated on one GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import nb_model_oracle as mo

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def gm():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_model.npz"))


def _build(gm, dev, tp_rank=0, tp_size=1):
    from nativebit_b200 import generate as G
    V, L, C, H, Fh, ctx = (int(v) for v in gm["cfg"])
    cfg = G.ModelConfig(vocab_size=V, n_layers=L, n_embd=C, n_head=H, ffn_hidden=Fh, context_len=ctx)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    blocks = []
    for l in range(L):
        full = {k2: (cu(gm[f"p_{k1}{l}"]), cu(gm[f"c_{k1}{l}"])) for k1, k2 in
                (("qkv", "qkv"), ("out", "out_proj"), ("gate", "gate"), ("up", "up"), ("down", "down"))}
        ones = torch.ones(C, device=dev)
        blocks.append(G.shard_block(cfg, full, ones, ones.clone(), tp_rank, tp_size))
    emb = cu(gm["embedding"])
    return G.PackedGPT(cfg, emb, blocks, torch.ones(C, device=dev), tp_rank, tp_size), cfg


def test_decoder_matches_reference_logits(built_lib, gm):
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    model, cfg = _build(gm, dev)
    caches = G.init_kv_cache(model, 1, dev)
    prompt = torch.from_numpy(gm["prompt"]).to(dev)
    logits, caches = model(prompt, kv_caches=caches)
    ref = gm["logits_prompt"]
    # fp16 activations inside the packed linears: 2e-3 of max|logit| is the stated gate
    assert np.abs(logits[0].cpu().numpy() - ref).max() <= 2e-3 * np.abs(ref).max()
    for t, r in zip(gm["forced"].tolist(), gm["logits_steps"]):
        lg, caches = G.step(model, torch.tensor([[t]], device=dev), caches)
        assert np.abs(lg[0].cpu().numpy() - r).max() <= 2e-3 * np.abs(ref).max()
    # no-cache forward equals the cached one
    nc = model(prompt)
    assert (nc - logits).abs().max() <= 1e-5


def test_graph_session_equals_eager_and_oracle_greedy(built_lib, gm):
    """Free-running greedy decode from the CUDA-graph session against the dense oracle run
    teacher-forced on the session's tokens: the oracle's argmax must agree at >= 99 % of steps."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    model, cfg = _build(gm, dev)
    prompt = torch.from_numpy(gm["prompt"]).to(dev)
    n_gen = 20
    toks_graph = G.DecodeSession(model, 1, use_graph=True).generate(prompt, n_gen)
    toks_eager = G.DecodeSession(model, 1, use_graph=False).generate(prompt, n_gen)
    assert torch.equal(toks_graph, toks_eager)
    V, L, C, H, Fh, ctx = (int(v) for v in gm["cfg"])
    layers = {f"{nm}{l}": (gm[f"p_{nm}{l}"], gm[f"c_{nm}{l}"], tuple(int(v) for v in gm[f"s_{nm}{l}"]))
              for l in range(L) for nm in ("qkv", "out", "gate", "up", "down")}
    om = mo.DenseModel(mo.dense_weights_from_packed(layers, gm["embedding"], L), L, H, ctx)
    caches = om.init_cache()
    lg = om.forward(torch.from_numpy(gm["prompt"]), caches)[0, -1]
    agree, ours = 0, toks_graph[0].cpu().tolist()
    for i, t in enumerate(ours):
        agree += int(int(lg.argmax()) == t)
        lg = om.forward(torch.tensor([[t]]), caches)[0, -1]
    assert agree / len(ours) >= 0.99


def test_fused_step_equals_torch_step(built_lib, gm):
    """The fused glue kernels (RMSNorm, RoPE + cache write, single-query attention, SwiGLU) against the
    same step written with torch ops: identical greedy tokens and logits within fp32 rounding."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    model, cfg = _build(gm, dev)
    prompt = torch.from_numpy(gm["prompt"]).to(dev)
    for B in (1, 3):
        a = G.DecodeSession(model, B, use_graph=False, fused=True)
        b = G.DecodeSession(model, B, use_graph=False, fused=False)
        a.prefill(prompt.repeat(B, 1)); b.prefill(prompt.repeat(B, 1))
        for _ in range(12):
            a.step(); b.step()
            assert torch.equal(a.token, b.token)
            assert (a.logits - b.logits).abs().max() <= 1e-4 * b.logits.abs().max()


def test_rope_attention_fusion_equals_two_kernels(built_lib):
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    B, H, hd, ctx = 3, 4, 80, 64
    from nativebit_b200.generate import precompute_rope
    cos2, sin2 = precompute_rope(hd, ctx, 10000.0, dev)
    ka = torch.randn(B, H, ctx, hd, device=dev, generator=g); va = torch.randn(B, H, ctx, hd, device=dev, generator=g)
    kb, vb = ka.clone(), va.clone()
    for p_ in (0, 5, 37):
        pos = torch.tensor([p_], device=dev)
        qkv = torch.randn(B, 3 * H * hd, device=dev, generator=g)
        q = torch.empty(B, H, hd, device=dev)
        o1 = torch.zeros(B, H * hd + 16, device=dev); o2 = torch.zeros_like(o1)
        ops.rope_kv_write(qkv, H, hd, cos2, sin2, pos, ka, va, q)
        ops.decode_attention(q, ka, va, pos, o1, 8)
        ops.decode_attention_rope(qkv, cos2, sin2, pos, kb, vb, o2, 8)
        torch.cuda.synchronize()
        assert torch.equal(ka, kb) and torch.equal(va, vb) and torch.equal(o1, o2)


@pytest.mark.parametrize("B,H,hd,ctx", [(1, 32, 80, 1024), (1, 4, 80, 1024), (8, 32, 80, 512), (24, 32, 64, 256), (2, 3, 128, 200),
                                         (1, 2, 4, 16)])
def test_decode_attention_against_torch(built_lib, B, H, hd, ctx):
    """Every cluster size (8, 4, 2, 1 CTAs per head), positions at the edges of the key ranges."""
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(B * 1000 + H)
    k = torch.randn(B, H, ctx, hd, device=dev, generator=g)
    v = torch.randn(B, H, ctx, hd, device=dev, generator=g)
    for p_ in sorted({0, 1, 7, 8, 63, 64, 65, 127, 128, ctx // 2, ctx - 2, ctx - 1} & set(range(ctx))):
        pos = torch.tensor([p_], device=dev)
        q = torch.randn(B, H, hd, device=dev, generator=g)
        out = torch.zeros(B, H * hd, device=dev)
        ops.decode_attention(q, k, v, pos, out, 0)
        n = p_ + 1
        sc = torch.einsum("bhd,bhjd->bhj", q.double(), k[:, :, :n].double()) / hd ** 0.5
        ref = torch.einsum("bhj,bhjd->bhd", torch.softmax(sc, -1), v[:, :, :n].double()).reshape(B, H * hd)
        assert (out.double() - ref).abs().max() <= 2e-5 * ref.abs().max(), p_


@pytest.mark.parametrize("B,T,H,hd,ctx,pos0,o_stride,o_off", [(1, 128, 32, 80, 1024, 0, 2560, 0), (2, 37, 4, 80, 256, 0, 320, 0),
                                                                (1, 1, 3, 64, 64, 0, 192, 0), (3, 50, 2, 128, 200, 23, 384, 128),
                                                                (1, 16, 4, 80, 64, 48, 320, 0), (2, 200, 5, 80, 512, 100, 400, 0)])
def test_prefill_attention_against_torch(built_lib, B, T, H, hd, ctx, pos0, o_stride, o_off):
    """RoPE + cache write + causal attention of a prompt chunk in one launch against the torch expressions of the
    reference's cached path in fp64; prompts that are no multiple of the query tile, chunks that continue a cache,
    an output wider than the heads (the padded out_proj input of an 8-way shard)."""
    from nativebit_b200 import ops
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(B * 1000 + T)
    cos2, sin2 = G.precompute_rope(hd, ctx, 10000.0, dev)
    qkv = torch.randn(B, T, 3 * H * hd, device=dev, generator=g)
    k_cache = torch.randn(B, H, ctx, hd, device=dev, generator=g)      # below pos0: an earlier chunk's keys; above: stale values
    v_cache = torch.randn(B, H, ctx, hd, device=dev, generator=g)
    k0, v0 = k_cache.clone(), v_cache.clone()
    out = torch.full((B * T, o_stride), 7.0, device=dev)
    ops.prefill_attention(qkv.view(B * T, -1), T, cos2, sin2, pos0, k_cache, v_cache, out, o_off)
    q, k, v = (t.reshape(B, T, H, hd).transpose(1, 2) for t in qkv.split(H * hd, dim=-1))
    qr = G.apply_rope(q, cos2[pos0:pos0 + T], sin2[pos0:pos0 + T])
    kr = G.apply_rope(k, cos2[pos0:pos0 + T], sin2[pos0:pos0 + T])
    # the caches: rotated keys and the values at pos0 .. pos0 + T - 1, everything else untouched
    assert torch.allclose(k_cache[:, :, pos0:pos0 + T], kr, rtol=0, atol=2e-6)
    assert torch.equal(v_cache[:, :, pos0:pos0 + T], v)
    for c, c0 in ((k_cache, k0), (v_cache, v0)):
        assert torch.equal(c[:, :, :pos0], c0[:, :, :pos0]) and torch.equal(c[:, :, pos0 + T:], c0[:, :, pos0 + T:])
    n = pos0 + T
    kk = torch.cat((k0[:, :, :pos0], kr), dim=2).double()
    vv = torch.cat((v0[:, :, :pos0], v), dim=2).double()
    sc = torch.einsum("bhtd,bhjd->bhtj", qr.double(), kk) / hd ** 0.5
    mask = torch.arange(n, device=dev)[None, :] <= (pos0 + torch.arange(T, device=dev))[:, None]
    sc = sc.masked_fill(~mask, float("-inf"))
    ref = torch.einsum("bhtj,bhjd->bhtd", torch.softmax(sc, -1), vv).transpose(1, 2).reshape(B * T, H * hd)
    got = out[:, o_off:o_off + H * hd].double()
    assert (got - ref).abs().max() <= 2e-5 * ref.abs().max()
    assert bool((out[:, :o_off] == 7.0).all()) and bool((out[:, o_off + H * hd:] == 7.0).all())   # nothing outside the heads' columns


@pytest.mark.parametrize("V,C", [(32000, 2560), (515, 256), (1000, 3072), (40, 512)])
def test_lm_head_kernel_against_torch(built_lib, V, C):
    """Final add + RMSNorm, tied head over the bf16 table, soft-cap, arg-max and position increment in two launches,
    against the torch expressions of the reference's step in fp64; equal rows: the lowest index wins."""
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(V + C)
    table = (0.05 * torch.randn(V, C, device=dev, generator=g)).bfloat16()
    table[V // 2] = table[3]                                        # two equal rows ...
    x = torch.randn(1, C, device=dev, generator=g)
    x = x + 10.0 * table[3].float() / table[3].float().norm()       # ... that carry the largest logit by a wide margin
    delta = 0.1 * torch.randn(1, C, device=dev, generator=g)
    w = 1.0 + 0.1 * torch.randn(C, device=dev, generator=g)
    cap = 30.0
    for d, wt in ((delta, w), (None, w), (None, None)):
        logits = torch.full((1, V), float("nan"), device=dev)
        tok = torch.full((1, 1), -1, dtype=torch.long, device=dev)
        pos = torch.tensor([41], device=dev)
        ops.lm_head(x, d, wt, 1e-6, table, cap, logits, tok, pos)
        v = x.double() + (0 if d is None else d.double())
        h = v if wt is None else v / torch.sqrt((v * v).mean() + 1e-6) * wt.double()
        ref = cap * torch.tanh((h @ table.double().T) / cap)
        assert (logits.double() - ref).abs().max() <= 2e-5 * ref.abs().max()
        assert int(pos.item()) == 42
        best = logits.max()
        assert int(tok.item()) == int((logits[0] == best).nonzero()[0].item())       # lowest index among equals
        assert int(tok.item()) == 3 and bool(logits[0, 3] == logits[0, V // 2])


def test_step_ends_match_torch(built_lib):
    """Embedding lookup and soft-cap + argmax kernels against the torch expressions of the reference's step."""
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    V, C, B = 32000, 2560, 5
    table = (0.02 * torch.randn(V, C, device=dev, generator=g)).bfloat16()
    token = torch.tensor([[0], [V - 1], [17], [31999], [12345]], device=dev)
    out = torch.empty(B, C, device=dev)
    ops.embed_rows(table, token, out)
    assert torch.equal(out, table[token[:, 0]].float())
    for dtype in (torch.bfloat16, torch.float32):
        logits = (40 * torch.randn(B, V, device=dev, generator=g)).to(dtype)
        logits[1, 100] = logits[1, 7] = 1000.0                   # saturated: equal capped values, lowest index wins
        cap = 30.0
        ref = cap * torch.tanh(logits.float() / cap)
        capped = torch.empty(B, V, device=dev)
        tok = torch.zeros(B, 1, dtype=torch.long, device=dev)
        pos = torch.tensor([41], device=dev)
        ops.softcap_argmax(logits, cap, capped, tok, pos)
        assert torch.allclose(capped, ref, rtol=1e-6, atol=1e-6)   # torch divides by multiplying with 1/cap: last-bit differences
        assert int(pos.item()) == 42
        best = capped.max(dim=1).values
        for b in range(B):
            first = int((capped[b] == best[b]).nonzero()[0])       # lowest index among equal capped values
            assert int(tok[b, 0]) == first
        assert int(tok[1, 0]) == 7


def test_batched_session(built_lib, gm):
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    model, cfg = _build(gm, dev)
    prompt = torch.from_numpy(gm["prompt"]).to(dev)
    one = G.DecodeSession(model, 1).generate(prompt, 8)
    four = G.DecodeSession(model, 4).generate(prompt.repeat(4, 1), 8)
    assert all(torch.equal(four[i:i + 1], one) for i in range(4))


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_shards_sum_to_single_rank(built_lib, gm, world):
    """All ranks' shards evaluated one after another on one GPU with the all-reduce done by hand:
    the block output equals the unsharded block's (exact up to fp32 summation order)."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    full, cfg = _build(gm, dev)
    ranks = [_build(gm, dev, r, world)[0] for r in range(world)]
    x = torch.randn(1, 3, cfg.n_embd, device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    blk = full.blocks[0]
    q, k, v = full._attn_inputs(x, blk, 0, 3)
    att = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(1, 3, -1)
    ref_o = blk.out_proj(att).float()
    ref_ffn = blk.down(torch.nn.functional.silu(blk.gate_up(x).float()[..., :cfg.ffn_hidden]) *
                       blk.gate_up(x).float()[..., cfg.ffn_hidden:]).float()
    acc_o = torch.zeros_like(ref_o)
    acc_f = torch.zeros_like(ref_ffn)
    for r, m in enumerate(ranks):
        b = m.blocks[0]
        qr, kr, vr = m._attn_inputs(x, b, 0, 3)
        hl = cfg.n_head // world
        assert torch.equal(qr, q[:, r * hl:(r + 1) * hl]) and torch.equal(vr, v[:, r * hl:(r + 1) * hl])
        a = torch.nn.functional.scaled_dot_product_attention(qr, kr, vr, is_causal=True).transpose(1, 2).reshape(1, 3, -1)
        pad = a.new_zeros(1, 3, m.o_cols)
        pad[..., m.o_col0:m.o_col0 + a.shape[-1]] = a
        acc_o += b.out_proj(pad).float()
        gu = b.gate_up(x).float()
        g_, u_ = gu.split(gu.shape[-1] // 2, dim=-1)
        acc_f += b.down(torch.nn.functional.silu(g_) * u_).float()
    assert (acc_o - ref_o).abs().max() <= 1e-4 * ref_o.abs().max()
    assert (acc_f - ref_ffn).abs().max() <= 1e-4 * ref_ffn.abs().max()


def test_large_batch_takes_the_tensor_core_kernel_and_agrees_with_the_gemv(built_lib, gm):
    """A batch of 32 sequences sends every packed linear through the tcgen05 kernel that dequantises inside
    (one pass over the weights, exact fp16 weights, fp32 activations as two fp16 terms); a batch of 16 runs the
    fused GEMV.  Same prompts: the logits must agree far inside the stated 2e-3."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    model, cfg = _build(gm, dev)
    prompt = torch.from_numpy(gm["prompt"]).to(dev).repeat(32, 1)
    a = G.DecodeSession(model, 16, use_graph=False)
    b = G.DecodeSession(model, 32, use_graph=False)
    a.prefill(prompt[:16]); b.prefill(prompt)
    for _ in range(3):
        a.step(); b.step()
    torch.cuda.synchronize()
    a.check(); b.check()
    assert (a.logits - b.logits[:16]).abs().max() <= 1e-4 * a.logits.abs().max()
    assert torch.equal(a.token, b.token[:16])


def test_graph_session_equals_eager_session_full_size(built_lib):
    """The 2.2B configuration, no synchronisation between prefill and the first (capturing) step: the
    graph session's logits equal the eager session's bit for bit, step after step."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    cfg = G.ModelConfig()
    model = G.PackedGPT.random_init(cfg, seed=0, device=dev)
    prompt = torch.randint(0, cfg.vocab_size, (1, 128), generator=torch.Generator().manual_seed(0)).to(dev)
    outs = {}
    for graph in (False, True):
        s = G.DecodeSession(model, 1, use_graph=graph)
        s.prefill(prompt)
        outs[graph] = []
        for _ in range(6):
            s.step()
            outs[graph].append((s.token.clone(), s.logits.clone()))
        s.check()
    torch.cuda.synchronize()
    for (ta, la), (tb, lb) in zip(outs[False], outs[True]):
        assert torch.equal(ta, tb) and torch.equal(la, lb)


def _dense_oracle_of(model, cfg, dev):
    """The dense fp32 oracle of a single-rank PackedGPT: every packed linear is materialised on the CPU by
    the oracle's own numpy gather (the reference's recipe, inference/compare.py:260-288) and evaluated with
    the oracle's torch ops on the GPU in fp32 (TF32 off)."""
    from oracle import nb_oracle as o
    C, Fh, L = cfg.n_embd, cfg.ffn_hidden, cfg.n_layers
    w = {"embedding": model.embedding.float()}
    for l, blk in enumerate(model.blocks):
        def dense(lin, rows=None):
            p, c = lin.packed_indices.cpu().numpy(), lin.codebook.float().cpu().numpy()
            W = o.dequant_packed(p, c, lin.out_features, lin.in_features, cfg.bits)
            return torch.from_numpy(W).to(dev)
        w[f"qkv{l}"], w[f"out{l}"], w[f"down{l}"] = dense(blk.qkv), dense(blk.out_proj), dense(blk.down)
        gu = dense(blk.gate_up)
        w[f"gate{l}"], w[f"up{l}"] = gu[:Fh].contiguous(), gu[Fh:].contiguous()
        del gu
        w[f"ln1_{l}"], w[f"ln2_{l}"] = blk.ln1.float(), blk.ln2.float()
    w["ln_f"] = model.ln_f.float()
    return mo.DenseModel(w, L, cfg.n_head, cfg.context_len)


def test_full_size_decoder_against_dense_oracle_teacher_forced(built_lib):
    """The 2.2B configuration (26 layers, hidden 2560, 32 heads, FFN 6912, vocab 32000, seed 0): a 128-token
    prompt and 256 teacher-forced steps.  At every step both models are fed the ORACLE's greedy token;
    the argmax of the CUDA-graph decode session must equal the oracle's at >= 99 % of the steps, and the
    logits of the prompt's last position and of the last step must agree within 2e-3 of max|logit|."""
    from nativebit_b200 import generate as G
    dev = torch.device("cuda:0")
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    cfg = G.ModelConfig()
    model = G.PackedGPT.random_init(cfg, seed=0, device=dev)
    om = _dense_oracle_of(model, cfg, dev)
    prompt = torch.randint(0, cfg.vocab_size, (1, 128), generator=torch.Generator().manual_seed(0)).to(dev)
    n_steps = 256
    ocache = om.init_cache()
    olog = om.forward(prompt, ocache)[0, -1]
    sess = G.DecodeSession(model, 1, use_graph=True)
    sess.prefill(prompt)
    scale = float(olog.abs().max())
    assert float((sess.logits[0] - olog).abs().max()) <= 2e-3 * scale
    agree, worst = 0, 0.0
    for i in range(n_steps):
        tok = olog.argmax().reshape(1, 1)
        sess.token.copy_(tok)                       # teacher forcing: the oracle's token, not ours
        sess.step()
        olog = om.forward(tok, ocache)[0, -1]
        agree += int(int(sess.token[0, 0]) == int(olog.argmax()))
        worst = max(worst, float((sess.logits[0] - olog).abs().max()) / float(olog.abs().max()))
    sess.check()
    print(f"teacher-forced greedy agreement {agree}/{n_steps}, worst logit error {worst:.2e} of max|logit|")
    assert agree / n_steps >= 0.99
    assert worst <= 2e-3

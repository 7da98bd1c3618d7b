"""The decoder oracle (dense fp32 restatement) against logits of the reference's own PackedGPT, and
the tensor-parallel shard arithmetic on CPU (single process and a world_size-2 gloo group)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import nb_oracle as o
from oracle import nb_model_oracle as mo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def gm():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_model.npz"))


def _packed_layers(gm, L):
    return {f"{nm}{l}": (gm[f"p_{nm}{l}"], gm[f"c_{nm}{l}"], tuple(int(v) for v in gm[f"s_{nm}{l}"]))
            for l in range(L) for nm in ("qkv", "out", "gate", "up", "down")}


def test_dense_oracle_matches_reference_model(gm):
    V, L, C, H, Fh, ctx = (int(v) for v in gm["cfg"])
    w = mo.dense_weights_from_packed(_packed_layers(gm, L), gm["embedding"], L)
    model = mo.DenseModel(w, L, H, ctx)
    caches = model.init_cache()
    logits = model.forward(torch.from_numpy(gm["prompt"]), caches)[0].numpy()
    assert np.abs(logits - gm["logits_prompt"]).max() <= 1e-5
    for t, ref in zip(gm["forced"].tolist(), gm["logits_steps"]):
        lg = model.forward(torch.tensor([[t]]), caches)[0, -1].numpy()
        assert np.abs(lg - ref).max() <= 1e-5
    assert (logits.argmax(-1) == gm["logits_prompt"].argmax(-1)).all()


# ------------------------------------------------------------------ tensor-parallel shard arithmetic
def test_split_even_and_ffn_plan():
    from nativebit_b200 import tp
    assert tp.split_even(54, 4) == [14, 14, 13, 13]
    assert tp.split_even(54, 8) == [7, 7, 7, 7, 7, 7, 6, 6]
    assert tp.split_even(20, 8) == [3, 3, 3, 3, 2, 2, 2, 2]
    spans = [tp.ffn_shard_plan(6912, 8, r) for r in range(8)]
    assert spans[0] == (0, 896) and spans[-1] == (6144, 768)
    assert sum(n for _, n in spans) == 6912 and all(s % 128 == 0 and n % 128 == 0 for s, n in spans)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_reassemble_bit_exact_and_sum_to_full_output(world):
    """Row shards are byte slices of the packed weight; column shards are whole blocks.  Dequantised
    shards equal the matching slices of the dense weight, and the row-parallel partial products sum
    to the unsharded product."""
    from nativebit_b200 import tp
    n, k = 256, 1280            # k = 10 blocks: uneven over 4 and 8 ranks
    packed, cb, _ = o.make_packed_linear(n, k, 3, seed=world)
    W = o.dequant_packed(packed, cb.astype(np.float32), n, k, 3)
    x = o.make_activation(2, k, 1)
    pt, ct = torch.from_numpy(packed), torch.from_numpy(cb)
    y = np.zeros((2, n), np.float64)
    for r in range(world):
        b0, bn = tp.share(k // 128, world, r)
        p, c = tp.slice_cols(pt, ct, n, k, 3, b0, bn)
        Wr = o.dequant_packed(p.numpy(), c.numpy().astype(np.float32), n, bn * 128, 3)
        assert np.array_equal(Wr, W[:, b0 * 128:(b0 + bn) * 128])
        y += x[:, b0 * 128:(b0 + bn) * 128].astype(np.float64) @ Wr.T.astype(np.float64)
        r0, rn = tp.share(n // 16, world, r)
        p2, c2 = tp.slice_rows(pt, ct, n, k, 3, r0 * 16, rn * 16)
        assert np.array_equal(o.dequant_packed(p2.numpy(), c2.numpy().astype(np.float32), rn * 16, k, 3),
                              W[r0 * 16:(r0 + rn) * 16])
    ref = x.astype(np.float64) @ W.T.astype(np.float64)
    assert np.abs(y - ref).max() <= 1e-9 * np.abs(ref).max()


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from nativebit_b200 import tp
    from oracle import nb_oracle as oo
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, k = 64, 768
    packed, cb, _ = oo.make_packed_linear(n, k, 3, seed=7)
    x = oo.make_activation(1, k, 3)
    b0, bn = tp.share(k // 128, world, rank)
    p, c = tp.slice_cols(torch.from_numpy(packed), torch.from_numpy(cb), n, k, 3, b0, bn)
    Wr = oo.dequant_packed(p.numpy(), c.numpy().astype(np.float32), n, bn * 128, 3)
    part = torch.from_numpy(x[:, b0 * 128:(b0 + bn) * 128].astype(np.float64) @ Wr.T.astype(np.float64))
    dist.all_reduce(part)
    if rank == 0:
        W = oo.dequant_packed(packed, cb.astype(np.float32), n, k, 3)
        ref = x.astype(np.float64) @ W.T.astype(np.float64)
        q.put(float(np.abs(part.numpy() - ref).max() / np.abs(ref).max()))
    dist.destroy_process_group()


def test_row_parallel_all_reduce_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=10) <= 1e-12


@pytest.mark.parametrize("world", [2, 4, 8])
def test_block_shards_cover_every_weight_exactly_once(world):
    """shard_block on CPU tensors for a head_dim-80 model whose per-rank attention columns are not
    whole codebook blocks (the 2.2B case at 8 ranks: 320 columns = 2.5 blocks): every rank's out_proj
    shard is the run of whole blocks covering its columns, activations outside its own columns are
    zero, and the partial products add up to the unsharded product; FFN shards split 9 blocks
    unevenly."""
    from nativebit_b200 import generate as G
    cfg = G.ModelConfig(vocab_size=64, n_layers=1, n_embd=640, n_head=8, ffn_hidden=1152, context_len=16)
    C, Fh = cfg.n_embd, cfg.ffn_hidden
    full_np = {"qkv": o.make_packed_linear(3 * C, C, 3, 1), "out_proj": o.make_packed_linear(C, C, 3, 2),
               "gate": o.make_packed_linear(Fh, C, 3, 3), "up": o.make_packed_linear(Fh, C, 3, 4),
               "down": o.make_packed_linear(C, Fh, 3, 5)}
    full = {k: (torch.from_numpy(v[0]), torch.from_numpy(v[1])) for k, v in full_np.items()}
    dense = {k: o.dequant_packed(v[0], v[1].astype(np.float32), *shape, 3) for (k, v), shape in
             zip(full_np.items(), ((3 * C, C), (C, C), (Fh, C), (Fh, C), (C, Fh)))}
    rng = np.random.default_rng(0)
    att = rng.standard_normal((2, C)).astype(np.float32)           # attention output, all heads
    hmid = rng.standard_normal((2, Fh)).astype(np.float32)         # SwiGLU output, all channels
    acc_o = np.zeros((2, C)); acc_d = np.zeros((2, C))
    hl = cfg.n_head // world
    rows = hl * cfg.head_dim
    seen_ffn = 0
    for r in range(world):
        blk = G.shard_block(cfg, full, torch.ones(C), torch.ones(C), r, world)
        deq = lambda lin: o.dequant_packed(lin.packed_indices.numpy(), lin.codebook.numpy().astype(np.float32),
                                           lin.out_features, lin.in_features, 3)
        # qkv rows: this rank's heads out of q, k and v
        Wq = deq(blk.qkv)
        want = np.concatenate([dense["qkv"][j * C + r * rows: j * C + (r + 1) * rows] for j in range(3)])
        assert np.array_equal(Wq, want)
        # out_proj: whole blocks covering [r*rows, (r+1)*rows); zero-padded activations
        Wo = deq(blk.out_proj)
        b0 = (r * rows) // 128
        assert np.array_equal(Wo, dense["out_proj"][:, b0 * 128: b0 * 128 + blk.out_proj.in_features])
        pad = np.zeros((2, blk.out_proj.in_features), np.float32)
        off = r * rows - b0 * 128
        pad[:, off:off + rows] = att[:, r * rows:(r + 1) * rows]
        acc_o += pad.astype(np.float64) @ Wo.T.astype(np.float64)
        # FFN channels in whole blocks
        ch0, chn = G.tp.ffn_shard_plan(Fh, world, r)
        assert ch0 == seen_ffn
        seen_ffn += chn
        Wgu = deq(blk.gate_up)
        assert np.array_equal(Wgu, np.concatenate([dense["gate"][ch0:ch0 + chn], dense["up"][ch0:ch0 + chn]]))
        Wd = deq(blk.down)
        assert np.array_equal(Wd, dense["down"][:, ch0:ch0 + chn])
        acc_d += hmid[:, ch0:ch0 + chn].astype(np.float64) @ Wd.T.astype(np.float64)
    assert seen_ffn == Fh
    ref_o = att.astype(np.float64) @ dense["out_proj"].T.astype(np.float64)
    ref_d = hmid.astype(np.float64) @ dense["down"].T.astype(np.float64)
    assert np.abs(acc_o - ref_o).max() <= 1e-9 * np.abs(ref_o).max()
    assert np.abs(acc_d - ref_d).max() <= 1e-9 * np.abs(ref_d).max()

"""The persistent multi-matrix kernel (nb_stream_run) through the C ABI: groups of packed matvecs
against the fp64 oracle (both epilogues, plain / fp32 activations, ragged shapes, 2-, 3- and 4-bit),
replays that must be bit-identical, and the one-launch decode step against the chain of fused
kernels and the reference's own logits."""
import os

import numpy as np
import pytest
import torch

from oracle import nb_oracle as o

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    return torch.device("cuda:0")


def _cu(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("bits,n,k", [(3, 6912, 2560), (3, 2560, 6912), (3, 1000, 640), (3, 24, 128), (2, 2560, 2560), (4, 512, 1280),
                                      (3, 7680, 2560), (3, 320, 384)])
@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float32])
def test_group_of_matvecs_against_oracle(built_lib, bits, n, k, xdt):
    from nativebit_b200 import stream as S
    dev = _dev()
    prog = S.StreamProgram(dev)
    cases = []
    slots = S.n_slots(n, k)
    for j in range(3):
        packed, cb, _ = o.make_packed_linear(n, k, bits, seed=10 * j + bits)
        x = o.make_activation(1, k, seed=j)
        if xdt == torch.float32:
            x = (x.astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)   # not fp16-representable
        w = S.stream_pack(_cu(packed, dev), _cu(cb, dev), bits, n, k)
        xt = _cu(x, dev).to(xdt).reshape(k)
        y_store = torch.full((n,), float("nan"), dtype=torch.float32, device=dev)
        part = torch.full((slots, n), float("nan"), dtype=torch.float32, device=dev)
        y_red = torch.full((n,), float("nan"), dtype=torch.float32, device=dev)
        prog.gemv_vec(w, n, k, bits, xt, y_store)                       # whole row tiles per CTA, final store
        prog.gemv_vec(w, n, k, bits, xt, part, slots=slots, reuse_x=True)   # free split, partial slots
        cases.append((packed, cb, xt, y_store, part, y_red))
    for j, (_, _, _, _, part, y_red) in enumerate(cases):
        prog.reduce(part, n, y_red, wait=(j == 0))
    prog.run()
    torch.cuda.synchronize()
    assert prog.status() == 0
    first = [(c[3].clone(), c[5].clone()) for c in cases]
    for packed, cb, xt, y_store, part, y_red in cases:
        ref = o.packed_linear_forward(xt.double().cpu().numpy().reshape(1, k), packed, cb.astype(np.float32), n, k, bits,
                                      acc_dtype=np.float64)[0]
        scale = np.abs(ref).max()
        assert np.abs(y_store.double().cpu().numpy() - ref).max() <= 2e-5 * scale
        assert np.abs(y_red.double().cpu().numpy() - ref).max() <= 2e-5 * scale
    prog.run()                                                          # replay: same bits
    torch.cuda.synchronize()
    for (a, b), c in zip(first, cases):
        assert torch.equal(a, c[3]) and torch.equal(b, c[5])
    assert prog.status() == 0


def test_chain_of_dependent_matvecs(built_lib):
    """gate_up with the SwiGLU epilogue -> down with partial slots -> reduce, each waiting for the one
    before: the FFN of one layer without norms, against the oracle."""
    from nativebit_b200 import stream as S
    dev = _dev()
    C, F = 640, 1408
    pg, cg, _ = o.make_packed_linear(F, C, 3, seed=1)
    pu, cu_, _ = o.make_packed_linear(F, C, 3, seed=2)
    pd, cd, _ = o.make_packed_linear(C, F, 3, seed=3)
    x = o.make_activation(1, C, seed=4)
    gu_p = torch.cat([_cu(pg, dev), _cu(pu, dev)])
    gu_c = torch.cat([_cu(cg, dev), _cu(cu_, dev)])
    w_gu = S.stream_pack(gu_p, gu_c, 3, 2 * F, C, row_mode=1)
    w_d = S.stream_pack(_cu(pd, dev), _cu(cd, dev), 3, C, F)
    xt = _cu(x, dev).float().reshape(C)
    act = torch.zeros(F, device=dev)
    slots = S.n_slots(C, F)
    part = torch.zeros(slots, C, device=dev)
    y = torch.zeros(C, device=dev)
    prog = S.StreamProgram(dev)
    prog.add(S._op(S.SOP_GEMV, S.SOPF_ALIGN, S.SPRO_VEC, S.SEPI_SWIGLU, p=(w_gu, xt, None, None, act),
                   i=(2 * F, C, 3, S.NB_F32, 0, 0, 0, 0, 0)), w_gu, xt, act)
    prog.gemv_vec(w_d, C, F, 3, act, part, slots=slots, wait=True)
    prog.reduce(part, C, y, wait=True)
    for _ in range(3):
        prog.run()
    torch.cuda.synchronize()
    assert prog.status() == 0
    f32 = np.float32
    g = o.packed_linear_forward(x, pg, cg.astype(f32), F, C, 3, acc_dtype=np.float64)[0]
    u = o.packed_linear_forward(x, pu, cu_.astype(f32), F, C, 3, acc_dtype=np.float64)[0]
    a = g / (1.0 + np.exp(-g)) * u
    assert np.abs(act.double().cpu().numpy() - a).max() <= 2e-5 * np.abs(a).max()
    ref = o.packed_linear_forward(a.reshape(1, F), pd, cd.astype(f32), C, F, 3, acc_dtype=np.float64)[0]
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()


def test_one_launch_decode_step_equals_kernel_chain(built_lib):
    """Tiny seeded model (bf16 embedding table): the decode step as ONE persistent launch gives the tokens
    of the step run as a chain of fused kernels and logits within fp32 rounding of it, eager and from a
    CUDA graph.  (The chain is pinned to the reference's own PackedGPT logits in test_gpu_model.py; the
    full-size model is compared with the dense oracle there, through this one-launch step.)"""
    from nativebit_b200 import generate as G
    from tests.test_gpu_model import _build
    dev = _dev()
    gm = np.load(os.path.join(ROOT, "tests", "golden", "reference_model.npz"))
    model, cfg = _build(gm, dev)
    model.embedding = model.embedding.bfloat16()
    prompt = torch.from_numpy(gm["prompt"]).to(dev)
    for graph in (False, True):
        a = G.DecodeSession(model, 1, use_graph=graph, stream=True)
        b = G.DecodeSession(model, 1, use_graph=False, stream=False)
        a.prefill(prompt); b.prefill(prompt)
        for _ in range(12):
            a.step(); b.step()
            assert torch.equal(a.token, b.token)
            assert (a.logits - b.logits).abs().max() <= 1e-4 * b.logits.abs().max()
        a.check()


def test_matvec_group_api(built_lib):
    """The user-facing group: FFN-shaped matvecs of two layers in one launch, bf16 and fp32 outputs."""
    import nativebit_b200 as nbt
    dev = _dev()
    H, F = 2560, 6912
    x = _cu(o.make_activation(1, H, seed=1), dev).bfloat16()
    h = _cu(o.make_activation(1, F, seed=2), dev).bfloat16()
    items, refs = [], []
    for l in range(2):
        for j, (n, k, src) in enumerate(((F, H, x), (F, H, x), (H, F, h))):
            packed, cb, _ = o.make_packed_linear(n, k, 3, seed=10 * l + j)
            lin = nbt.PackedLinear(_cu(packed, dev), _cu(cb, dev), n, k)
            out = torch.full((1, n), float("nan"), dtype=torch.float32 if j == 2 else torch.bfloat16, device=dev)
            items.append((lin, src, out))
            refs.append(o.packed_linear_forward(src.float().cpu().numpy(), packed, cb.astype(np.float32), n, k, 3, acc_dtype=np.float64)[0])
    grp = nbt.MatvecGroup(items)
    grp.run()
    torch.cuda.synchronize()
    grp.check()
    for (lin, _, out), ref in zip(items, refs):
        tol = 2e-5 if out.dtype == torch.float32 else 2.0 ** -8
        assert np.abs(out.double().cpu().numpy()[0] - ref).max() <= tol * np.abs(ref).max()
        # and equal to the single-matrix kernel's answer up to the output rounding
        y1 = lin(items[0][1] if lin.in_features == H else h)
        assert np.abs(y1.double().cpu().numpy()[0] - ref).max() <= 2.0 ** -8 * np.abs(ref).max()


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_matvec_group_ragged_shapes_and_types(built_lib, bits):
    """One launch over matrices of unlike shapes: rows that do not fill a 16-row tile, one k-block per row (every
    unit is a tile of its own), odd and even numbers of k-blocks, fp32 / fp16 / bf16 activations (fp32 needs both
    fp16 terms), every output type; twice, and the second run must reproduce the first bit for bit."""
    import nativebit_b200 as nbt
    dev = _dev()
    shapes = [(1000, 640, torch.float32, torch.float32), (24, 128, torch.bfloat16, torch.float32), (320, 384, torch.float16, torch.bfloat16),
              (2560, 2560, torch.bfloat16, torch.float16), (17, 1280, torch.float32, torch.float32), (4096, 128, torch.bfloat16, torch.float32)]
    items, refs, shared = [], [], {}
    for j, (n, k, xdt, ydt) in enumerate(shapes):
        packed, cb, _ = o.make_packed_linear(n, k, bits, seed=20 + j)
        x = o.make_activation(1, k, seed=j)
        if xdt == torch.float32:
            x = (x.astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)
        xt = shared.setdefault((k, xdt), _cu(x, dev).to(xdt))           # matrices of one width share the vector
        lin = nbt.PackedLinear(_cu(packed, dev), _cu(cb, dev), n, k, bits=bits)
        out = torch.full((n,), float("nan"), dtype=ydt, device=dev)
        items.append((lin, xt.reshape(k), out))
        refs.append(o.packed_linear_forward(xt.double().cpu().numpy().reshape(1, k), packed, cb.astype(np.float32), n, k, bits,
                                            acc_dtype=np.float64)[0])
    grp = nbt.MatvecGroup(items)
    grp.run()
    torch.cuda.synchronize()
    first = [out.clone() for _, _, out in items]
    for (_, _, out), ref in zip(items, refs):
        tol = {torch.float32: 2e-5, torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[out.dtype]
        assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    for _, _, out in items:
        out.fill_(float("nan"))
    grp.run()
    torch.cuda.synchronize()
    for (_, _, out), f in zip(items, first):
        assert torch.equal(out, f)


def test_matvec_group_refuses_what_it_cannot_run(built_lib):
    import nativebit_b200 as nbt
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(64, 256, 3, seed=1)
    lin = nbt.PackedLinear(_cu(packed, dev), _cu(cb, dev), 64, 256)
    xs = [torch.zeros(256, dtype=torch.float32, device=dev) for _ in range(7)]
    out = torch.zeros(64, dtype=torch.float32, device=dev)
    with pytest.raises(RuntimeError):
        nbt.MatvecGroup([(lin, x, out) for x in xs])                    # seven distinct activation vectors
    with pytest.raises(RuntimeError):
        nbt.MatvecGroup([(lin, torch.zeros(128, device=dev), out)])     # wrong length


@pytest.mark.parametrize("bits,m", [(3, 2), (3, 4), (3, 8), (2, 5), (4, 3)])
def test_matvec_group_with_several_activation_rows(built_lib, bits, m):
    """Up to eight activation rows per matrix ride in the eight columns of the MMA: FFN-shaped matrices against (m, k)
    activations, against the fp64 oracle; twice, bit-identical.  The 3-bit case at 4 rows needs the shorter copy rings."""
    import nativebit_b200 as nbt
    dev = _dev()
    H, F = 2560, 6912
    # the staged activations must fit the kernel's shared memory: 6912-wide rows only up to four of them
    shapes = [(1000, H), (320, 1280)] if bits == 4 else [(F, H), (1000, H)] + ([(H, F)] if m <= 4 else [(640, 1280)])
    xs = {}
    items, refs = [], []
    for j, (n, k) in enumerate(shapes):
        packed, cb, _ = o.make_packed_linear(n, k, bits, seed=40 + j)
        if k not in xs:
            x = o.make_activation(m, k, seed=100 + k)
            xs[k] = (x, _cu(x, dev).to(torch.bfloat16 if j % 2 == 0 else torch.float16))
        x, xt = xs[k]
        lin = nbt.PackedLinear(_cu(packed, dev), _cu(cb, dev), n, k, bits=bits)
        out = torch.full((m, n), float("nan"), dtype=torch.float32 if j != 1 else torch.bfloat16, device=dev)
        items.append((lin, xt, out))
        refs.append(o.packed_linear_forward(xt.double().cpu().numpy(), packed, cb.astype(np.float32), n, k, bits, acc_dtype=np.float64))
    grp = nbt.MatvecGroup(items)
    grp.run()
    torch.cuda.synchronize()
    first = [out.clone() for _, _, out in items]
    for (_, _, out), ref in zip(items, refs):
        tol = 2e-5 if out.dtype == torch.float32 else 2.0 ** -8
        assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    for _, _, out in items:
        out.fill_(float("nan"))
    grp.run()
    torch.cuda.synchronize()
    for (_, _, out), f in zip(items, first):
        assert torch.equal(out, f)


def test_matvec_group_refuses_rows_it_cannot_stage(built_lib):
    import nativebit_b200 as nbt
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(64, 6912, 3, seed=1)
    lin = nbt.PackedLinear(_cu(packed, dev), _cu(cb, dev), 64, 6912)
    with pytest.raises(RuntimeError):                                   # 8 rows of 6912 activations: 138 KB of shared memory
        nbt.MatvecGroup([(lin, torch.zeros(8, 6912, dtype=torch.bfloat16, device=dev), torch.zeros(8, 64, device=dev))])
    with pytest.raises(RuntimeError):                                   # several rows need 16-bit activations
        nbt.MatvecGroup([(lin, torch.zeros(2, 6912, dtype=torch.float32, device=dev), torch.zeros(2, 64, device=dev))])
    with pytest.raises(RuntimeError):                                   # nine rows
        nbt.MatvecGroup([(lin, torch.zeros(9, 6912, dtype=torch.bfloat16, device=dev), torch.zeros(9, 64, device=dev))])


@pytest.mark.parametrize("bits,n,k", [(3, 7680, 2560), (3, 2560, 6912), (3, 1000, 640), (3, 24, 128), (2, 2560, 2560), (4, 512, 1280),
                                      (3, 13824, 2560), (3, 320, 384), (3, 40, 7168)])
def test_chain_gemv_over_the_stream_layout(built_lib, bits, n, k):
    """nb_gemv_stream, the decode step's matvec: plain activations of every type, residual add + RMSNorm in front
    (with the updated residual written out), SwiGLU in front; against the fp64 oracle, and twice bit-identical."""
    from nativebit_b200 import ops, stream as S
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=n % 97 + bits)
    w = S.stream_pack(_cu(packed, dev), _cu(cb, dev), bits, n, k)
    cbf = cb.astype(np.float32)
    rng = np.random.default_rng(n + k)

    def check(y, act):
        ref = o.packed_linear_forward(act.reshape(1, k), packed, cbf, n, k, bits, acc_dtype=np.float64)[0]
        assert np.abs(y.double().cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()

    for xdt in (torch.float32, torch.bfloat16, torch.float16):
        x = o.make_activation(1, k, seed=3)[0]
        if xdt == torch.float32:
            x = (x.astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)
        xt = _cu(x, dev).to(xdt)
        y = torch.full((n,), float("nan"), device=dev)
        ops.gemv_stream(ops.PRO_NONE, xt, w, bits, n, k, y)
        y2 = torch.full((n,), float("nan"), device=dev)
        ops.gemv_stream(ops.PRO_NONE, xt, w, bits, n, k, y2)
        torch.cuda.synchronize()
        check(y, xt.double().cpu().numpy())
        assert torch.equal(y, y2)
    # y += W x: the residual update inside the matvec
    x32 = rng.standard_normal(k).astype(np.float32)
    y0 = rng.standard_normal(n).astype(np.float32)
    yacc = _cu(y0, dev).clone()
    ops.gemv_stream(ops.PRO_NONE, _cu(x32, dev), w, bits, n, k, yacc, accumulate=True)
    yplain = torch.empty(n, device=dev)
    ops.gemv_stream(ops.PRO_NONE, _cu(x32, dev), w, bits, n, k, yplain)
    torch.cuda.synchronize()
    assert torch.equal(yacc, yplain + _cu(y0, dev))
    # residual add + RMSNorm
    h = rng.standard_normal(k).astype(np.float32)
    d = rng.standard_normal(k).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    for delta in (d, None):
        v = h.astype(np.float64) + (0 if delta is None else delta.astype(np.float64))
        act = v / np.sqrt((v * v).mean() + 1e-6) * g
        y = torch.full((n,), float("nan"), device=dev)
        x_out = torch.full((k,), float("nan"), device=dev)
        ops.gemv_stream(ops.PRO_ADD_RMSNORM, _cu(h, dev), w, bits, n, k, y, delta=None if delta is None else _cu(delta, dev),
                        norm_weight=_cu(g, dev), eps=1e-6, x_out=x_out)
        torch.cuda.synchronize()
        check(y, act)
        # the one-term option: activations rounded to fp16 once (11 bits), the same sums otherwise
        y1 = torch.full((n,), float("nan"), device=dev)
        ops.gemv_stream(ops.PRO_ADD_RMSNORM, _cu(h, dev), w, bits, n, k, y1, delta=None if delta is None else _cu(delta, dev),
                        norm_weight=_cu(g, dev), eps=1e-6, single_term=True)
        # (the kernel rounds (x + delta) * weight, computed in fp32, and applies the norm's scale to the sums)
        staged = (((h + delta) if delta is not None else h) * g).astype(np.float16).astype(np.float64)
        ref1 = o.packed_linear_forward(staged.reshape(1, k), packed, cbf, n, k, bits, acc_dtype=np.float64)[0] / np.sqrt((v * v).mean() + 1e-6)
        assert np.abs(y1.double().cpu().numpy() - ref1).max() <= 5e-5 * np.abs(ref1).max()
        assert np.abs(y1.double().cpu().numpy() - y.double().cpu().numpy()).max() <= 2e-3 * np.abs(ref1).max()
        assert np.array_equal(x_out.cpu().numpy(), (h + delta).astype(np.float32) if delta is not None else h)
    # SwiGLU
    gu = rng.standard_normal(2 * k).astype(np.float32)
    gate, up = gu[:k].astype(np.float64), gu[k:].astype(np.float64)
    y = torch.full((n,), float("nan"), device=dev)
    ops.gemv_stream(ops.PRO_SILU_MUL, _cu(gu, dev), w, bits, n, k, y)
    torch.cuda.synchronize()
    ref = o.packed_linear_forward((gate / (1 + np.exp(-gate)) * up).reshape(1, k), packed, cbf, n, k, bits, acc_dtype=np.float64)[0]
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 5e-5 * np.abs(ref).max()     # __expf in the activation


def test_decode_step_on_the_stream_layout_equals_the_workspace_kernels(built_lib):
    """The decode session with its packed linears on nb_gemv_stream against the same session on nb_gemv_fused:
    identical greedy tokens, logits within fp32 summation-order differences."""
    from nativebit_b200 import generate as G
    dev = _dev()
    cfg = G.ModelConfig(vocab_size=512, n_layers=3, n_embd=512, n_head=4, ffn_hidden=1408, context_len=64)
    model = G.PackedGPT.random_init(cfg, seed=5, device=dev)
    prompt = torch.randint(0, cfg.vocab_size, (1, 7), generator=torch.Generator().manual_seed(1)).to(dev)
    a = G.DecodeSession(model, 1, use_graph=False, tile_gemv=True)
    b = G.DecodeSession(model, 1, use_graph=False, tile_gemv=False)
    assert a.tile_gemv and not b.tile_gemv
    a.prefill(prompt); b.prefill(prompt)
    for _ in range(12):
        a.step(); b.step()
        assert torch.equal(a.token, b.token)
        assert (a.logits - b.logits).abs().max() <= 1e-4 * b.logits.abs().max()
    g = G.DecodeSession(model, 1, use_graph=True, tile_gemv=True)
    toks_g = g.generate(prompt, 12)
    toks_e = G.DecodeSession(model, 1, use_graph=False, tile_gemv=True).generate(prompt, 12)
    assert torch.equal(toks_g, toks_e)


@pytest.mark.parametrize("B", [2, 5, 8])
def test_batched_decode_step_on_the_rows_kernel_equals_the_workspace_kernels(built_lib, B):
    """A session of 2 .. 8 sequences with its packed linears on nb_gemv_stream_rows against the same session on
    nb_gemv_fused: identical greedy tokens for different prompts per sequence, logits within summation-order
    differences; graph replay equals the eager loop."""
    from nativebit_b200 import generate as G
    dev = _dev()
    cfg = G.ModelConfig(vocab_size=512, n_layers=3, n_embd=512, n_head=4, ffn_hidden=1408, context_len=64)
    model = G.PackedGPT.random_init(cfg, seed=5, device=dev)
    prompt = torch.randint(0, cfg.vocab_size, (B, 7), generator=torch.Generator().manual_seed(B)).to(dev)
    a = G.DecodeSession(model, B, use_graph=False)
    b = G.DecodeSession(model, B, use_graph=False, tile_gemv=False)
    assert a.tile_rows and not b.tile_rows
    a.prefill(prompt); b.prefill(prompt)
    for _ in range(10):
        a.step(); b.step()
        assert torch.equal(a.token, b.token)
        assert (a.logits - b.logits).abs().max() <= 1e-4 * b.logits.abs().max()
    toks_g = G.DecodeSession(model, B, use_graph=True).generate(prompt, 10)
    toks_e = G.DecodeSession(model, B, use_graph=False).generate(prompt, 10)
    assert torch.equal(toks_g, toks_e)


@pytest.mark.parametrize("bits,n,k,m", [(3, 7680, 2560, 8), (3, 2560, 6912, 3), (3, 13824, 2560, 5), (3, 1000, 640, 2), (2, 2560, 2560, 7),
                                        (4, 512, 1280, 4), (3, 320, 384, 8), (3, 40, 7168, 1), (3, 2560, 6912, 8)])
def test_chain_gemv_rows(built_lib, bits, n, k, m):
    """nb_gemv_stream_rows: a few fp32 activation rows in one pass over the weights (more rows than fit one launch are
    split by the wrapper), plain / residual add + RMSNorm / SwiGLU in front; against the fp64 oracle row by row, twice
    bit-identical, and nothing written outside the m rows."""
    from nativebit_b200 import ops, stream as S
    dev = _dev()
    assert ops.gemv_stream_max_rows(3, 2560) == 8 and ops.gemv_stream_max_rows(3, 6912) == 3
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=n % 97 + bits)
    w = S.stream_pack(_cu(packed, dev), _cu(cb, dev), bits, n, k)
    cbf = cb.astype(np.float32)
    rng = np.random.default_rng(n + k + m)

    def check(y, act, tol=2e-5):
        ref = o.packed_linear_forward(act, packed, cbf, n, k, bits, acc_dtype=np.float64)
        got = y.double().cpu().numpy()
        for r in range(m):
            assert np.abs(got[r] - ref[r]).max() <= tol * np.abs(ref[r]).max(), r

    x = (rng.standard_normal((m, k)) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)
    y = torch.full((m + 1, n), float("nan"), device=dev)
    y2 = torch.full((m, n), float("nan"), device=dev)
    ops.gemv_stream_rows(ops.PRO_NONE, _cu(x, dev), w, bits, n, k, y[:m])
    ops.gemv_stream_rows(ops.PRO_NONE, _cu(x, dev), w, bits, n, k, y2)
    torch.cuda.synchronize()
    check(y[:m], x.astype(np.float64))
    assert torch.equal(y[:m], y2) and bool(torch.isnan(y[m]).all())
    # residual add + RMSNorm, every row with its own scale
    h = (rng.standard_normal((m, k)) * (1.0 + np.arange(m))[:, None]).astype(np.float32)
    d = rng.standard_normal((m, k)).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    for delta in (d, None):
        v = h.astype(np.float64) + (0 if delta is None else delta.astype(np.float64))
        act = v / np.sqrt((v * v).mean(axis=1, keepdims=True) + 1e-6) * g
        y = torch.full((m, n), float("nan"), device=dev)
        x_out = torch.full((m, k), float("nan"), device=dev)
        ops.gemv_stream_rows(ops.PRO_ADD_RMSNORM, _cu(h, dev), w, bits, n, k, y, delta=None if delta is None else _cu(delta, dev),
                             norm_weight=_cu(g, dev), eps=1e-6, x_out=x_out)
        torch.cuda.synchronize()
        check(y, act)
        assert np.array_equal(x_out.cpu().numpy(), (h + delta).astype(np.float32) if delta is not None else h)
    # SwiGLU
    gu = rng.standard_normal((m, 2 * k)).astype(np.float32)
    gate, up = gu[:, :k].astype(np.float64), gu[:, k:].astype(np.float64)
    y = torch.full((m, n), float("nan"), device=dev)
    ops.gemv_stream_rows(ops.PRO_SILU_MUL, _cu(gu, dev), w, bits, n, k, y)
    torch.cuda.synchronize()
    check(y, gate / (1 + np.exp(-gate)) * up, tol=5e-5)                 # __expf in the activation


@pytest.mark.parametrize("bits,f,k", [(3, 6912, 2560), (3, 704, 640), (2, 1408, 1280)])
def test_chain_gemv_swiglu_epilogue(built_lib, bits, f, k):
    """A fused [gate | up] matrix packed with 8 gate and the 8 matching up channels per tile: the matvec's epilogue
    writes silu(gate) * up, with the residual add + RMSNorm in front as in the decoder."""
    from nativebit_b200 import ops, stream as S
    dev = _dev()
    n = 2 * f
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=f % 89)
    w = S.stream_pack(_cu(packed, dev), _cu(cb, dev), bits, n, k, row_mode=1)
    rng = np.random.default_rng(f)
    h = rng.standard_normal(k).astype(np.float32)
    d = rng.standard_normal(k).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    v = h.astype(np.float64) + d.astype(np.float64)
    act = v / np.sqrt((v * v).mean() + 1e-6) * g
    gu = o.packed_linear_forward(act.reshape(1, k), packed, cb.astype(np.float32), n, k, bits, acc_dtype=np.float64)[0]
    ref = gu[:f] / (1 + np.exp(-gu[:f])) * gu[f:]
    y = torch.full((f,), float("nan"), device=dev)
    ops.gemv_stream(ops.PRO_ADD_RMSNORM, _cu(h, dev), w, bits, n, k, y, delta=_cu(d, dev), norm_weight=_cu(g, dev), eps=1e-6,
                    x_out=torch.empty(k, device=dev), swiglu=True)
    torch.cuda.synchronize()
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 5e-5 * np.abs(ref).max()
    # the same epilogue for five rows in one pass over the weights
    m = 5
    hm = rng.standard_normal((m, k)).astype(np.float32)
    dm = rng.standard_normal((m, k)).astype(np.float32)
    vm = hm.astype(np.float64) + dm.astype(np.float64)
    actm = vm / np.sqrt((vm * vm).mean(axis=1, keepdims=True) + 1e-6) * g
    gum = o.packed_linear_forward(actm, packed, cb.astype(np.float32), n, k, bits, acc_dtype=np.float64)
    refm = gum[:, :f] / (1 + np.exp(-gum[:, :f])) * gum[:, f:]
    ym = torch.full((m, f), float("nan"), device=dev)
    ops.gemv_stream_rows(ops.PRO_ADD_RMSNORM, _cu(hm, dev), w, bits, n, k, ym, delta=_cu(dm, dev), norm_weight=_cu(g, dev), eps=1e-6,
                         x_out=torch.empty(m, k, device=dev), swiglu=True)
    torch.cuda.synchronize()
    got = ym.double().cpu().numpy()
    for r in range(m):
        assert np.abs(got[r] - refm[r]).max() <= 5e-5 * np.abs(refm[r]).max(), r

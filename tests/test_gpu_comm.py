"""One-shot all-reduce kernel on a single GPU: the world-size-1 case (a rank pushing to itself must
return its input bit for bit, over many calls, alternating buffer sets) and the bounded wait (a
peer that never raises its flag makes the kernel give up with NB_ERR_TIMEOUT instead of hanging;
the context stays usable).  The multi-rank path runs in bench.py --gpus N."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, max_count, dev):
    from nativebit_b200 import _lib
    l = _lib.lib()
    nbytes = l.nb_allreduce_buffer_bytes(world, max_count)
    assert nbytes > 0
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    arr = (ctypes.c_uint64 * world)(*[b.data_ptr() for b in bufs])
    return l, bufs, arr


def test_single_rank_is_identity_over_many_calls(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    l, bufs, arr = _setup(1, 4096, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    for call, n in enumerate([2560, 4096, 4, 1000, 2560, 2560]):
        x = torch.randn(n, device=dev)
        y = torch.empty_like(x)
        assert l.nb_allreduce(x.data_ptr(), y.data_ptr(), n, arr, 1, 0, 4096, 0, status.data_ptr(), st) == 0
        z = x.clone()
        assert l.nb_allreduce(z.data_ptr(), z.data_ptr(), n, arr, 1, 0, 4096, 0, status.data_ptr(), st) == 0   # in place
        torch.cuda.synchronize()
        assert torch.equal(y, x) and torch.equal(z, x), call
    assert int(status.item()) == 0


def test_missing_peer_times_out_without_hanging(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    l, bufs, arr = _setup(2, 1024, dev)          # "rank 1" is a second local buffer that nobody drives
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    x = torch.ones(1024, device=dev)
    y = torch.empty_like(x)
    rc = l.nb_allreduce(x.data_ptr(), y.data_ptr(), 1024, arr, 2, 0, 1024, 2000, status.data_ptr(),
                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()                      # returns promptly: the wait is bounded
    assert int(status.item()) == 6                # NB_ERR_TIMEOUT
    assert torch.isfinite(y).all()
    # the context is still healthy
    assert float((x + 1).sum()) == 2048.0


def test_argument_checks(built_lib):
    from nativebit_b200 import _lib
    l = _lib.lib()
    assert l.nb_allreduce_buffer_bytes(9, 1024) == 0 and l.nb_allreduce_buffer_bytes(2, 1022) == 0
    fake = ctypes.c_void_p(4096)
    arr = (ctypes.c_uint64 * 2)(4096, 8192)
    assert l.nb_allreduce(fake, fake, 6, arr, 2, 0, 1024, 0, None, None) == 3      # count % 4
    assert l.nb_allreduce(fake, fake, 2048, arr, 2, 0, 1024, 0, None, None) == 3   # count > max_count
    assert l.nb_allreduce(fake, fake, 8, arr, 2, 2, 1024, 0, None, None) == 1      # rank out of range


# ------------------------------------------------------------------ all-reduce folded into the GEMVs (nb_gemv_tp)
def _exchange(world, max_count, dev, spin_limit=0):
    from nativebit_b200.comm import Exchange
    nbytes = Exchange.buffer_bytes(world, max_count)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    return [Exchange(max_count, dev, rank=r, local_buffers=bufs, spin_limit=spin_limit) for r in range(world)]


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("m", [1, 3])
def test_row_parallel_push_then_gather_equals_unsharded(built_lib, world, m):
    """The ranks of a row-sharded projection run one after another on this GPU, each pushing into all
    (local) exchange buffers; then every rank's next GEMV gathers.  Nothing waits at run time: all
    flags are raised before the consumers start.  Three rounds exercise both buffer sets."""
    import numpy as np
    from oracle import nb_oracle as o
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    C, Fh, N2 = 512, 1024, 384                       # hidden, row-sharded K, next layer's rows
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    p_down, c_down, _ = o.make_packed_linear(C, Fh, 3, 5)          # (C, Fh): K is sharded
    p_next, c_next, _ = o.make_packed_linear(N2, C, 3, 6)
    kb = Fh // 128 // world                                         # k-blocks per rank
    rows_p = p_down.reshape(C, Fh // 128, 48)
    rows_c = c_down.reshape(C, Fh // 128, 8)
    shards = [(cu(rows_p[:, r * kb:(r + 1) * kb].reshape(-1)), cu(rows_c[:, r * kb:(r + 1) * kb].reshape(-1, 8))) for r in range(world)]
    xs = _exchange(world, 8 * C, dev)
    w = cu((1.0 + 0.1 * np.random.default_rng(1).standard_normal(C)).astype(np.float32))
    pn, cn = cu(p_next), cu(c_next)
    for rnd in range(3):
        rng = np.random.default_rng(10 + rnd)
        gu = rng.standard_normal((m, 2 * Fh)).astype(np.float32)    # [gate | up] of the full FFN width
        h = rng.standard_normal((m, C)).astype(np.float32)
        g, u = gu[:, :Fh].astype(np.float64), gu[:, Fh:].astype(np.float64)
        act = g / (1 + np.exp(-g)) * u
        d = o.packed_linear_forward(act, p_down, c_down.astype(np.float32), C, Fh, 3, acc_dtype=np.float64)
        v = h + d
        ref = o.packed_linear_forward(v / np.sqrt((v * v).mean(1, keepdims=True) + 1e-6) * w.cpu().numpy().astype(np.float64),
                                      p_next, c_next.astype(np.float32), N2, C, 3, acc_dtype=np.float64)
        for r in range(world):                                      # producers: SwiGLU prologue + push
            cols = slice(r * kb * 128, (r + 1) * kb * 128)
            gu_r = cu(np.concatenate([gu[:, :Fh][:, cols], gu[:, Fh:][:, cols]], axis=1))
            ops.gemv_tp(ops.PRO_SILU_MUL, gu_r, *shards[r], 3, 128, C, kb * 128, xs[r], push=True)
        ys, hs = [], []
        for r in range(world):                                      # consumers: gather + add + RMSNorm + GEMV
            y = torch.empty(m, N2, device=dev)
            h_out = torch.empty(m, C, device=dev)
            ops.gemv_tp(ops.PRO_ADD_RMSNORM, cu(h), pn, cn, 3, 128, N2, C, xs[r], out=y, gather=True, norm_weight=w, eps=1e-6,
                        x_out=h_out)
            ys.append(y); hs.append(h_out)
        torch.cuda.synchronize()
        assert all(torch.equal(ys[0], y) for y in ys) and all(torch.equal(hs[0], x) for x in hs)   # same bits on every rank
        assert np.abs(hs[0].double().cpu().numpy() - v).max() <= 1e-5 * np.abs(v).max()
        assert np.abs(ys[0].double().cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()
    # standalone gather of a pushed vector (the step's last all-reduce)
    x = torch.randn(m, C, device=dev)
    p_id, c_id, _ = o.make_packed_linear(C, C, 3, 7)
    for r in range(world):
        ops.gemv_tp(ops.PRO_NONE, x, cu(p_id), cu(c_id), 3, 128, C, C, xs[r], push=True)
    one = ops.gemv(x, cu(p_id), cu(c_id), 3, 128, C, C)
    out = torch.empty(m, C, device=dev)
    ops.exchange_gather(out, xs[0], xs[0].status)
    torch.cuda.synchronize()
    assert torch.allclose(out, world * one, rtol=1e-5, atol=1e-6)
    ws = ops.workspace(dev, 0)
    assert ops.workspace_status(ws) == 0 and int(xs[0].status.item()) == 0


def test_gather_without_the_peers_push_times_out(built_lib):
    """Rank 0 pushed, "rank 1" never did: the consumer's bounded wait runs out, the status word says so,
    and the context stays usable."""
    import numpy as np
    from oracle import nb_oracle as o
    from nativebit_b200 import ops
    dev = torch.device("cuda:0")
    xs = _exchange(2, 1024, dev, spin_limit=500)
    p, c, _ = o.make_packed_linear(256, 256, 3, 1)
    pc, cc = torch.from_numpy(p).to(dev), torch.from_numpy(c).to(dev)
    x = torch.randn(1, 256, device=dev)
    ops.gemv_tp(ops.PRO_NONE, x, pc, cc, 3, 128, 256, 256, xs[0], push=True)
    y = torch.empty(1, 256, device=dev)
    ops.gemv_tp(ops.PRO_ADD_RMSNORM, x, pc, cc, 3, 128, 256, 256, xs[0], out=y, gather=True,
                norm_weight=torch.ones(256, device=dev), eps=1e-6, x_out=torch.empty_like(x))
    torch.cuda.synchronize()                          # returns promptly
    ws = ops.workspace(dev, 0)
    assert ops.workspace_status(ws) == 6              # NB_ERR_TIMEOUT
    ws[4095 * 4:4096 * 4].zero_()
    out = torch.empty(1, 256, device=dev)
    ops.exchange_gather(out, xs[0], xs[0].status)
    torch.cuda.synchronize()
    assert int(xs[0].status.item()) == 6
    assert float((x * 0 + 1).sum()) == 256.0          # the context is healthy

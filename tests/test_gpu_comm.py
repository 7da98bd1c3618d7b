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

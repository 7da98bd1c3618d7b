"""nb_gemv_static: the GEMV entry point for callers that cannot allocate device memory (a plugin
given only input and output buffers, code under a frozen memory budget).  Its split-K scratch is
a fixed array inside the library, so the test calls it through the C ABI with nothing but x,
weights and y, twice in a row, and compares with nb_gemv run on an ordinary workspace.

This file is collected last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import nb_oracle as o

pytestmark = pytest.mark.gpu
NB_F16, NB_BF16, NB_F32 = 1, 2, 0


def _cu(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("n,k,m", [(2560, 6912, 16), (2560, 6912, 1), (6912, 2560, 1), (1000, 640, 3)])
def test_static_scratch_matches_workspace_entry_point(built_lib, n, k, m):
    from nativebit_b200 import _lib, ops
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    l = _lib.lib()
    packed, cb, _ = o.make_packed_linear(n, k, 3, seed=n + m)
    p, c = _cu(packed, dev), _cu(cb, dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                       # the second call finds the first call's leftovers in the array
        x = _cu(o.make_activation(m, k, seed=call), dev).bfloat16()
        ref = ops.gemv(x, p, c, 3, 128, n, k, out_dtype=torch.float32)
        y = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
        rc = l.nb_gemv_static(x.data_ptr(), NB_BF16, m, p.data_ptr(), c.data_ptr(), NB_F16, 3, 128, n, k,
                              y.data_ptr(), NB_F32, stream)
        assert rc == 0, l.nb_status_string(rc)
        torch.cuda.synchronize()
        # same plan, same fixed summation order: the tolerance of the GEMV tests (2e-5 of max|y|)
        # is met with room to spare; in practice the two results are identical
        assert (y - ref).abs().max() <= 2e-5 * ref.abs().max()
        oracle = o.packed_linear_forward(x.float().cpu().numpy(), packed, cb.astype(np.float32), n, k, 3,
                                         acc_dtype=np.float64)
        assert np.abs(y.cpu().numpy() - oracle).max() <= 2e-5 * np.abs(oracle).max()
    word = ctypes.c_int(-1)
    assert l.nb_gemv_static_status(ctypes.byref(word), 0) == 0 and word.value == 0   # no bounded wait ran out


def test_static_scratch_refuses_oversized_shapes(built_lib):
    from nativebit_b200 import _lib
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    l = _lib.lib()
    m, n, k = 16, 262144, 8192                 # needs more than the 4 MiB the library carries
    assert l.nb_gemv_workspace_bytes(m, n, k, 3, 128) > (4 << 20)
    dummy = torch.zeros(64, dtype=torch.uint8, device=dev)   # never dereferenced: the call is refused first
    rc = l.nb_gemv_static(dummy.data_ptr(), NB_BF16, m, dummy.data_ptr(), dummy.data_ptr(), NB_F16, 3, 128, n, k,
                          dummy.data_ptr(), NB_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == 7                             # NB_ERR_WORKSPACE
    assert b"built-in array" in l.nb_last_cuda_error()
